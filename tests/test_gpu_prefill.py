"""CUDA prefill MoE (sorted tokens, tcgen05 grouped GEMM) against the decode path and the oracle, through the C ABI."""
import numpy as np
import pytest

from ijah_b200 import packgen
from oracle import c_oracle as CO
from tests.helpers import rel_max

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    import torch
    assert torch.cuda.is_available()
    from ijah_b200 import engine as E
    return E.Engine()


def test_prefill_matches_oracle_small(eng):
    # 37 tokens, 32 experts top-4: some experts empty, some with several rows, ragged 8-row padding everywhere
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(21)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    x = rng.standard_normal((37, 512)).astype(np.float16).astype(np.float32)
    blk = E.MoeBlock(eng, t, top_k=4, max_rows=16)
    y = blk.prefill(torch.from_numpy(x).cuda()).cpu().numpy()
    assert eng.lib.ne_device_wait_status() == 0
    want = CO.moe_block_emul(t, x, top_k=4)
    assert rel_max(y, want["out"]) < 2e-4
    y2 = blk.prefill(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(y, y2), "two runs must be bit-identical"


def test_prefill_equals_decode_path_with_skewed_routing(eng):
    # 300 tokens whose routing is skewed so that one expert gets more than 128 rows (several passes) and many get none;
    # the decode-width kernels (16 rows per call) are the reference here
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(22)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    pre = "language_model.model.layers.0.mlp."
    x = rng.standard_normal((300, 512)).astype(np.float16).astype(np.float32)
    # bias the router: add a common direction to x and to the rows of a few experts
    d = rng.standard_normal(512).astype(np.float32)
    x = (x + 1.5 * d).astype(np.float16).astype(np.float32)
    from oracle import opref_port as O
    w = O.bf16_bits_to_f32(t[pre + "gate.weight"][1]).copy()
    w[:3] += 0.02 * d
    t[pre + "gate.weight"] = ("BF16", O.f32_to_bf16_bits(w))
    blk = E.MoeBlock(eng, t, top_k=4, max_rows=16)
    xd = torch.from_numpy(x).cuda()
    y = blk.prefill(xd).cpu().numpy()
    assert eng.lib.ne_device_wait_status() == 0
    ref = np.concatenate([blk.forward(xd[i:i + 16]).cpu().numpy() for i in range(0, 300, 16)])
    assert rel_max(y, ref) < 2e-4  # fp32 accumulation order differs (tcgen05 vs mma.sync + k-splits)
    ids = np.concatenate([CO.moe_block_emul(t, x[i:i + 1], top_k=4)["ids"] for i in range(0, 300, 37)])
    assert ids.shape[1] == 4


def test_prefill_at_model_dims(eng):
    # hidden 2048, intermediate 768, K5 / K6, top-10 of 64 experts, 200 tokens; decode path as the reference
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(23)
    t = packgen.moe_layer(rng, hidden=2048, inter=768, experts=64)
    x = rng.standard_normal((200, 2048)).astype(np.float16).astype(np.float32)
    blk = E.MoeBlock(eng, t, top_k=10, max_rows=16)
    xd = torch.from_numpy(x).cuda()
    y = blk.prefill(xd).cpu().numpy()
    assert eng.lib.ne_device_wait_status() == 0
    ref = np.concatenate([blk.forward(xd[i:i + 16]).cpu().numpy() for i in range(0, 200, 16)])
    assert rel_max(y, ref) < 2e-4  # fp32 accumulation order differs (tcgen05 vs mma.sync + k-splits)
    want = CO.moe_block_emul(t, x[:3], top_k=10)
    assert rel_max(y[:3], want["out"]) < 2e-4


@pytest.mark.parametrize("n_in,n_out,K,rows", [(512, 256, 6, 77), (2048, 512, 8, 300), (256, 768, 4, 129)])
def test_trunk_linear_prefill_matches_oracle_and_decode_path(eng, n_in, n_out, K, rows):
    # one EXL3 Linear over many rows through the grouped tensor-core GEMM: ragged last pass, several 128-row passes
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(n_in + rows)
    tr, suh, svh = packgen.exl3_linear(rng, n_in, n_out, K)
    lin = E.Exl3Linear(eng, tr, suh, svh)
    x = rng.standard_normal((rows, n_in)).astype(np.float16).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    y = lin.prefill(xd).cpu().numpy()
    assert eng.lib.ne_device_wait_status() == 0
    want = np.concatenate([CO.linear_emul(tr, suh, svh, x[i:i + 64]) for i in range(0, rows, 64)])  # the oracle takes <= 64 rows
    assert np.linalg.norm(y - want) / np.linalg.norm(want) < 5e-5
    ref = np.concatenate([lin(xd[i:i + 64]).cpu().numpy() for i in range(0, rows, 64)])
    assert rel_max(y, ref) < 2e-4
    assert np.array_equal(y, lin.prefill(xd).cpu().numpy()), "two runs must be bit-identical"


def test_trunk_linear_prefill_rejects_unsupported_dims(eng):
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(3)
    tr, suh, svh = packgen.exl3_linear(rng, 256, 128, 4)
    lin = E.Exl3Linear(eng, tr, suh, svh)
    with pytest.raises(E.EngineError):
        lin.prefill(torch.zeros((70, 256), device="cuda"))


def test_prefill_ep_summands_add_up_to_the_block(eng):
    # three expert-parallel "ranks" as three objects on one GPU: tokens of all ranks in, each returns its summand
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(31)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=48)
    x = rng.standard_normal((150, 512)).astype(np.float16).astype(np.float32)
    x_all = torch.from_numpy(x).cuda()
    full = E.MoeBlock(eng, t, top_k=4, max_rows=8).prefill(x_all).cpu().numpy()
    total = np.zeros_like(full)
    for r in range(3):
        blk = E.MoeBlock(eng, t, top_k=4, max_rows=8, expert_first=16 * r, expert_count=16)
        part = blk.prefill_ep(x_all, 50 * r, 50).cpu().numpy()
        assert eng.lib.ne_device_wait_status() == 0
        for i in (0, 64, 128):
            want = CO.moe_block_emul(t, x[i:i + 22], top_k=4, expert_range=(16 * r, 16 * r + 16),
                                     shared_rows=(max(50 * r - i, 0), max(min(50 * r + 50, i + 22) - max(50 * r, i), 0)))["out"]
            assert rel_max(part[i:i + 22], want) < 2e-4
        total += part
    assert rel_max(total, full) < 1e-5
    with pytest.raises(E.EngineError):  # the single-GPU entry point refuses an object that holds a slice
        blk.prefill(x_all)


def test_prefill_all_to_all_pieces_reproduce_the_block_bit_for_bit(eng):
    # the all-to-all expert-parallel prefill with its three "ranks" as three objects on one GPU and the two exchanges done
    # by indexing: routing + shared expert at home, every (token, slot) pair through the object that owns its expert, slots
    # added in slot order
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(32)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=48)
    k = 4
    x = torch.from_numpy(rng.standard_normal((300, 512)).astype(np.float16).astype(np.float32)).cuda()
    full = E.MoeBlock(eng, t, top_k=k, max_rows=8)
    want = full.prefill(x)
    ids_full = full.buffer("prefill_route", np.uint32).reshape(300, 2 * k)
    blks = [E.MoeBlock(eng, t, top_k=k, max_rows=8, expert_first=16 * r, expert_count=16) for r in range(3)]
    y_sh, route = blks[1].prefill_home(x)
    assert np.array_equal(route.cpu().numpy().view(np.uint32), ids_full), "home routing = the block's own routing"
    ids = route[:, :k].reshape(-1)
    back = torch.zeros((300 * k, 512), device="cuda")
    pos = torch.arange(300 * k, dtype=torch.int32, device="cuda")
    for r in range(3):
        mine = torch.nonzero((ids >= 16 * r) & (ids < 16 * r + 16)).reshape(-1)
        xr = blks[r].gather_rows(x, (mine // k).to(torch.int32))
        assert torch.equal(xr, x[mine // k])
        rr = torch.stack((ids[mine], route[:, k:].reshape(-1)[mine]), 1).contiguous()
        back[mine] = blks[r].prefill_routed(xr, rr)
    assert eng.lib.ne_device_wait_status() == 0
    got = blks[0].combine_slots(back, pos.view(300, k), y_sh)
    assert torch.equal(got, want)
    # the packing kernel: a stable counting sort of the pairs by owner rank
    tok, sr, ps, counts = blks[0].pairs_by_owner(route, 3)
    dest = ids // 16
    perm = torch.argsort(dest, stable=True)
    assert torch.equal(counts, torch.bincount(dest, minlength=3)) and torch.equal(tok, (perm // k).to(torch.int32))
    assert torch.equal(sr[:, 0], ids[perm]) and torch.equal(sr[:, 1], route[:, k:].reshape(-1)[perm])
    assert torch.equal(ps.reshape(-1)[perm], torch.arange(300 * k, dtype=torch.int32, device="cuda"))
    # an object asked for a pair whose expert it does not hold contributes nothing for it
    odd = torch.stack((torch.full((5,), 40, dtype=torch.int32, device="cuda"), route[:5, k]), 1).contiguous()
    assert float(blks[0].prefill_routed(x[:5].contiguous(), odd).abs().max()) == 0.0
    # more pairs than one call takes (65535): the wrapper cuts them into calls; rows do not depend on their neighbours
    big = 70000
    in0 = torch.nonzero((ids >= 0) & (ids < 16)).reshape(-1)          # pairs of the first object's experts
    sel = in0[torch.arange(big, device="cuda") % in0.numel()]
    xb = x[sel // k].contiguous()
    rb = torch.stack((ids[sel], route[:, k:].reshape(-1)[sel]), 1).contiguous()
    yb = blks[0].prefill_routed(xb, rb)
    assert torch.equal(yb[:200], blks[0].prefill_routed(xb[:200].contiguous(), rb[:200].contiguous()))
    assert torch.equal(yb[-200:], blks[0].prefill_routed(xb[-200:].contiguous(), rb[-200:].contiguous()))
    assert torch.equal(yb[:in0.numel()], back[in0])
    assert eng.lib.ne_device_wait_status() == 0
