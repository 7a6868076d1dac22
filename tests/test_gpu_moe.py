"""CUDA MoE block against the oracle and the reference-generated fixture, through the C ABI."""
import numpy as np
import pytest

from ijah_b200 import packgen
from oracle import c_oracle as CO
from tests.helpers import rel_max, small_pack

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    import torch
    assert torch.cuda.is_available()
    from ijah_b200 import engine as E
    return E.Engine()


def check_block(eng, tensors, x, top_k, max_rows=None, tol_emul=2e-4):
    import torch
    from ijah_b200 import engine as E
    rows = x.shape[0]
    blk = E.MoeBlock(eng, tensors, top_k=top_k, max_rows=max_rows or rows)
    xd = torch.from_numpy(x).cuda()
    y = blk.forward(xd).cpu().numpy()
    ids, w = blk.route(rows)
    want = CO.moe_block_emul(tensors, x, top_k=top_k, want_gu=True)
    logits = blk.buffer("logits").reshape(rows, -1)
    assert rel_max(logits, want["logits"]) < 1e-5
    assert np.array_equal(ids, want["ids"]), "router top-k ids must match exactly"
    assert np.allclose(w, want["weights"], rtol=1e-5, atol=1e-7)
    assert rel_max(blk.experts_gu(rows), want["experts_gu"]) < tol_emul
    assert rel_max(blk.buffer("shared_gu").reshape(rows, 2, -1), want["shared_gu"]) < tol_emul
    assert rel_max(blk.buffer("shared_down").reshape(rows, -1), want["shared_down"]) < tol_emul
    assert rel_max(y, want["out"]) < tol_emul
    y2 = blk.forward(xd).cpu().numpy()
    assert np.array_equal(y, y2), "two runs must be bit-identical"
    yh = blk.forward_host(x)
    assert np.array_equal(y, yh)
    assert eng.lib.ne_device_wait_status() == 0
    blk.free()
    return y, want


def test_small_block_matches_reference_fixture(eng):
    t, g = small_pack()
    y, _ = check_block(eng, t, g["x"], int(g["topk"]))
    # fixture produced by the reference's tools/opref.py: layer outputs within 2e-3 max-abs
    assert rel_max(y, g["block_out"]) < 2e-3


@pytest.mark.parametrize("rows", [1, 4, 16])
def test_block_at_model_dims(eng, rows):
    # hidden 2048, intermediate 768, K5 experts, K6 shared, top-10; 64 experts keep the CPU oracle quick
    rng = np.random.default_rng(100 + rows)
    t = packgen.moe_layer(rng, hidden=2048, inter=768, experts=64)
    x = rng.standard_normal((rows, 2048)).astype(np.float16).astype(np.float32)
    check_block(eng, t, x, 10)


def test_rows_beyond_one_mma_tile(eng):
    rng = np.random.default_rng(7)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    x = rng.standard_normal((40, 512)).astype(np.float16).astype(np.float32)
    check_block(eng, t, x, 6, max_rows=64)


def test_duplicate_rows_share_experts(eng):
    # identical rows route alike: every expert is used by all rows (the grouped path), outputs identical per row
    rng = np.random.default_rng(8)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    x = np.repeat(rng.standard_normal((1, 512)).astype(np.float16).astype(np.float32), 5, 0)
    y, _ = check_block(eng, t, x, 4)
    assert all(np.array_equal(y[0], y[i]) for i in range(5))


def test_staged_run_equals_forward(eng):
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(9)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    x = torch.from_numpy(rng.standard_normal((3, 512)).astype(np.float32)).cuda()
    blk = E.MoeBlock(eng, t, top_k=4, max_rows=4)
    y = blk.forward(x).clone()
    y2 = torch.zeros_like(y)
    for s in (7, 8, 9):
        blk.stage(s, x, y2)
    assert torch.equal(y, y2)


def test_expert_parallel_partials_sum_to_the_block(eng):
    # two "ranks" on one GPU: each holds half the experts; routed partial sums add up to the routed output
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(11)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    x = torch.from_numpy(rng.standard_normal((6, 512)).astype(np.float16).astype(np.float32)).cuda()
    full = E.MoeBlock(eng, t, top_k=4, max_rows=8)
    full.forward(x)
    route = torch.from_numpy(full.buffer("route", np.uint32).view(np.int32).reshape(6, 8)).cuda()
    want = CO.moe_block_emul(t, x.cpu().numpy(), top_k=4)
    parts = []
    for r in range(2):
        blk = E.MoeBlock(eng, t, top_k=4, max_rows=8, expert_first=16 * r, expert_count=16)
        parts.append(blk.forward_routed(x, route).cpu().numpy())
    assert rel_max(parts[0] + parts[1], want["routed"]) < 2e-4


def test_layer_entry_points(eng, tmp_path):
    # the reference's layer API on a pack written in its on-disk layout (odd data offsets included)
    t, g = small_pack()
    k = int(g["topk"])
    packgen.write_pack(tmp_path / "pack", t, {"num_experts_per_tok": k}, shards=3, misalign=2)
    p = eng.pack_open(tmp_path / "pack")
    x = g["x"]
    L = eng.fn_layer(p, 0, rows=x.shape[0])
    p.close()  # the layer keeps the pack alive
    assert L.size("logits") == x.shape[0] * 33 and L.size("route") == x.shape[0] * 2 * k
    L.write("mlp_in", x)
    hm = np.random.default_rng(1).standard_normal((x.shape[0], 4, 256)).astype(np.float32)
    inj = np.random.default_rng(2).standard_normal((x.shape[0], 8)).astype(np.float32)
    L.write("h_mid", hm)
    L.write("mlp_inj", inj)
    L.run_stage(5)
    y = L.read("mlp_out").reshape(x.shape[0], -1)
    assert rel_max(y, g["block_out"]) < 2e-3
    rt = L.read("route").reshape(x.shape[0], 2 * k)
    assert np.array_equal(rt[:, :k].view(np.uint32), g["ids"].astype(np.uint32))
    assert np.allclose(rt[:, k:], g["weights"], rtol=1e-5)
    assert rel_max(L.read("shared_gu").reshape(x.shape[0], 2, -1)[:, 0], g["shared_gate_proj"]) < 2e-3
    assert rel_max(L.read("shared_down").reshape(x.shape[0], -1), g["shared_out"]) < 2e-3
    hout = L.read("h_out").reshape(x.shape[0], 4, 256)
    assert np.allclose(hout, hm + y[:, None, :] * inj[:, :4, None], rtol=1e-6, atol=1e-6)
    y1 = y.copy()
    for s in (7, 8, 9):
        L.run_dispatch(s)
    assert np.array_equal(L.read("mlp_out").reshape(x.shape[0], -1), y1)
    gu = L.read("experts_gu")
    assert gu.size == x.shape[0] * k * 2 * 128 and np.isfinite(gu).all()
    us, _ = L.time(2, 6, 0)
    assert us > 0
    from ijah_b200 import engine as E
    with pytest.raises(E.EngineError):
        L.run_stage(3)
    with pytest.raises(E.EngineError):
        L.step()
    L.free()


def test_forward_ep_summands_add_up_to_the_block(eng):
    # two expert-parallel "ranks" as two objects on one GPU: rows of both ranks in, each returns its summand
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(12)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    x_all = torch.from_numpy(rng.standard_normal((6, 512)).astype(np.float16).astype(np.float32)).cuda()
    full = E.MoeBlock(eng, t, top_k=4, max_rows=8).forward(x_all).cpu().numpy()
    total = np.zeros_like(full)
    for r in range(2):
        blk = E.MoeBlock(eng, t, top_k=4, max_rows=8, expert_first=16 * r, expert_count=16)
        part = blk.forward_ep(x_all, 3 * r, 3).cpu().numpy()
        want = CO.moe_block_emul(t, x_all.cpu().numpy(), top_k=4, expert_range=(16 * r, 16 * r + 16), shared_rows=(3 * r, 3))["out"]
        assert rel_max(part, want) < 2e-4
        total += part
    assert rel_max(total, full) < 1e-5


def test_forward_ep_with_home_rank_routing(eng):
    # as above, but every "rank" routes only its own rows and gets the routes of all rows from outside
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(13)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    x_all = torch.from_numpy(rng.standard_normal((20, 512)).astype(np.float16).astype(np.float32)).cuda()
    fullb = E.MoeBlock(eng, t, top_k=4, max_rows=32)
    full = fullb.forward(x_all).cpu().numpy()
    blks = [E.MoeBlock(eng, t, top_k=4, max_rows=32, expert_first=16 * r, expert_count=16) for r in range(2)]
    route_all = torch.empty((20, 8), dtype=torch.int32, device="cuda")
    for r in range(2):
        blks[r].route_rows(x_all[10 * r:10 * r + 10], route_all[10 * r:10 * r + 10])
    ids, _ = fullb.route(20)
    assert np.array_equal(route_all[:, :4].cpu().numpy(), ids)
    total = np.zeros_like(full)
    for r in range(2):
        total += blks[r].forward_ep_routed(x_all, route_all, 10 * r, 10).cpu().numpy()
    assert rel_max(total, full) < 1e-5
    # the same with rows and routes packed side by side (what one all-gather delivers)
    packed = torch.zeros((20, 512 + 8), dtype=torch.float32, device="cuda")
    packed[:, :512] = x_all
    for r in range(2):
        blks[r].route_rows(x_all[10 * r:10 * r + 10], packed[10 * r:10 * r + 10, 512:].view(torch.int32))
    assert torch.equal(packed[:, 512:].view(torch.int32), route_all)
    total2 = np.zeros_like(full)
    for r in range(2):
        total2 += blks[r].forward_ep_routed(packed[:, :512], packed[:, 512:].view(torch.int32), 10 * r, 10).cpu().numpy()
    assert np.array_equal(total2, total)
    assert eng.lib.ne_device_wait_status() == 0


def _tie_pack(mode):
    """Small MoE layer whose router produces exact ties: 'all' = zero router (every logit 0), 'dups' = every router row
    repeated four times (ids 4j .. 4j+3 share a logit)."""
    rng = np.random.default_rng(7)
    t = packgen.moe_layer(rng, hidden=256, inter=256, experts=64, k_expert=4, k_shared=4)
    name = "language_model.model.layers.0.mlp.gate.weight"
    dt, w = t[name]
    w = w.copy()
    if mode == "all":
        w[:] = 0
    else:
        w[:] = np.repeat(w[::4], 4, axis=0)
    t[name] = (dt, w)
    return t, rng


@pytest.mark.parametrize("mode", ["all", "dups"])
def test_router_ties_go_to_the_lowest_index(eng, mode):
    import torch
    from ijah_b200 import engine as E
    t, rng = _tie_pack(mode)
    rows, k = 5, 6
    x = rng.standard_normal((rows, 256)).astype(np.float16).astype(np.float32)
    blk = E.MoeBlock(eng, t, top_k=k, max_rows=rows)
    y = blk.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    ids, w = blk.route(rows)
    want = CO.moe_block_emul(t, x, top_k=k)
    if mode == "all":  # more candidates than a warp holds: the round-based fallback decides
        assert np.array_equal(ids, np.tile(np.arange(k), (rows, 1)))
        assert np.allclose(w, 1.0 / k)
    else:
        assert (ids[:, 0] % 4 == 0).all() and np.array_equal(ids[:, 1], ids[:, 0] + 1)
    assert np.array_equal(ids, want["ids"])
    assert rel_max(y, want["out"]) < 2e-4
    # the prefill router must pick the same experts
    yp = blk.prefill(torch.from_numpy(x).cuda()).cpu().numpy()
    assert rel_max(yp, want["out"]) < 2e-4
    assert eng.lib.ne_device_wait_status() == 0
    blk.free()


def test_misaligned_pointers_are_refused_on_the_host(eng):
    # a view that starts 4 bytes into a row would make the 16-byte copies of the kernels fault on the device: the entry
    # points check on the host and launch nothing
    import ctypes as C
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(12)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    blk = E.MoeBlock(eng, t, top_k=4, max_rows=4)
    x = torch.zeros((4, 513), device="cuda")
    y = torch.zeros((4, 512), device="cuda")
    off = C.c_void_p(x.data_ptr() + 4)
    assert eng.lib.ne_moe_forward(blk.ptr, off, 2, C.c_void_p(y.data_ptr()), None) == -1
    assert "16-byte aligned" in eng.last_error()
    assert eng.lib.ne_moe_forward(blk.ptr, C.c_void_p(x.data_ptr()), 2, C.c_void_p(y.data_ptr() + 8), None) == -1
    assert eng.lib.ne_moe_route(blk.ptr, off, 2, None, 0, None) == -1
    d = blk.desc
    bad = E.MoeDescC.from_buffer_copy(bytes(d))
    bad.router = d.router + 2
    assert eng.lib.ne_moe_create(C.byref(bad), 4) is None and "16-byte aligned" in eng.last_error()
    bad = E.MoeDescC.from_buffer_copy(bytes(d))
    bad.gate.trellis = d.gate.trellis + 8
    assert eng.lib.ne_moe_create(C.byref(bad), 4) is None and "16-byte aligned" in eng.last_error()
    assert eng.lib.ne_device_wait_status() == 0
    blk.free()
