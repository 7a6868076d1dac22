"""Hyper-connection read in front of the MoE block (sub-block 4 of the reference's layer, dispatches 5 and 6) against the
fixture made by the reference's own hc_read and against the numpy restatement, through the reference's layer API."""
import numpy as np
import pytest

from ijah_b200 import packgen
from tests.helpers import hc_oracle, hc_small, rel_max, small_pack

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    import torch
    assert torch.cuda.is_available()
    from ijah_b200 import engine as E
    return E.Engine()


def test_mlp_hc_matches_reference_fixture(eng, tmp_path):
    t, g = small_pack()
    ht, hg = hc_small()
    t = dict(t)
    t.update(ht)
    packgen.write_pack(tmp_path / "pack", t, {"num_experts_per_tok": int(g["topk"])}, shards=3, misalign=2)
    p = eng.pack_open(tmp_path / "pack")
    h = hg["h"]
    rows = h.shape[0]
    L = eng.fn_layer(p, 0, rows=rows)
    assert L.size("mlp_mix") == rows * 128 and L.size("mlp_inj") == rows * 8
    L.write("h_mid", h)
    L.run_stage(4)
    mix = L.read("mlp_mix").reshape(rows, -1)
    inj = L.read("mlp_inj").reshape(rows, 8)
    xin = L.read("mlp_in").reshape(rows, -1)
    assert rel_max(mix, hg["f32_mix"]) < 1e-4
    assert rel_max(inj[:, :4], hg["f32_inject_w"]) < 1e-5
    assert rel_max(xin, hg["f32_block_in"]) < 1e-4
    assert rel_max(xin, hg["bf16_block_in"]) < 2e-2  # the reference's bf16-rounded flow
    # the per-stream 1 / rms values sit behind the inject gates (reference kernels/fn_trunk.metal:75)
    want_inv = 1.0 / np.sqrt((h.reshape(rows, 4, -1) ** 2).mean(-1) + 1e-6)
    assert np.allclose(inj[:, 4:], want_inv, rtol=1e-5)
    # the two dispatches one by one give the same bits; then the MoE block runs on the mixed input and writes the streams
    L.write("mlp_in", np.zeros_like(xin))
    L.run_dispatch(5)
    L.run_dispatch(6)
    assert np.array_equal(L.read("mlp_in").reshape(rows, -1), xin)
    L.run_stage(5)
    y = L.read("mlp_out").reshape(rows, -1)
    hout = L.read("h_out").reshape(rows, 4, -1)
    assert np.allclose(hout, h.reshape(rows, 4, -1) + y[:, None, :] * inj[:, :4, None], rtol=1e-6, atol=1e-6)
    L.free()
    p.close()


@pytest.mark.parametrize("rows", [1, 11, 19])
def test_mlp_hc_reference_sizes(eng, tmp_path, rows):
    # the reference's hyper-connection sizes (stream width 2560, 320 mix rows, groups of 64) over a small MoE block;
    # 11 and 19 rows take more than one pass of eight rows
    rng = np.random.default_rng(5)
    t = packgen.moe_layer(rng, layer=0, hidden=2560, inter=128, experts=16, k_expert=5, k_shared=6)
    t.update(packgen.hc_block(rng, layer=0, which="mlp", hidden=2560, lr=320, group=64))
    packgen.write_pack(tmp_path / "pack", t, {"num_experts_per_tok": 4}, shards=2)
    p = eng.pack_open(tmp_path / "pack")
    L = eng.fn_layer(p, 0, rows=rows)
    h = (rng.standard_normal((rows, 4 * 2560)) * 1.5).astype(np.float32)
    L.write("h_mid", h)
    L.run_stage(4)
    want = hc_oracle(t, h)
    assert rel_max(L.read("mlp_mix").reshape(rows, -1), want["mix"]) < 1e-4
    assert rel_max(L.read("mlp_inj").reshape(rows, 8)[:, :4], want["inject_w"]) < 1e-5
    assert rel_max(L.read("mlp_in").reshape(rows, -1), want["block_in"]) < 1e-4
    L.free()
    p.close()


def test_layer_without_hc_refuses_stage_4(eng, tmp_path):
    t, g = small_pack()
    packgen.write_pack(tmp_path / "pack", t, {"num_experts_per_tok": int(g["topk"])})
    p = eng.pack_open(tmp_path / "pack")
    L = eng.fn_layer(p, 0, rows=1)
    from ijah_b200 import engine as E
    with pytest.raises(E.EngineError, match="mlp_hyper_connection"):
        L.run_stage(4)
    L.free()
    p.close()
