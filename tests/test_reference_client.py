"""Drop-in check: the reference's OWN ctypes client (its tools/engine.py, unmodified) driving this library through NE_LIB.

The reference tree is looked for in $IJAH_REFERENCE_DIR or beside this repository (a directory named `reference`); the
tests skip when it is not there. Nothing of the reference is copied: its module is imported from where it lies.
The CPU test covers loading, symbol binding and the pack reader; the GPU test covers buffers, the layer entry points,
the kernel-by-name entry and the model step, each against this repository's own client or the oracle.
"""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import pytest

from ijah_b200 import packgen

ROOT = Path(__file__).resolve().parents[1]
REF = Path(os.environ.get("IJAH_REFERENCE_DIR", ROOT.parent / "reference"))
CLIENT = REF / "tools" / "engine.py"
pytestmark = pytest.mark.skipif(not CLIENT.exists(), reason="the reference tree (tools/engine.py) is not on this machine")


@pytest.fixture(scope="module")
def ref():
    """the reference's tools/engine.py, imported with NE_LIB pointing at libijah_b200.so (the one-line change a maintainer makes)"""
    os.environ["NE_LIB"] = str(ROOT / "ijah_b200" / "libijah_b200.so")
    sys.path.insert(0, str(REF / "tools"))
    try:
        spec = importlib.util.spec_from_file_location("reference_engine_client", CLIENT)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        sys.path.remove(str(REF / "tools"))
    return mod


def small_pack(tmp_path):
    rng = np.random.default_rng(31)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    t.update(packgen.trunk_layer(rng, hidden=512, q_out=256, kv_out=128, K=6))
    H, V = 512, 1024
    t["language_model.model.embed_tokens.weight"] = ("BF16", packgen.f32_to_bf16_bits(rng.standard_normal((V, H))))
    cfg = {"num_experts_per_tok": 4, "num_hidden_layers": 1, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64}
    packgen.write_pack(tmp_path / "pack", t, cfg, shards=3, misalign=2)
    return t, tmp_path / "pack"


def test_reference_client_binds_and_reads_packs(ref, tmp_path):
    eng = ref.Engine()
    assert eng.abi_version() == 1
    # what the reference's client could not bind are entry points of subsystems outside this library (attention / GDN state,
    # sampler knobs, generation loop, n-gram embedding), none of the MoE / trunk path
    assert set(eng.missing) <= {"ne_fn_layer_set_state", "ne_fn_layer_get_state", "ne_fn_layer_set_kv", "ne_fn_layer_get_kv",
                                "ne_fn_model_set_sampler", "ne_fn_model_set_mask", "ne_fn_model_set_sampler_ex", "ne_fn_model_set_seen",
                                "ne_fn_model_set_logit_bias", "ne_fn_model_set_rng_step", "ne_fn_model_top", "ne_fn_model_generate",
                                "ne_fn_model_run_head", "ne_fn_ngram", "ne_fn_model_prefill"}
    t, path = small_pack(tmp_path)
    p = eng.pack_open(path)
    assert p.config()["num_experts_per_tok"] == 4 and p.config()["expert_quant"]["codebook"] == "mcg"
    assert p.names() == sorted(t)
    for name in ("language_model.model.layers.0.mlp.gate.weight", "language_model.model.layers.0.mlp.switch_mlp.down_proj.trellis",
                 "language_model.model.layers.0.self_attn.q_proj.svh"):
        d = p.info(name)
        dt, arr = t[name]
        assert d.dtype == dt and d.shape == arr.shape and d.nbytes == arr.nbytes
        assert np.array_equal(np.asarray(d.host).view(np.uint16), np.ascontiguousarray(arr).view(np.uint16))
    with pytest.raises(KeyError):
        p.info("no.such.tensor")
    assert eng.kernel_exists("exl3_linear") and not eng.kernel_exists("fn_moe_gateup_k5_r1")
    p.close()
    with pytest.raises(ref.EngineError):
        eng.pack_open(tmp_path / "missing")


@pytest.mark.gpu
def test_reference_client_drives_buffers_layer_kernel_and_model(ref, tmp_path):
    import torch
    assert torch.cuda.is_available()
    from ijah_b200 import engine as E
    from oracle import c_oracle as CO
    eng = ref.Engine()
    dev = eng.device()
    assert dev["backend"] == "cuda" and dev["has_nax"] and "B200" in dev["name"]
    # buffers: managed memory behaves like the reference's shared storage
    a = np.arange(1000, dtype=np.float32)
    buf = eng.from_numpy(a)
    assert buf.size >= a.nbytes and np.array_equal(buf.download(np.float32, (1000,)), a)
    view = buf.numpy(np.float32, (1000,))
    view[3] = -7.0
    assert buf.download(np.float32, (1000,))[3] == -7.0
    buf.free()
    t, path = small_pack(tmp_path)
    p = eng.pack_open(path)
    rows, k = 3, 4
    x = np.random.default_rng(5).standard_normal((rows, 512)).astype(np.float16).astype(np.float32)
    # the layer entry points, as tests/test_fn_layer.py of the reference uses them
    L = eng.fn_layer(p, 0, rows=rows)
    L.write("mlp_in", x)
    L.run_stage(5)
    y = L.read("mlp_out").reshape(rows, 512)
    want = CO.moe_block_emul(t, x, top_k=k)
    assert np.abs(y - want["out"]).max() / np.abs(want["out"]).max() < 2e-4
    route = L.read("route").reshape(rows, 2 * k)
    assert np.array_equal(route[:, :k].copy().view(np.uint32), want["ids"].astype(np.uint32))
    us, _ = L.time(2, 6, 0)
    assert us > 0
    L.free()
    # kernel by name: one EXL3 Linear on pack tensors (TensorDesc arguments) and caller buffers, timed over repetitions
    pre = "language_model.model.layers.0.self_attn.q_proj."
    xb, yb = eng.from_numpy(x), eng.alloc(rows * 256 * 4)
    ms = eng.run_kernel("exl3_linear", [p.info(pre + "trellis"), p.info(pre + "suh"), p.info(pre + "svh"), xb, yb,
                                        np.array([512, 256, 6, rows], np.uint32)], grid=(1, 1, 1), tg=(1, 1, 1), reps=5)
    assert ms > 0
    got = yb.download(np.float32, (rows, 256))
    ref_y = CO.linear_emul(t[pre + "trellis"][1], t[pre + "suh"][1], t[pre + "svh"][1], x)
    assert np.linalg.norm(got - ref_y) / np.linalg.norm(ref_y) < 5e-5
    with pytest.raises(ref.EngineError, match="Metal"):
        eng.run_kernel("fn_moe_router_r1", [xb], grid=(1, 1, 1), tg=(32, 1, 1))
    # the model entry point: the reference client's one-token step against this repository's own client
    m = eng.fn_model(p, tmax=64)
    nx, lp, am, lg = m.step(7, head=True, logits=True)
    mine = E.Engine().fn_model(E.Engine().pack_open(path), tmax=64, max_rows=1)
    lg2, nx2, lp2, _ = mine.step(7)
    assert nx == nx2 == am and np.array_equal(lg[:1024], lg2) and abs(lp - lp2) < 1e-5
    p.close()
