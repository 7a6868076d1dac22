"""Generate tests/golden/*.npz by running the REFERENCE's own numpy operator reference (tools/opref.py, unmodified) on
a small seeded synthetic pack.

    python tests/golden/make_golden.py --reference /path/to/reference/checkout

The reference's tools import `exl3_codec` (and convert_trunk_enc also `encode`), lab modules the reference does not
ship. A scratch IJAH_REF_DIR is built with convert/exl3_codec.py = this repository's oracle/exl3_codec.py and an
`encode.py` whose encoder-only names raise if called; everything else that runs is the reference's code. The fixtures
therefore pin the operator semantics (routing, Hadamard placement, scale order, SwiGLU, slot sum, shared expert,
trunk decode) but not the codec's bit layout, which has no reference-side golden (see oracle/exl3_codec.py).

The pack itself is not stored: tests regenerate it from the seed with ijah_b200.packgen and check the SHA-256 of its
tensors against the one recorded here, so a drift of the random stream is reported, not silently compared.
"""
import argparse
import hashlib
import os
import shutil
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
from ijah_b200 import packgen  # noqa: E402

SEED = 20261125
DIMS = dict(hidden=256, inter=128, experts=32, k_expert=5, k_shared=6)
TOPK = 4
HC = dict(hidden=256, lr=128, group=64)  # hyper-connection read of layer 0 (the reference's sizes: 2560, 320, 64)
TRUNK = [dict(layer=0, hidden=256, q_out=512, kv_out=64, K=6), dict(layer=1, hidden=256, q_out=512, kv_out=64, K=8)]


def small_pack_tensors():
    rng = np.random.default_rng(SEED)
    t = packgen.moe_layer(rng, layer=0, **DIMS)
    for tr in TRUNK:
        t.update(packgen.trunk_layer(rng, **tr))
    return t


def hc_tensors():
    """the mlp hyper-connection tensors of layer 0, from a random stream of their own (the MoE fixture's pack is unchanged)"""
    return packgen.hc_block(np.random.default_rng(SEED + 2), layer=0, which="mlp", **HC)


def hc_inputs():
    rng = np.random.default_rng(SEED + 3)
    return (rng.standard_normal((5, 4 * HC["hidden"])) * np.array([0.5, 1.0, 2.0, 4.0]).repeat(HC["hidden"])).astype(np.float32)


Q8 = dict(vocab=1024, hidden=256, group=64)  # 8-bit affine LM head and token embedding (the reference's: 248320 x 2560, group 64 / 128)


def q8_tensors():
    rng = np.random.default_rng(SEED + 4)
    t = {}
    for name in ("language_model.lm_head", "language_model.model.embed_tokens"):
        w, sc, bi = packgen.q8_linear(rng, Q8["vocab"], Q8["hidden"], Q8["group"])
        t[name + ".weight"], t[name + ".scales"], t[name + ".biases"] = ("U32", w), ("BF16", sc), ("BF16", bi)
    return t


def shared_q8_tensors():
    """an 8-bit affine shared expert (layer 3 of the scratch pack: no EXL3 shared expert there to shadow it)"""
    return packgen.shared_expert_q8(np.random.default_rng(SEED + 6), layer=3, hidden=DIMS["hidden"], inter=DIMS["inter"], group=64)


def q8_inputs():
    rng = np.random.default_rng(SEED + 5)
    return rng.standard_normal((6, Q8["hidden"])).astype(np.float32), rng.integers(0, Q8["vocab"], 9).astype(np.int32)


def tensors_digest(t):
    h = hashlib.sha256()
    for name in sorted(t):
        h.update(name.encode())
        h.update(np.ascontiguousarray(t[name][1]).tobytes())
    return h.hexdigest()


def inputs():
    rng = np.random.default_rng(SEED + 1)
    return rng.standard_normal((4, DIMS["hidden"])).astype(np.float16).astype(np.float32)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository (its tools/opref.py is imported unmodified)")
    ap.add_argument("--which", default="all", choices=["all", "moe", "hc", "q8"], help="which fixture file to (re)write")
    a = ap.parse_args()
    tmp = Path(tempfile.mkdtemp(prefix="ijah_golden_"))
    try:
        (tmp / "ref/convert").mkdir(parents=True)
        shutil.copy(ROOT / "oracle/exl3_codec.py", tmp / "ref/convert/exl3_codec.py")
        (tmp / "ref/convert/encode.py").write_text(
            "def _enc(*a, **k):\n    raise NotImplementedError('encoder-only name; not on the decode path')\n"
            "block_ldl = block_rms = refit_scales = sample_scale_tiles = _enc\n")
        tens = small_pack_tensors()
        hct = hc_tensors()
        tens.update(hct)
        q8t = q8_tensors()
        q8t.update(shared_q8_tensors())
        tens.update(q8t)
        pack = packgen.write_pack(tmp / "pack", tens, {"num_experts_per_tok": TOPK}, shards=3, misalign=2)
        os.environ["IJAH_REF_DIR"] = str(tmp / "ref")
        os.environ["IJAH_PACK"] = str(pack)
        sys.path.insert(0, str(Path(a.reference) / "tools"))
        import opref as O  # the reference's module

        P = O.PackNP()
        if a.which in ("all", "hc"):
            # the reference's hc_read with its two module constants (stream width D = 2560, HC = 4) set to the small pack's
            O.D = HC["hidden"]
            h = hc_inputs()
            hc = dict(seed=np.int64(SEED), digest=np.array(tensors_digest(hct)), h=h)
            for tag, bf in (("f32", False), ("bf16", True)):
                r = O.hc_read(h, P, "language_model.model.layers.0.mlp_hyper_connection", bf=bf)
                for k in ("normed", "mix", "block_in", "inject_w"):
                    hc[f"{tag}_{k}"] = np.asarray(r[k], np.float32)
            np.savez_compressed(HERE / "hc_small.npz", **hc)
            print("wrote", HERE / "hc_small.npz", {k: np.shape(v) for k, v in hc.items()})
            if a.which == "hc":
                return
        if a.which in ("all", "q8"):
            x, ids = q8_inputs()
            q8 = dict(seed=np.int64(SEED), digest=np.array(tensors_digest(q8t)), x=x, ids=ids)
            q8["head_y"] = np.asarray(O.linear_big(x, P, "language_model.lm_head", bf=False), np.float32)
            q8["embed_rows"] = np.asarray(P.linear_rows("language_model.model.embed_tokens", ids), np.float32)
            sh = O.shared_expert(x, P, "language_model.model.layers.3.mlp", bf=False)  # x: [6, 256] = the small pack's hidden size
            for k, v in sh.items():
                q8["sh8_" + k] = np.asarray(v, np.float32)
            np.savez_compressed(HERE / "q8_small.npz", **q8)
            print("wrote", HERE / "q8_small.npz", {k: np.shape(v) for k, v in q8.items()})
            if a.which == "q8":
                return
        for k in list(hct) + list(q8t):
            del tens[k]
        x = inputs()
        out = dict(seed=np.int64(SEED), digest=np.array(tensors_digest(tens)), x=x, topk=np.int64(TOPK))
        pre = "language_model.model.layers.0.mlp"
        Wg = P.tensor(pre + ".gate.weight")
        logits, p, ids, w = O.moe_route(x, Wg, top_k=TOPK, bf=False)
        out.update(logits=logits, probs=p, ids=ids.astype(np.int32), weights=w)
        out["routed"] = O.moe_routed(x, ids, w, P, 0, bf=False)
        sh = O.shared_expert(x, P, pre, bf=False)
        for k, v in sh.items():
            out[k] = np.asarray(v, np.float32)
        out["block_out"] = (out["routed"] + sh["shared_scale"] * sh["shared_out"]).astype(np.float32)
        # dense expert weights of two experts (all three projections), subsampled to keep the file small, + sums
        for e in (int(ids[0, 0]), 31):
            for proj in ("gate", "up", "down"):
                W = P.expert(0, proj, e)
                out[f"W_{proj}_{e}_sub"] = W[::7, ::5].copy()
                out[f"W_{proj}_{e}_sum"] = np.float64(W.astype(np.float64).sum())
                inner, suh, svh = P.expert_parts(0, proj, e)
                out[f"inner_{proj}_{e}_sub"] = inner[::7, ::5].copy()
        e = int(ids[0, 0])
        inner, suh, svh = P.expert_parts(0, "gate", e)
        io = O.exl3_inner_out(x[0], inner, suh)
        out["gate_inner_out"] = io
        out["gate_finish"] = O.exl3_finish(io, svh)
        out["gate_expert_id"] = np.int64(e)
        # trunk linears (convert_trunk_enc.decode through PackNP.linear): y = x @ W^T, W [out, in]
        for tr in TRUNK:
            for proj in ("q", "k", "v", "o"):
                name = f"language_model.model.layers.{tr['layer']}.self_attn.{proj}_proj"
                W = P.linear(name)
                xin = x if W.shape[1] == DIMS["hidden"] else np.tile(x, (1, W.shape[1] // DIMS["hidden"]))
                out[f"trunk_L{tr['layer']}_{proj}_y"] = O.linear(xin, W, bf=False)
                out[f"trunk_L{tr['layer']}_{proj}_Wsub"] = W[::5, ::7].copy()
        np.savez_compressed(HERE / "moe_small.npz", **out)
        print("wrote", HERE / "moe_small.npz", {k: np.shape(v) for k, v in out.items()})
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()
