"""ctypes wrapper of oracle/exl3_oracle.c (the fast CPU restatement). TEST INFRASTRUCTURE ONLY: tests/, smoke() and
bench.py's cpu_baseline / --impl reference legs."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None


def build():
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)


def lib():
    global _LIB
    if _LIB is None:
        so = HERE / "libexl3_oracle.so"
        if not so.exists():
            build()
        _LIB = C.CDLL(str(so))
        _LIB.oracle_threads.restype = C.c_int
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _u16(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == np.float16 else np.ascontiguousarray(a, np.uint16)


def threads():
    return lib().oracle_threads()


def decode_inner(trellis):
    tr = _u16(trellis)
    it, ot, n = tr.shape
    out = np.empty((it * 16, ot * 16), np.float32)
    lib().exl3_decode_inner(_p(tr), it, ot, n // 16, _p(out))
    return out


def linear_emul(trellis, suh, svh, x, summands=False):
    """the Linear in the device arithmetic; summands: each weight multiplied as its two float16 summands (the CUDA decode
    kernels' opt-in product mode), False: as the rounded float16 value (the reference's kernels, the CUDA kernels by default)"""
    lib().exl3_emul_summands(int(bool(summands)))
    tr, su, sv = _u16(trellis), _u16(np.asarray(suh, np.float16)), _u16(np.asarray(svh, np.float16))
    x = np.ascontiguousarray(x, np.float32).reshape(-1, tr.shape[0] * 16)
    y = np.empty((x.shape[0], tr.shape[1] * 16), np.float32)
    lib().exl3_linear_emul(_p(tr), _p(su), _p(sv), tr.shape[0] * 16, tr.shape[1] * 16, tr.shape[2] // 16, _p(x), x.shape[0], _p(y))
    return y


def router_logits(w_bf16, x):
    w = np.ascontiguousarray(w_bf16, np.uint16)
    x = np.ascontiguousarray(x, np.float32).reshape(-1, w.shape[1])
    out = np.empty((x.shape[0], w.shape[0]), np.float32)
    lib().router_logits(_p(w), w.shape[0], w.shape[1], _p(x), x.shape[0], _p(out))
    return out


def moe_block_emul(tensors, x, top_k=10, layer=0, ids=None, weights=None, want_gu=False, expert_range=None,
                   shared_rows=None, summands=False):
    """The MoE block in the device arithmetic on a packgen-style tensor dict. Returns dict(logits [M, E+1], ids,
    weights, routed, shared_gu, shared_down, out[, experts_gu]). expert_range (e0, e1) keeps only the slots whose
    expert lies in [e0, e1); shared_rows (r0, n) adds the shared expert for rows [r0, r0 + n) only (the summand one
    expert-parallel rank contributes)."""
    from . import opref_port as O
    pre = f"language_model.model.layers.{layer}.mlp."
    g = lambda n: np.asarray(tensors[pre + n][1])  # noqa: E731
    x = np.ascontiguousarray(x, np.float32)
    M, H = x.shape
    router = g("gate.weight")
    logits = router_logits(router, x)
    if ids is None:
        ids, weights = O.route_device_order(logits, top_k)
    st = {p: tuple(_u16(g(f"switch_mlp.{p}_proj.{s}")) for s in ("trellis", "suh", "svh")) for p in ("gate", "up", "down")}
    I = st["gate"][0].shape[2] * 16
    K = st["gate"][0].shape[3] // 16
    routed = np.zeros((M, H), np.float64)
    gu = np.zeros((M, top_k, 2, I), np.float32)
    L = lib()
    L.exl3_emul_summands(int(bool(summands)))
    for r in range(M):
        for k in range(top_k):
            e = int(ids[r, k])
            if expert_range is not None and not (expert_range[0] <= e < expert_range[1]):
                continue
            a = [np.ascontiguousarray(st[p][j][e]) for p in ("gate", "up", "down") for j in range(3)]
            xr = np.ascontiguousarray(x[r])
            L.moe_expert_emul(*[_p(v) for v in a], H, I, K, _p(xr), C.c_double(float(weights[r, k])),
                              _p(routed[r]), _p(gu[r, k]))
    res = dict(ids=ids, weights=weights, routed=routed.astype(np.float32))
    if pre + "shared_expert.gate_proj.trellis" in tensors:
        sg_logit = router_logits(g("shared_expert_gate.weight").reshape(1, H), x)[:, 0]
        sh = {p: tuple(g(f"shared_expert.{p}_proj.{s}") for s in ("trellis", "suh", "svh")) for p in ("gate", "up", "down")}
        sgu = np.stack([linear_emul(*sh["gate"], x, summands), linear_emul(*sh["up"], x, summands)], 1)
        act = (sgu[:, 0] / (1.0 + np.exp(-sgu[:, 0]))) * sgu[:, 1]
        sdown = linear_emul(*sh["down"], act.astype(np.float32), summands)
        gate = (1.0 / (1.0 + np.exp(-sg_logit.astype(np.float64))))[:, None]
        if shared_rows is not None:
            keep = np.zeros((M, 1))
            keep[shared_rows[0]:shared_rows[0] + shared_rows[1]] = 1.0
            gate = gate * keep
        out = routed + gate * sdown
        res.update(logits=np.concatenate([logits, sg_logit[:, None]], 1), shared_gu=sgu, shared_down=sdown)
    else:
        out = routed
        res.update(logits=logits)
    res["out"] = out.astype(np.float32)
    if want_gu:
        res["experts_gu"] = gu
    return res
