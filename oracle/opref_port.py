"""CPU restatement (numpy) of the reference's operator reference for the EXL3 MoE / trunk hot path. TEST INFRASTRUCTURE.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this module.

Each function names the reference function it follows (paths inside the reference project). Two flavours exist for the
EXL3 linears, as in the reference's own tests:
  *_exact   float64 x @ W_hat with W_hat = diag(suh) H W' H diag(svh)           (tools/opref.py:142-151,401-435)
  *_emul    the device arithmetic: (x*suh) and the input Hadamard in float32 with the kernels' butterfly order, the
            result rounded to float16, times the exact float16 W', float32/64 afterwards
            (tests/trunk6/check_kernels.py:47-60,93-99; kernels/fn_moe.metal:304-311,370-384)
Pinned by tests/golden/*.npz, which tests/golden/make_golden.py produced by running the reference's tools/opref.py
itself (on top of oracle/exl3_codec.py, the one module the reference does not ship).
"""
import numpy as np

from . import exl3_codec as X


# ------------------------------------------------------------------ dtype helpers (tools/opref.py:28-46)
def bf16_round(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return r.view(np.float32).reshape(np.shape(x))


def bf16_bits_to_f32(u16):
    return (np.asarray(u16, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) >> 16).astype(np.uint16)


def sigmoid(x):
    with np.errstate(over="ignore"):
        return 1.0 / (1.0 + np.exp(-np.asarray(x, np.float32)))


def silu(x):
    x = np.asarray(x, np.float32)
    return x * sigmoid(x)


def linear(x, W):
    """y = x @ W^T, W [out, in], float32 (tools/opref.py:197-199 with bf=False)"""
    return np.asarray(x, np.float32) @ np.asarray(W, np.float32).T


# ------------------------------------------------------------------ router (tools/opref.py:388-398, bf=False)
def moe_route(x, Wg, top_k=10):
    """logits = x @ Wg^T; p = softmax; ids = top-k by p, ties -> lowest index; w = p[ids] / sum(p[ids])"""
    logits = linear(x, Wg)
    z = logits - logits.max(-1, keepdims=True)
    p = np.exp(z)
    p = (p / p.sum(-1, keepdims=True)).astype(np.float32)
    ids = np.argsort(-p, axis=-1, kind="stable")[..., :top_k]
    w = np.take_along_axis(p, ids, -1)
    w = (w / w.sum(-1, keepdims=True)).astype(np.float32)
    return logits, p, ids, w


def route_device_order(logits, top_k=10):
    """What the device router computes (kernels/fn_moe.metal:76-131): top-k on the LOGITS, ties -> lowest index,
    w = exp(l - l_max) / sum over the k selected. Same ids as moe_route unless two probabilities round together."""
    lg = np.asarray(logits, np.float32)
    ids = np.argsort(-lg, axis=-1, kind="stable")[..., :top_k]
    sel = np.take_along_axis(lg, ids, -1)
    p = np.exp(sel - sel[..., :1])
    return ids, (p / p.sum(-1, keepdims=True, dtype=np.float32)).astype(np.float32)


# ------------------------------------------------------------------ Hadamard
def had_blocks(x, n):
    """x @ blockdiag(H_n) along the last axis, float64 (tools/opref.py:401-405 for n = 128)"""
    s = np.shape(x)
    return (np.asarray(x, np.float64).reshape(*s[:-1], s[-1] // n, n) @ X._had(n)).reshape(s)


def had128(x):
    return had_blocks(x, 128)


def fwht_f32(x, n):
    """The kernels' input Hadamard in float32: butterflies over index bits 0, 1, 2, ... inside blocks of n, then the
    1/sqrt(n) scale (tests/trunk6/check_kernels.py:47-60; kernels/ne_common.h:95-103)."""
    x = np.asarray(x, np.float32)
    lead, k = x.shape[:-1], x.shape[-1]
    v = x.reshape(-1, k // n, n).copy()
    R = v.shape[0]
    b = 1
    while b < n:
        v = v.reshape(R, k // n, n // (2 * b), 2, b)
        lo, hi = v[:, :, :, 0, :].copy(), v[:, :, :, 1, :].copy()
        v[:, :, :, 0, :] = lo + hi
        v[:, :, :, 1, :] = lo - hi
        v = v.reshape(R, k // n, n)
        b *= 2
    return (v * np.float32(1.0 / np.sqrt(n))).reshape(*lead, k)


# ------------------------------------------------------------------ EXL3 linear
def exl3_inner_out(x, inner, suh):
    """((x * suh) H) W' before the output transform (tools/opref.py:408-410)"""
    n = X.had_size(np.shape(x)[-1])
    return (had_blocks(np.asarray(x, np.float64) * np.asarray(suh, np.float64), n) @ np.asarray(inner, np.float64)).astype(np.float32)


def exl3_finish(inner_out, svh):
    """(raw H) * svh (tools/opref.py:413-414)"""
    n = X.had_size(np.shape(inner_out)[-1])
    return (had_blocks(inner_out, n) * np.asarray(svh, np.float64)).astype(np.float32)


def exl3_prep_emul(x, suh):
    """float16(H(x * suh)) with the product and butterflies in float32: the A operand the kernels build"""
    x = np.asarray(x, np.float32)
    n = X.had_size(x.shape[-1])
    xs = (x * np.asarray(suh, np.float16).astype(np.float32)).astype(np.float32)
    return fwht_f32(xs, n).astype(np.float16)


def exl3_linear_exact(x, trellis, suh, svh):
    """float64 x @ W_hat (tools/convert_trunk_enc.py:176-180 decode, tools/opref.py:116-131)"""
    W = X.reconstruct(X.decode_inner(trellis), np.asarray(suh, np.float16), np.asarray(svh, np.float16))
    return np.asarray(x, np.float64) @ W


def exl3_linear_emul(x, trellis, suh, svh, inner=None, summands=False):
    """y_emul of tests/trunk6/check_kernels.py:93-99: device arithmetic, float64 after the float16 operand. summands:
    every weight enters the product as its two float16 summands (the CUDA decode kernels' opt-in mode: no half add, hence
    no rounding of the sum); False: as the rounded float16 value (the reference's kernels, the CUDA kernels by default)"""
    inner = X.decode_inner(trellis, rounded=not summands).astype(np.float64) if inner is None else np.asarray(inner, np.float64)
    raw = exl3_prep_emul(x, suh).astype(np.float64) @ inner
    m = raw.shape[-1]
    return had_blocks(raw, X.had_size(m)) * np.asarray(svh, np.float16).astype(np.float64)


# ------------------------------------------------------------------ experts (tools/opref.py:417-446, bf=False)
def swiglu_expert(x, Wg, Wu, Wd):
    return (silu(x @ Wg) * (x @ Wu)) @ Wd


class Exl3Linear:
    """trellis u16 [in/16, out/16, 16K], suh f16 [in], svh f16 [out] of one Linear"""

    def __init__(self, trellis, suh, svh):
        self.trellis = np.asarray(trellis, np.uint16)
        self.suh = np.asarray(suh, np.float16)
        self.svh = np.asarray(svh, np.float16)
        self._inner = None
        self._inner_sum = None
        self._dense = None

    @property
    def inner(self):
        if self._inner is None:
            self._inner = X.decode_inner(self.trellis)
        return self._inner

    @property
    def inner_sum(self):
        """W' with every value the unrounded sum of its two float16 summands"""
        if self._inner_sum is None:
            self._inner_sum = X.decode_inner(self.trellis, rounded=False)
        return self._inner_sum

    @property
    def dense(self):
        """W_hat [in, out] float32 (tools/opref.py:142-151 `expert`)"""
        if self._dense is None:
            self._dense = X.reconstruct(self.inner, self.suh, self.svh).astype(np.float32)
        return self._dense


def moe_routed(x, ids, w, experts):
    """sum_k w_k expert_{ids_k}(x) per row in slot order; experts(e) -> (gate, up, down) Exl3Linear
    (tools/opref.py:422-435 with bf=False)"""
    x = np.asarray(x, np.float32).reshape(-1, np.shape(x)[-1])
    y = np.zeros_like(x)
    for r in range(x.shape[0]):
        for e, we in zip(np.asarray(ids)[r], np.asarray(w, np.float32)[r]):
            g, u, d = experts(int(e))
            y[r] += we * swiglu_expert(x[r], g.dense, u.dense, d.dense)
    return y


def shared_expert(x, gate, up, down, sgate_w):
    """(shared_out, shared_scale): down(silu(gate x) * up x), sigmoid(x . w_sg) (tools/opref.py:438-446, bf=False)"""
    x = np.asarray(x, np.float32)
    act = silu(x @ gate.dense) * (x @ up.dense)
    return (act @ down.dense).astype(np.float32), sigmoid(linear(x, sgate_w))


def moe_block_exact(x, router_w, sgate_w, experts, shared, top_k=10):
    """The whole block in the operator reference's float32 arithmetic: dict logits, ids, weights, routed, shared, out"""
    x = np.asarray(x, np.float32).reshape(-1, np.shape(x)[-1])
    logits, _, ids, w = moe_route(x, router_w, top_k)
    routed = moe_routed(x, ids, w, experts)
    sh, scale = shared_expert(x, *shared, sgate_w)
    return dict(logits=logits, ids=ids, weights=w, routed=routed, shared=sh, shared_scale=scale,
                out=(routed + scale * sh).astype(np.float32))


def moe_block_emul(x, router_w, sgate_w, experts, shared, top_k=10, ids=None, w=None, summands=False):
    """The block in the device arithmetic order (kernels/fn_moe.metal:304-343 gate/up, :370-445 down): float16
    prepared operands, raw inner products, H * svh, silu(g) * u * suh_down, H, float16, down, H * svh * w_k, slots
    summed in slot order, + sigmoid(shared logit) * shared. Returns dict with the intermediates the C ABI exposes."""
    x = np.asarray(x, np.float32).reshape(-1, np.shape(x)[-1])
    M = x.shape[0]
    logits = linear(x, router_w)
    sg_logit = linear(x, sgate_w).reshape(M)
    if ids is None:
        ids, w = route_device_order(logits, top_k)
    gu = np.zeros((M, top_k, 2, experts(0)[0].inner.shape[1]), np.float32)
    y = np.zeros((M, x.shape[1]), np.float64)
    inner = (lambda l: l.inner_sum) if summands else (lambda l: l.inner)  # noqa: E731
    for r in range(M):
        for k in range(top_k):
            g, u, d = experts(int(ids[r, k]))
            gr = exl3_prep_emul(x[r], g.suh).astype(np.float64) @ inner(g).astype(np.float64)
            ur = exl3_prep_emul(x[r], u.suh).astype(np.float64) @ inner(u).astype(np.float64)
            gu[r, k, 0], gu[r, k, 1] = gr, ur
            gv = (had128(gr) * g.svh.astype(np.float64)).astype(np.float32)
            uv = (had128(ur) * u.svh.astype(np.float64)).astype(np.float32)
            mid = (gv / (1.0 + np.exp(-gv))) * uv
            y[r] += np.float64(w[r, k]) * exl3_linear_emul(mid, None, d.suh, d.svh, inner=inner(d))
    sgu = np.stack([exl3_linear_emul(x, None, shared[0].suh, shared[0].svh, inner=inner(shared[0])),
                    exl3_linear_emul(x, None, shared[1].suh, shared[1].svh, inner=inner(shared[1]))], 1)
    sgu = sgu.astype(np.float32)
    act = silu(sgu[:, 0]) * sgu[:, 1]
    sdown = exl3_linear_emul(act, None, shared[2].suh, shared[2].svh, inner=inner(shared[2])).astype(np.float32)
    out = y + sigmoid(sg_logit)[:, None].astype(np.float64) * sdown
    return dict(logits=np.concatenate([logits, sg_logit[:, None]], 1), ids=ids, weights=w, experts_gu=gu,
                shared_gu=sgu, shared_down=sdown, routed=y.astype(np.float32), out=out.astype(np.float32))


# ------------------------------------------------------------------ hyper-connection read (8-bit affine weights)
def affine_dequant(wq_u32, scales_bf16, biases_bf16):
    """MLX 8-bit affine (reference tools/opref.py:172-180): wq U32 [out, in/4] = codes little-endian within each word,
    scales / biases bf16 bits [out, in/group]; w = q * scale + bias -> f32 [out, in]."""
    q = np.ascontiguousarray(wq_u32).view(np.uint8).astype(np.float32)
    out, n_in = q.shape
    sc, bi = bf16_bits_to_f32(scales_bf16), bf16_bits_to_f32(biases_bf16)
    ng = sc.shape[-1]
    q = q.reshape(out, ng, n_in // ng)
    return (q * sc[..., None] + bi[..., None]).reshape(out, n_in)


def q8_linear(x, wq_u32, scales_bf16, biases_bf16):
    """x @ W^T for an 8-bit affine Linear in f32 (reference tools/opref.py:183-194 `linear_big` with bf=False)"""
    return np.asarray(x, np.float32) @ affine_dequant(wq_u32, scales_bf16, biases_bf16).T


def q8_embed(ids, wq_u32, scales_bf16, biases_bf16):
    """rows `ids` of an 8-bit affine table, dequantised and rounded to bf16 (reference tools/opref.py:133-141 `linear_rows`)"""
    ids = np.asarray(ids).reshape(-1)
    return bf16_round(affine_dequant(np.asarray(wq_u32)[ids], np.asarray(scales_bf16)[ids], np.asarray(biases_bf16)[ids]))


class AffineLinear:
    """An 8-bit affine Linear seen as the float32 matrix it stands for: .dense is [in, out] like Exl3Linear.dense, so
    the float64 block and stack references take either kind of projection."""

    def __init__(self, weight, scales, biases):
        self.dense = np.ascontiguousarray(affine_dequant(weight, scales, biases).T)


def shared_expert_q8(x, gate, up, down, sgate_w):
    """the shared expert with 8-bit affine projections (reference tools/opref.py:438-446 with bf=False; each of gate, up,
    down = (weight u32, scales, biases)): (gate_proj, up_proj, out, sigmoid scale [rows, 1])"""
    x = np.asarray(x, np.float32)
    g = q8_linear(x, *gate)
    u = q8_linear(x, *up)
    out = q8_linear(silu(g) * u, *down)
    return g, u, out, sigmoid(linear(x, sgate_w)).reshape(-1, 1)


def hc_read(h, norm_w, inject_w, down, up, streams=4, eps=1e-6):
    """Hyper-connection read in f32 (reference tools/opref.py:221-236 with bf=False; models/flash_next/layer.mm:524-531):
    h [rows, streams*H]; norm_w f32 [streams*H]; inject_w f32 [streams, streams*H]; down f32 [LR, streams*H]; up f32
    [streams*H, LR] (dense, from affine_dequant). Returns dict normed, mix, block_in, inject_w."""
    h = np.asarray(h, np.float32)
    rows, hcd = h.shape
    H = hcd // streams
    x = h.reshape(rows, streams, H)
    normed = (x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)).reshape(rows, hcd) * norm_w
    mix = silu((normed @ down.T) / streams)
    upv = mix @ up.T
    m = sigmoid(upv).reshape(rows, streams, H) * normed.reshape(rows, streams, H)
    return dict(normed=normed.astype(np.float32), mix=mix.astype(np.float32), block_in=np.mean(m, axis=-2).astype(np.float32),
                inject_w=(2.0 * sigmoid((normed @ inject_w.T) / streams)).astype(np.float32))
