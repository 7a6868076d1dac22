"""CPU restatement (numpy, float64) of the decoder stack the library runs behind ne_fn_model_*: bf16 embedding, per layer
RMS norm -> EXL3 q / k / v -> attention stand-in over a fixed KV cache plus the row's own key / value -> EXL3 o -> residual
-> RMS norm -> MoE block -> residual, final RMS norm, bf16 LM head. TEST INFRASTRUCTURE ONLY (tests/, smoke(), the CPU
legs of bench.py).

The EXL3 linears and the MoE block are the operator reference of oracle/opref_port.py (which restates the reference's
tools/opref.py:388-446); the glue ops around them are stand-ins of this build (the reference's attention, GDN and
hyper-connections are out of scope), restated here only so that whole-stack logits have something to be compared with.
"""
import numpy as np

from . import opref_port as O


def rms(x, w=None, eps=1e-6):
    x = np.asarray(x, np.float64)
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return y if w is None else y * np.asarray(w, np.float64)


def attn_standin(q, knew, vnew, kc, vc, heads, kv_heads, hd):
    """q [R, heads*hd], knew / vnew [R, kv_heads*hd], kc / vc [T, kv_heads, hd] -> [R, heads*hd]: per query head a softmax
    over the T cached positions and the row's own (k, v), grouped-query"""
    R = q.shape[0]
    G = heads // kv_heads
    out = np.zeros((R, heads * hd))
    kc, vc = np.asarray(kc, np.float64), np.asarray(vc, np.float64)
    for r in range(R):
        for h in range(heads):
            g = h // G
            qv = np.asarray(q[r, h * hd:(h + 1) * hd], np.float64)
            keys = np.concatenate([kc[:, g, :], np.asarray(knew[r, g * hd:(g + 1) * hd], np.float64)[None]], 0)
            vals = np.concatenate([vc[:, g, :], np.asarray(vnew[r, g * hd:(g + 1) * hd], np.float64)[None]], 0)
            s = keys @ qv / np.sqrt(hd)
            p = np.exp(s - s.max())
            out[r, h * hd:(h + 1) * hd] = (p / p.sum()) @ vals
    return out


def stack_logits(tokens, embed_bf16, head_bf16, layers, heads, kv_heads, hd, top_k, embed_q8=None, head_q8=None):
    """layers: list of dicts with q, k, v, o (opref_port.Exl3Linear), view (object with router, sgate, expert(e), shared as
    tests/helpers.MoeView), kc, vc (float16 [T, kv_heads, hd]). embed_q8 / head_q8: (weight u32, scales, biases) of an
    8-bit affine table instead of the bf16 one. Returns float64 logits [R, vocab]."""
    if embed_q8 is not None:
        x = O.q8_embed(tokens, *embed_q8).astype(np.float64)
    else:
        x = O.bf16_bits_to_f32(embed_bf16)[np.asarray(tokens)].astype(np.float64)
    y = None
    for L in layers:
        if y is not None:
            x = x + y
        xn = rms(x)
        q, k, v = (xn @ L[n].dense.astype(np.float64) for n in ("q", "k", "v"))
        att = attn_standin(q, k, v, L["kc"], L["vc"], heads, kv_heads, hd)
        x = x + att @ L["o"].dense.astype(np.float64)
        xn = rms(x)
        vw = L["view"]
        y = O.moe_block_exact(xn.astype(np.float32), vw.router, vw.sgate, vw.expert, vw.shared, top_k)["out"].astype(np.float64)
    xn = rms(x + y)
    if head_q8 is not None:  # the 8-bit head multiplies the f32 activations
        return xn.astype(np.float32).astype(np.float64) @ O.affine_dequant(*head_q8).astype(np.float64).T
    xb = O.bf16_bits_to_f32(O.f32_to_bf16_bits(xn.astype(np.float32))).astype(np.float64)  # the head multiplies bf16 activations
    return xb @ O.bf16_bits_to_f32(head_bf16).astype(np.float64).T


def kl(p_logits, q_logits):
    """KL(softmax(p) || softmax(q)) per row"""
    p = np.asarray(p_logits, np.float64)
    q = np.asarray(q_logits, np.float64)
    lp = p - p.max(-1, keepdims=True)
    lp = lp - np.log(np.exp(lp).sum(-1, keepdims=True))
    lq = q - q.max(-1, keepdims=True)
    lq = lq - np.log(np.exp(lq).sum(-1, keepdims=True))
    return (np.exp(lp) * (lp - lq)).sum(-1)
