"""The CPU restatement of the decoder stack's glue ops (oracle/stack_port.py): RMS norm, the attention stand-in, KL."""
import numpy as np

from oracle import stack_port as S


def test_rms_and_kl():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 64))
    y = S.rms(x)
    assert np.allclose((y * y).mean(-1), 1.0, atol=1e-5)
    assert np.allclose(S.kl(x, x), 0.0) and (S.kl(x, x + rng.standard_normal(x.shape) * 0.1) > 0).all()
    assert np.allclose(S.kl(x, x + 3.0), 0.0, atol=1e-12), "a constant shift of the logits is not a difference"


def test_attention_standin_is_a_softmax_over_cache_and_self():
    rng = np.random.default_rng(1)
    heads, kvh, hd, T = 4, 2, 8, 16
    q = rng.standard_normal((2, heads * hd))
    k, v = rng.standard_normal((2, kvh * hd)), rng.standard_normal((2, kvh * hd))
    kc, vc = rng.standard_normal((T, kvh, hd)).astype(np.float16), rng.standard_normal((T, kvh, hd)).astype(np.float16)
    out = S.attn_standin(q, k, v, kc, vc, heads, kvh, hd)
    # head 3 of row 1 uses KV head 1
    keys = np.concatenate([kc[:, 1].astype(np.float64), k[1, hd:2 * hd][None]])
    vals = np.concatenate([vc[:, 1].astype(np.float64), v[1, hd:2 * hd][None]])
    s = keys @ q[1, 3 * hd:4 * hd] / np.sqrt(hd)
    w = np.exp(s - s.max())
    assert np.allclose(out[1, 3 * hd:4 * hd], (w / w.sum()) @ vals)
    # a query that matches one cached key far better than the rest returns (almost) that position's value
    q2 = np.zeros((1, heads * hd))
    q2[0, :hd] = kc[5, 0].astype(np.float64) * 50
    o2 = S.attn_standin(q2, k[:1], v[:1], kc, vc, heads, kvh, hd)
    assert np.allclose(o2[0, :hd], vc[5, 0].astype(np.float64), atol=1e-3)
