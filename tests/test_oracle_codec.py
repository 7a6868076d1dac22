"""The codec oracle against restatements of the reference's device readers (CPU only).

Three readers exist in the reference: the K = 4..6 expert reader (kernels/ne_common.h:109-157: lane_load, lane_funnel,
win_off, cw_at, dec8), the any-K trunk reader (kernels/trunk6/trunk6.metal:91-127: t6_lane, t6_load, t6_dec) and the
prefill reader that feeds the matrix unit (kernels/prefill/pf_moe.metal:164-222: exl3_window, nax_wfrag, nax_quads,
nax_wfrag_k). All three are restated below step by step in scalar Python with 32- / 64-bit wrap-around; the oracle's ring
formula must give the same codeword for every slot of random tiles. The reference holds no known-answer vector for the
codec, so three readers written independently of each other agreeing with one formula is the pin there is.
"""
import numpy as np
import pytest

from oracle import exl3_codec as X

M32 = 0xFFFFFFFF


def _cw_at(vx, vy, E):
    c = 64 - E
    if c >= 32:
        return (vx >> (c - 32)) & 0xFFFF
    if c <= 16:
        return (vy >> c) & 0xFFFF
    return (((vx << (32 - c)) & M32) | (vy >> c)) & 0xFFFF


def reader_expert(words, K):
    """ne_common.h lane_load + lane_funnel + dec8's codeword extraction: 256 16-bit windows in slot order"""
    NW, TOT = 8 * K, 256 * K
    out = []
    for lane in range(32):
        s = 8 * K * lane + TOT + K - 16
        s = s - TOT if s >= TOT else s
        i0 = s >> 5
        i1 = i0 + 1 - NW if i0 + 1 >= NW else i0 + 1
        if (8 * K) % 32 == 0:
            vx, vy = int(words[i0]), int(words[i1])
            off = (256 * K + K - 16) & 31
        else:
            i2 = i1 + 1 - NW if i1 + 1 >= NW else i1 + 1
            a = (8 * K * lane + TOT + K - 16) & 31
            w0, w1, w2 = int(words[i0]), int(words[i1]), int(words[i2])
            vx = ((w0 << a) & M32) | ((w1 >> 1) >> (31 - a))
            vy = ((w1 << a) & M32) | ((w2 >> 1) >> (31 - a))
            off = 0
        for p in range(8):
            out.append(_cw_at(vx, vy, off + 16 + p * K))
    return np.array(out, np.uint32)


def reader_trunk(words, K):
    """trunk6.metal t6_lane + t6_dec's codeword extraction (low 15 bits are what it decodes)"""
    NW, TOT = 8 * K, 256 * K
    out = []
    for ln in range(32):
        s = (8 * ln + 1) * K + TOT - 15
        s = s - TOT if s >= TOT else s
        i0 = s >> 5
        i1 = i0 + 1 - NW if i0 + 1 >= NW else i0 + 1
        i2 = i1 + 1 - NW if i1 + 1 >= NW else i1 + 1
        a = s & 31
        w0, w1, w2 = int(words[i0]), int(words[i1]), int(words[i2])
        for j in range(8):
            if K == 8:
                E = 40 + 8 * j
                cw = _cw_at(w0, w1, E) if E <= 64 else _cw_at(w1, w2, E - 32)
            else:
                vx = ((w0 << a) & M32) | ((w1 >> 1) >> (31 - a))
                vy = ((w1 << a) & M32) | ((w2 >> 1) >> (31 - a))
                cw = _cw_at(vx, vy, j * K + 15)
            out.append(cw)
    return np.array(out, np.uint32)


M64 = 0xFFFFFFFFFFFFFFFF


def _exl3_window(words, end, nwords, full):
    """pf_moe.metal exl3_window: the bits that end at ring bit `end`, right-aligned (64 bits, or 96 folded when `full`)"""
    last = (end - 1) >> 5
    prev = nwords - 1 if last == 0 else last - 1
    s = (0 - end) & 31
    bits = (((int(words[prev]) << 32) | int(words[last])) & M64) >> s
    if full:
        pp = nwords - 1 if prev == 0 else prev - 1
        bits |= (((int(words[pp]) << 32) & M64) << (32 - s)) & M64
    return bits


def reader_prefill(words, K):
    """pf_moe.metal nax_wfrag_k<N = 16K> for the 32 lanes: (slot, 16-bit window) pairs in the order the fragment holds them.
    Lane l's fragment holds slots base + (0, 1, 8, 9, 4, 5, 12, 13), base = 128 (l >> 4) + 16 (l & 7) + 2 ((l >> 3) & 1)."""
    N = 16 * K
    W = N // 2
    end_of = lambda b, j: ((2 * b + j + 1) * N) >> 4  # nax_end
    out = []
    for lane in range(32):
        b = (lane >> 3) & 1
        base = 128 * (lane >> 4) + 16 * (lane & 7) + 2 * b
        if N == 64:  # nax_wfrag: K = 4, eight 4-bit steps per word
            source0 = (lane & 16) + ((lane & 7) << 1)
            cx, cy = int(words[source0]), int(words[source0 + 1])
            previous = int(words[(source0 + 31) & 31])
            slot = b * 2
            w0, w1 = (previous << 32) | cx, (cx << 32) | cy
            s0, s1 = 28 - slot * 4, 28 - (slot + 4) * 4
            cws = [(w0 >> s0) & 0xFFFF, (w0 >> (s0 - 4)) & 0xFFFF, (w1 >> s0) & 0xFFFF, (w1 >> (s0 - 4)) & 0xFFFF,
                   (w0 >> s1) & 0xFFFF, (w0 >> (s1 - 4)) & 0xFFFF, (w1 >> s1) & 0xFFFF, (w1 >> (s1 - 4)) & 0xFFFF]
        else:
            end = 8 * N * (lane >> 4) + N * (lane & 7) + (end_of(1, 5) - end_of(0, 5)) * b + end_of(0, 5)
            sh = lambda j: (end_of(0, 5) - end_of(0, j)) + b * ((end_of(1, 5) - end_of(1, j)) - (end_of(0, 5) - end_of(0, j)))  # nax_sh
            s0, s1, s4 = sh(0), sh(1), sh(4)
            fit = end_of(0, 5) - end_of(0, 0) <= 16 and end_of(1, 5) - end_of(1, 0) <= 16  # nax_quads_fit
            lo, hi = _exl3_window(words, end, W, not fit), _exl3_window(words, end + W, W, not fit)
            if fit:
                lo, hi = lo & M32, hi & M32
            q = lambda v: [(v >> s0) & 0xFFFF, (v >> s1) & 0xFFFF, (v >> s4) & 0xFFFF, v & 0xFFFF]
            p01, p23 = q(lo), q(hi)  # nax_quads: p0 = (s0, s1), p1 = (s4, 0) of lo; p2, p3 the same of hi
            cws = [p01[0], p01[1], p23[0], p23[1], p01[2], p01[3], p23[2], p23[3]]
        for off, cw in zip((0, 1, 8, 9, 4, 5, 12, 13), cws):
            out.append((base + off, cw))
    return out


def dec_mcg_scalar(cw):
    """ne_common.h dec_mcg for one codeword, half-precision add via numpy float16"""
    cw &= 0x7FFF
    r = (((cw * 0xCBAC1FED) & M32) & 0x8FFF8FFF) ^ 0x3B603B60
    lo = np.array([r & 0xFFFF], np.uint16).view(np.float16)[0]
    hi = np.array([r >> 16], np.uint16).view(np.float16)[0]
    return np.float16(lo + hi)


@pytest.mark.parametrize("K", [4, 5, 6, 7, 8])
def test_ring_formula_matches_both_device_readers(K):
    rng = np.random.default_rng(100 + K)
    for _ in range(4):
        tr = rng.integers(0, 1 << 16, 16 * K, dtype=np.uint16)
        words = tr.view("<u4")
        mine = X.tile_codewords(tr).astype(np.uint32)
        b = reader_trunk(words, K)
        assert np.array_equal(mine & 0x7FFF, b & 0x7FFF)
        if K <= 6:
            a = reader_expert(words, K)
            assert np.array_equal(mine, a)
        c = reader_prefill(words, K)
        assert sorted(slot for slot, _ in c) == list(range(256)), "the 32 fragments cover every slot once"
        for slot, cw in c:
            assert (cw & 0x7FFF) == (int(mine[slot]) & 0x7FFF), (K, slot)


def test_codebook_values_and_statistics():
    v = X.lut()[: 1 << 15].astype(np.float64)
    assert np.isfinite(v).all()
    assert abs(np.abs(v).max() - 3.9492) < 1e-3
    assert abs(v.std() - 1.2435) < 1e-3 and abs(v.mean()) < 0.01
    rng = np.random.default_rng(0)
    for cw in rng.integers(0, 1 << 16, 200):
        assert X.lut()[cw] == dec_mcg_scalar(int(cw))
    assert np.array_equal(X.lut()[: 1 << 15], X.lut()[1 << 15:])


def test_slot_placement():
    # lane l = 4c + q owns rows (2q, 2q+1, 2q+8, 2q+9) of column c (slots 0..3) and column c + 8 (slots 4..7)
    assert sorted(X.PERM.tolist()) == list(range(256))
    for lane in (0, 5, 31):
        q, c = lane & 3, lane >> 2
        for j in range(8):
            r = (2 * q, 2 * q + 1, 2 * q + 8, 2 * q + 9)[j & 3]
            assert X.PERM[8 * lane + j] == r * 16 + c + 8 * (j >> 2)


@pytest.mark.parametrize("K", [4, 5, 6, 8])
def test_pack_roundtrip_and_inner_layout(K):
    rng = np.random.default_rng(K)
    it, ot = 3, 2
    tr = rng.integers(0, 1 << 16, (it, ot, 16 * K), dtype=np.uint16)
    cw = X.tile_codewords(tr)
    assert np.array_equal(X.pack_codewords(cw, 16 * K), tr)  # every bit pattern is a valid tail-biting ring
    inner = X.decode_inner(tr, 16 * K)
    assert inner.shape == (it * 16, ot * 16)
    tiles, (a, b) = X.tiles_from_inner(inner)
    assert (a, b) == (it, ot)
    assert np.array_equal(tiles.reshape(it, ot, 256), X.decode_tiles(tr).astype(np.float32))
    # tile (tk, tn) covers W'[16 tk.., 16 tn..]
    v = X.decode_tiles(tr[1, 1])
    assert inner[16 + X.SLOT_ROW[37], 16 + X.SLOT_COL[37]] == np.float32(v[37])


def test_reconstruct_is_rotation_of_inner():
    rng = np.random.default_rng(3)
    inner = rng.standard_normal((256, 48))
    suh = rng.choice([-1.0, 1.0], 256)
    svh = rng.standard_normal(48)
    W = X.reconstruct(inner, suh, svh)
    x = rng.standard_normal((2, 256))
    y = ((x * suh).reshape(2, 2, 128) @ X.H128).reshape(2, 256) @ inner
    y = (y.reshape(2, 3, 16) @ X._had(16)).reshape(2, 48) * svh
    assert np.allclose(x @ W, y, atol=1e-10)
