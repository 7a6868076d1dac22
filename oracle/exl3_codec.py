"""CPU restatement of the EXL3 trellis codec (MCG codebook, window 15). TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this module; the
product path (ijah_b200/) never does.

The reference's numpy tools call a module named `exl3_codec` that ships neither with the reference nor on any package
index (tools/refenv.py:5-8 calls it "not part of this repository"; upstream lineage: exllamav3 and sushi, both MIT).
This file is a clean-room module with the same names (decode_inner, reconstruct, H128, lut, PERM, CODEBOOK_SCALE,
tiles_from_inner, pack_codewords, viterbi_tiles is NOT provided: it is encoder-only) so that the reference's own
tools/opref.py and tools/convert_trunk_enc.py import and run unmodified on top of it.

PARITY UNPINNED for the bit layout: the reference holds no golden vector or known-answer test for the codec. What pins
this restatement instead: (1) it is written from the two device readers of the reference (kernels/ne_common.h:105-161,
kernels/trunk6/trunk6.metal:87-127), and tests/test_oracle_codec.py holds literal restatements of both readers and
checks that all three agree on every slot for K = 4..8; (2) the value statistics the reference's notes quote for the
codebook hold (all 2^15 values finite, |v| <= 3.9492, std 1.2435).

Format (one 16x16 tile of W' = 16*K u16 = 8*K little-endian u32 words):
  ring    the 8K words concatenated MSB-first form a tail-biting ring of TOT = 256*K bits
  slot t  (t = 0..255) reads the 16 bits that END at ring bit (t+1)*K, i.e. bits [(t+1)K-16, (t+1)K) mod TOT;
          only the low 15 bits are the codeword (kernels/ne_common.h:139-141 `cw &= 0x7FFF`)
  value   r = ((cw * 0xCBAC1FED mod 2^32) & 0x8FFF8FFF) ^ 0x3B603B60; value = fp16(lo16(r)) + fp16(hi16(r)) computed
          in half precision, round-to-nearest-even (kernels/ne_common.h:139-144)
  place   slot t = 8*lane + j, q = lane & 3, c = lane >> 2: row = (2q, 2q+1, 2q+8, 2q+9)[j & 3], col = c + 8*(j >> 2)
          (kernels/ne_common.h:107-108)
"""
import numpy as np

CODEBOOK_SCALE = 1.24371088  # encoder-side normaliser (std of the codebook); not used on the decode path
WINDOW = 15
_MUL = np.uint32(0xCBAC1FED)
_MASK = np.uint32(0x8FFF8FFF)
_XOR = np.uint32(0x3B603B60)


def _slot_positions():
    t = np.arange(256)
    lane, j = t >> 3, t & 7
    q, c = lane & 3, lane >> 2
    rows = np.stack([2 * q, 2 * q + 1, 2 * q + 8, 2 * q + 9], 1)[np.arange(256), j & 3]
    cols = c + 8 * (j >> 2)
    return rows, cols


SLOT_ROW, SLOT_COL = _slot_positions()
PERM = (SLOT_ROW * 16 + SLOT_COL).astype(np.int64)  # slot -> row-major position inside the 16x16 tile


def mcg_value(cw, rounded=True):
    """codewords (any int array; low 15 bits used) -> float16 values, exactly as the device decoder produces them;
    rounded=False: the exact float32 sum of the two float16 summands (what a product that takes both summands as
    separate terms accumulates: the CUDA decode kernels)"""
    cw = (np.asarray(cw).astype(np.uint32)) & np.uint32(0x7FFF)
    r = ((cw * _MUL) & _MASK) ^ _XOR  # uint32 arithmetic wraps
    lo = (r & np.uint32(0xFFFF)).astype(np.uint16).view(np.float16)
    hi = (r >> np.uint32(16)).astype(np.uint16).view(np.float16)
    # the exact sum of two halfs with exponents this close fits a float32; one rounding to half = RN-even half add
    s = lo.astype(np.float32) + hi.astype(np.float32)
    return s.astype(np.float16) if rounded else s


_LUT = {}


def lut(codebook="mcg", window=WINDOW, rounded=True):
    """float16 [2^16]: value of every 16-bit window (the top bit is ignored, so the table repeats after 2^15);
    rounded=False: float32, the unrounded sums"""
    assert codebook == "mcg" and window == WINDOW, (codebook, window)
    if rounded not in _LUT:
        _LUT[rounded] = mcg_value(np.arange(1 << 16, dtype=np.uint32), rounded)
    return _LUT[rounded]


def tile_codewords(trellis):
    """trellis u16 [..., 16K] -> 16-bit windows u16 [..., 256] in slot order"""
    tr = np.ascontiguousarray(trellis, dtype=np.uint16)
    n = tr.shape[-1]
    assert n % 16 == 0 and 1 <= n // 16 <= 8, n
    K = n // 16
    lead = tr.shape[:-1]
    words = tr.reshape(-1, n).view("<u4")  # [T, 8K] little-endian u32 from the u16 halfwords
    T = words.shape[0]
    out = np.empty((T, 256), np.uint16)
    tot = 256 * K
    pos = ((np.arange(256)[:, None] + 1) * K - 16 + np.arange(16)[None, :]) % tot  # [256, 16] ring bit indices
    wts = (1 << np.arange(15, -1, -1)).astype(np.uint32)
    step = 4096
    for t0 in range(0, T, step):
        w = words[t0:t0 + step]
        bits = np.unpackbits(w.astype(">u4").view(np.uint8).reshape(w.shape[0], -1), axis=1)  # MSB-first ring
        out[t0:t0 + step] = (bits[:, pos].astype(np.uint32) * wts).sum(-1).astype(np.uint16)
    return out.reshape(*lead, 256)


def decode_tiles(trellis, rounded=True):
    """trellis u16 [..., 16K] -> float16 [..., 256] values in slot order (rounded=False: float32 unrounded sums)"""
    return lut(rounded=rounded)[tile_codewords(trellis)]


def decode_inner(trellis, n=None, codebook="mcg", window=WINDOW, rounded=True):
    """trellis u16 [in/16, out/16, 16K] -> W' float32 [in, out] (values are exact float16 numbers; rounded=False: the
    unrounded sums of the two summands)"""
    assert codebook == "mcg" and int(window) == WINDOW, (codebook, window)
    tr = np.asarray(trellis)
    assert tr.ndim == 3 and (n is None or n == tr.shape[-1])
    it, ot = tr.shape[:2]
    v = decode_tiles(tr, rounded)  # [it, ot, 256] slot order
    tiles = np.empty((it, ot, 256), v.dtype)
    tiles[:, :, PERM] = v
    return tiles.reshape(it, ot, 16, 16).transpose(0, 2, 1, 3).reshape(it * 16, ot * 16).astype(np.float32)


def tiles_from_inner(inner):
    """W' [in, out] -> (tiles [in/16 * out/16, 256] in slot order, (in/16, out/16))"""
    w = np.asarray(inner)
    k, m = w.shape
    t = w.reshape(k // 16, 16, m // 16, 16).transpose(0, 2, 1, 3).reshape(-1, 256)
    return t[:, PERM], (k // 16, m // 16)


def pack_codewords(cws, n):
    """codewords u16 [..., 256] (slot order; a valid tail-biting sequence: the top 16-K bits of cw[t+1] equal the low
    16-K bits of cw[t]) -> trellis u16 [..., n], n = 16K. Slot t contributes its low K bits at ring bits [tK, (t+1)K)."""
    cw = np.asarray(cws).astype(np.uint32)
    K = n // 16
    lead = cw.shape[:-1]
    cw = cw.reshape(-1, 256)
    sh = np.arange(K - 1, -1, -1, dtype=np.uint32)
    bits = ((cw[:, :, None] >> sh) & 1).astype(np.uint8).reshape(cw.shape[0], 256 * K)  # MSB-first ring
    words = np.packbits(bits, axis=1).view(">u4").astype("<u4")  # [T, 8K]
    return words.view(np.uint16).reshape(*lead, n)


def _had(n):
    i = np.arange(n)
    x = i[:, None] & i[None, :]
    pc = np.zeros((n, n), np.int64)
    while x.any():
        pc += x & 1
        x = x >> 1
    return np.where(pc % 2 == 0, 1.0, -1.0) / np.sqrt(n)


H128 = _had(128)


def had_size(d):
    for n in (128, 64, 32, 16):
        if d % n == 0:
            return n
    raise ValueError(d)


def reconstruct(inner, suh, svh):
    """W [in, out] float64 = diag(suh) H_in W' H_out diag(svh), H = block-diagonal normalised Sylvester Hadamard of
    size had_size(dim) (tools/convert_trunk_enc.py:59-63,125-129)."""
    q = np.asarray(inner, np.float64)
    k, m = q.shape
    hk, hm = had_size(k), had_size(m)
    w = np.einsum("ij,bjm->bim", _had(hk), q.reshape(k // hk, hk, m)).reshape(k, m)
    w = w * np.asarray(suh, np.float64)[:, None]
    w = (w.reshape(k, m // hm, hm) @ _had(hm)).reshape(k, m)
    return w * np.asarray(svh, np.float64)[None, :]
