// EXL3 trellis tile decode (MCG codebook, window 15) for sm_100a, register level.
//
// Format (reference: kernels/ne_common.h:105-161, kernels/trunk6/trunk6.metal:87-127): a 16x16 tile of W' is 8K
// little-endian u32 words read MSB-first as a tail-biting ring of 256K bits; slot t's codeword is the 15 bits that end
// at ring bit (t+1)K. Lane l of a warp owns slots 8l..8l+7 = rows (2q, 2q+1, 2q+8, 2q+9) of column c (slots 0-3)
// and of column c+8 (slots 4-7), q = l & 3, c = l >> 2 -- exactly the per-thread B fragment of two
// mma.m16n8k16 (k x n = 16 x 8) instructions, so decoded pairs go to the tensor core with no shuffle.
//
// A lane's 8 codewords span 15 + 7K bits starting at ring bit (8l+1)K - 15: three words cover it. For K = 5, 6, 7 the
// start bit inside the first word depends on the lane, so the window is first left-aligned with two funnel shifts;
// for K = 4 and 8 it is the same for all lanes and every field position is a compile-time constant.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace ijah {

template <int K>
struct Codec {
  static_assert(K >= 4 && K <= 8, "EXL3 bits per weight");
  static constexpr int NW = 8 * K;             // u32 words per tile
  static constexpr int TOT = 256 * K;          // ring bits
  static constexpr int TILE_BYTES = 32 * K;
  static constexpr bool UNIFORM = (8 * K) % 32 == 0;  // K = 4, 8: lane-independent bit offset
  static constexpr int A0 = (K + TOT - 15) & 31;      // that offset (start bit of lane 0's window inside its word)

  struct Lane {
    uint32_t o0, o1, o2;  // byte offsets of the window's three words inside the tile
    uint32_t a;           // start bit inside word 0
  };
  static __device__ __forceinline__ Lane lane(int ln) {
    uint32_t s = (8u * ln + 1u) * K + TOT - 15u;
    s = s >= (uint32_t)TOT ? s - TOT : s;
    const uint32_t i0 = s >> 5;
    const uint32_t i1 = i0 + 1 >= (uint32_t)NW ? i0 + 1 - NW : i0 + 1;
    const uint32_t i2 = i1 + 1 >= (uint32_t)NW ? i1 + 1 - NW : i1 + 1;
    return Lane{i0 * 4u, i1 * 4u, i2 * 4u, s & 31u};
  }
};

// Powers of two in constant memory. A left shift written as a multiply by one of these becomes an IMAD with a
// constant-bank operand, i.e. runs on the FMA pipe; the ALU pipe (shifts, logic ops, byte permutes: 64 lanes per
// clock per SM on B200, half the issue rate) is what bounds the decode, so every op moved off it counts.
static __constant__ uint32_t kPow2[32] = {
    1u << 0,  1u << 1,  1u << 2,  1u << 3,  1u << 4,  1u << 5,  1u << 6,  1u << 7,  1u << 8,  1u << 9,  1u << 10,
    1u << 11, 1u << 12, 1u << 13, 1u << 14, 1u << 15, 1u << 16, 1u << 17, 1u << 18, 1u << 19, 1u << 20, 1u << 21,
    1u << 22, 1u << 23, 1u << 24, 1u << 25, 1u << 26, 1u << 27, 1u << 28, 1u << 29, 1u << 30, 1u << 31};

// The two constants of the codebook function, read from constant memory into registers once per kernel (McgConst::load).
// Written as immediates, (r & A) ^ X compiles to TWO logic instructions per weight (an instruction encodes one
// immediate); as register operands of one three-input lop3 it is one.
static __constant__ uint32_t kMcgMaskXor[2] = {0x8FFF8FFFu, 0x3B603B60u};
struct McgConst {
  uint32_t mask, flip;
  static __device__ __forceinline__ McgConst load() { return McgConst{kMcgMaskXor[0], kMcgMaskXor[1]}; }
};

// 15-bit field whose first bit is `off` bits below the MSB of `w` (off + 15 <= 32): shift it to the top with a
// multiply (FMA pipe), then >> 17.
template <int off>
__device__ __forceinline__ uint32_t top15(uint32_t w) {
  static_assert(off >= 0 && off + 15 <= 32, "field must lie inside the word");
  if constexpr (off == 0) return w >> 17;
  else return (w * kPow2[off]) >> 17;
}

// 15-bit field starting P bits below the MSB of the 96-bit value (w0:w1:w2), P a compile-time constant. A field that
// straddles two words is read from `mid` = bits [16, 48) of the value when MID is set (one byte permute serves every
// straddling field of the tile), else through a funnel shift of its own.
template <int P, bool MID>
__device__ __forceinline__ uint32_t field15(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t mid) {
  constexpr int wi = P / 32, off = P % 32;
  if constexpr (off + 15 <= 32) {
    return top15<off>(wi == 0 ? w0 : (wi == 1 ? w1 : w2));
  } else if constexpr (MID && wi == 0) {
    return top15<P - 16>(mid);
  } else {
    const uint32_t hi = wi == 0 ? w0 : w1, lo = wi == 0 ? w1 : w2;
    return __funnelshift_l(lo, hi, off) >> 17;
  }
}

// two codewords -> half2(value(ca), value(cb)); value = fp16(lo16(r)) + fp16(hi16(r)), r = ((cw * M) & A) ^ X.
// One multiply and one three-input logic op per codeword, two half adds (the halves are selected by operand
// modifiers of the add), one pack.
__device__ __forceinline__ uint32_t mcg_pair(uint32_t ca, uint32_t cb, const McgConst &c) {
  uint32_t ra = ca * 0xCBAC1FEDu, rb = cb * 0xCBAC1FEDu;
  asm("lop3.b32 %0, %0, %1, %2, 0x6A;" : "+r"(ra) : "r"(c.mask), "r"(c.flip));  // (a & b) ^ c
  asm("lop3.b32 %0, %0, %1, %2, 0x6A;" : "+r"(rb) : "r"(c.mask), "r"(c.flip));
  const __half2 a = *reinterpret_cast<const __half2 *>(&ra), b = *reinterpret_cast<const __half2 *>(&rb);
  const __half2 r = __halves2half2(__hadd(__low2half(a), __high2half(a)), __hadd(__low2half(b), __high2half(b)));
  return *reinterpret_cast<const uint32_t *>(&r);
}

// one codeword -> the 32-bit word whose two fp16 halves add up to the weight (no add: see dec8_raw)
__device__ __forceinline__ uint32_t mcg_raw(uint32_t cw, const McgConst &c) {
  uint32_t r = cw * 0xCBAC1FEDu;
  asm("lop3.b32 %0, %0, %1, %2, 0x6A;" : "+r"(r) : "r"(c.mask), "r"(c.flip));  // (a & b) ^ c
  return r;
}

// The lane's 8 weights from its three window words: b[0] = (slot 0, slot 1), b[1] = (2, 3): column c;
// b[2] = (4, 5), b[3] = (6, 7): column c + 8. `a` = Codec<K>::Lane::a (ignored for K = 4, 8).
template <int K>
__device__ __forceinline__ void dec8(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t a, const McgConst &c, uint32_t (&b)[4]) {
  if constexpr (Codec<K>::UNIFORM) {
    constexpr int A = Codec<K>::A0;
    // K = 4: three fields straddle w0 | w1 and share the middle word; K = 8: one field per boundary, funnel shifts
    constexpr bool MID = K == 4;
    const uint32_t mid = MID ? __byte_perm(w0, w1, 0x1076) : 0u;  // (w0 << 16) | (w1 >> 16)
    b[0] = mcg_pair(field15<A + 0 * K, MID>(w0, w1, w2, mid), field15<A + 1 * K, MID>(w0, w1, w2, mid), c);
    b[1] = mcg_pair(field15<A + 2 * K, MID>(w0, w1, w2, mid), field15<A + 3 * K, MID>(w0, w1, w2, mid), c);
    b[2] = mcg_pair(field15<A + 4 * K, MID>(w0, w1, w2, mid), field15<A + 5 * K, MID>(w0, w1, w2, mid), c);
    b[3] = mcg_pair(field15<A + 6 * K, MID>(w0, w1, w2, mid), field15<A + 7 * K, MID>(w0, w1, w2, mid), c);
  } else {
    // K = 5, 6, 7: align the lane's window to bit 0 of x (two funnel shifts), then every field position is a constant;
    // the three fields that straddle x | y are read from the middle word
    const uint32_t x = __funnelshift_l(w1, w0, a), y = __funnelshift_l(w2, w1, a);
    const uint32_t mid = __byte_perm(x, y, 0x1076);
    b[0] = mcg_pair(field15<0 * K, true>(x, y, 0u, mid), field15<1 * K, true>(x, y, 0u, mid), c);
    b[1] = mcg_pair(field15<2 * K, true>(x, y, 0u, mid), field15<3 * K, true>(x, y, 0u, mid), c);
    b[2] = mcg_pair(field15<4 * K, true>(x, y, 0u, mid), field15<5 * K, true>(x, y, 0u, mid), c);
    b[3] = mcg_pair(field15<6 * K, true>(x, y, 0u, mid), field15<7 * K, true>(x, y, 0u, mid), c);
  }
}

// The same 8 slots left as their summand pairs: r[t] = (lo, hi) with weight = fp16(lo + hi). The stream kernels build the
// tensor-core operand from these words directly (one half add per word for the exact weight, none for the opt-in summand
// product), so the pack of dec8 (two weights per register) is not executed.
template <int K>
__device__ __forceinline__ void dec8_raw(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t a, const McgConst &c, uint32_t (&r)[8]) {
  if constexpr (Codec<K>::UNIFORM) {
    constexpr int A = Codec<K>::A0;
    constexpr bool MID = K == 4;
    const uint32_t mid = MID ? __byte_perm(w0, w1, 0x1076) : 0u;
    r[0] = mcg_raw(field15<A + 0 * K, MID>(w0, w1, w2, mid), c);
    r[1] = mcg_raw(field15<A + 1 * K, MID>(w0, w1, w2, mid), c);
    r[2] = mcg_raw(field15<A + 2 * K, MID>(w0, w1, w2, mid), c);
    r[3] = mcg_raw(field15<A + 3 * K, MID>(w0, w1, w2, mid), c);
    r[4] = mcg_raw(field15<A + 4 * K, MID>(w0, w1, w2, mid), c);
    r[5] = mcg_raw(field15<A + 5 * K, MID>(w0, w1, w2, mid), c);
    r[6] = mcg_raw(field15<A + 6 * K, MID>(w0, w1, w2, mid), c);
    r[7] = mcg_raw(field15<A + 7 * K, MID>(w0, w1, w2, mid), c);
  } else {
    const uint32_t x = __funnelshift_l(w1, w0, a), y = __funnelshift_l(w2, w1, a);
    const uint32_t mid = __byte_perm(x, y, 0x1076);
    r[0] = mcg_raw(field15<0 * K, true>(x, y, 0u, mid), c);
    r[1] = mcg_raw(field15<1 * K, true>(x, y, 0u, mid), c);
    r[2] = mcg_raw(field15<2 * K, true>(x, y, 0u, mid), c);
    r[3] = mcg_raw(field15<3 * K, true>(x, y, 0u, mid), c);
    r[4] = mcg_raw(field15<4 * K, true>(x, y, 0u, mid), c);
    r[5] = mcg_raw(field15<5 * K, true>(x, y, 0u, mid), c);
    r[6] = mcg_raw(field15<6 * K, true>(x, y, 0u, mid), c);
    r[7] = mcg_raw(field15<7 * K, true>(x, y, 0u, mid), c);
  }
}

// Layout of a prepared activation row (the B operand of the stream kernels) for that product: per k-tile of 16 inputs
// 32 halfs = 16 pairs in the order inputs 0, 2, .. 14, then 1, 3, .. 15, so that one ldmatrix.x4 of an 8-row group
// yields the even-input and the odd-input fragments. A row of n inputs is 2 n halfs. The pair is (v, 0) for the exact
// product (the kernel feeds (w, w), w = fp16(lo + hi): the accumulator receives w * v) and (v, v) for the summand
// product (the kernel feeds (lo, hi): lo * v + hi * v).
constexpr int A_HALFS_PER_INPUT = 2;
__device__ __forceinline__ void store_a(__half *row, int i, float v, int dup) {
  const int w = (i >> 4) * 16 + (i & 1) * 8 + ((i & 15) >> 1);
  const __half h = __float2half_rn(v);
  reinterpret_cast<__half2 *>(row)[w] = __halves2half2(h, dup ? h : __ushort_as_half((unsigned short)0));
}

// normalised Hadamard of size N (16..128) over a 128-element chunk held by a warp as (lane, lane+32, lane+64, lane+96);
// butterflies over index bits 0,1,2,... then one multiply by 1/sqrt(N) (reference: kernels/ne_common.h:95-103,
// kernels/trunk6/trunk6.metal:42-51). Blocks of N < 128 stay inside the chunk.
__device__ __forceinline__ void fwht_chunk(float (&v)[4], int lane, int N, float scale) {
#pragma unroll
  for (int bit = 1; bit < 32; bit <<= 1) {
    if (bit < N) {
      const float sgn = (lane & bit) == 0 ? 1.0f : -1.0f;  // lower partner: v + p, upper: p - v; one FMA, same rounding
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float p = __shfl_xor_sync(0xFFFFFFFFu, v[j], bit);
        v[j] = __fmaf_rn(v[j], sgn, p);
      }
    }
  }
  if (N >= 64) {
    const float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
    v[0] = a; v[1] = b; v[2] = c; v[3] = d;
  }
  if (N >= 128) {
    const float a = v[0] + v[2], b = v[1] + v[3], c = v[0] - v[2], d = v[1] - v[3];
    v[0] = a; v[1] = b; v[2] = c; v[3] = d;
  }
#pragma unroll
  for (int j = 0; j < 4; j++) v[j] *= scale;
}

// The same transform of size 128 with the chunk held as (4 lane .. 4 lane + 3) per lane, so that a lane reads and writes 16
// contiguous bytes. Same butterflies in the same order (index bits 0, 1 inside the lane, bits 2..6 across lanes), hence
// bit-identical to fwht_chunk.
__device__ __forceinline__ void fwht128_contig(float (&v)[4], int lane, float scale) {
  {
    const float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
    v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
  }
#pragma unroll
  for (int bit = 1; bit < 32; bit <<= 1) {
    const float sgn = (lane & bit) == 0 ? 1.0f : -1.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float p = __shfl_xor_sync(0xFFFFFFFFu, v[j], bit);
      v[j] = __fmaf_rn(v[j], sgn, p);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; j++) v[j] *= scale;
}

__host__ __device__ inline int had_size(int d) { return d % 128 == 0 ? 128 : d % 64 == 0 ? 64 : d % 32 == 0 ? 32 : 16; }

}  // namespace ijah
