// 8-bit affine Linear for decode widths: an HBM stream of weight bytes (one byte per weight; the LM head of the
// reference's model is 636 MB) into legacy tensor-core MMAs.
//
// One warp per 16 output rows, 8 warps per CTA. The tensor core computes D^T = Q X^T per group of `group` inputs: the bytes
// q (0..255, exact in fp16) are the A operand, streamed from global memory straight into fragments (each lane reads 8
// contiguous bytes of output rows g and g + 8 per 32 inputs; the order of the inputs inside such a step is permuted the
// same way for both operands, which a dot product does not mind), the activations the B operand. An activation x is
// used as hi + lo, hi = fp16(x), lo = fp16(x - hi): two MMAs per step, which keeps 22 bits of x, so the result agrees
// with f32 arithmetic to rounding. Per group: y += scale * (q . x) + bias * sum(x), in f32.
#include <cuda_fp16.h>

#include "common.hpp"
#include "launch.cuh"
#include "pipeline.cuh"
#include "q8_linear.cuh"

namespace ijah {
namespace {

constexpr int Q8_KC = 2560;  // inputs staged per chunk (the reference's hidden size; wider Linears take several chunks)
constexpr int Q8_PF = 4;     // 64-input steps whose weight bytes are in flight per lane (2 x 16 bytes each)

__device__ __forceinline__ float bf16f(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }

// bytes (b0, b1) of `u` selected by `sel` -> half2(b0, b1): 0x6400 | b is the half 1024 + b; subtracting 1024 is exact
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t u, uint32_t sel) {
  const uint32_t h = __byte_perm(u, 0x64646464u, sel);
  const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half((unsigned short)0x6400)));
  return *reinterpret_cast<const uint32_t *>(&r);
}

__host__ __device__ inline int q8_ldx(int kc) { return kc + 8; }  // halfs per staged row (+16 bytes: rows on distinct banks)
__host__ __device__ inline size_t q8_smem_bytes(int nt, int kc) { return (size_t)nt * 8 * q8_ldx(kc) * 2 * 2 + (size_t)nt * 8 * (kc / 32) * 4; }

// One warp per 16 output rows, 8 warps per CTA. Per chunk of up to Q8_KC inputs the activations are staged once (hi / lo
// halves, and their sums over 32 inputs); the loop over 64-input steps then has no barrier: every lane keeps Q8_PF steps of
// weight bytes in flight (16 bytes of row g and of row g + 8 per step: a warp reads whole 64-byte runs of 16 rows).
// Input order inside a step: MMA j of the step takes the lane's bytes 4j .. 4j+3, i.e. inputs 16 qq + 4j + {0,1} as the
// fragment's k pair (2qq, 2qq+1) and + {2,3} as (2qq+8, 2qq+9); the activation fragments are read with the same mapping.
template <int NT>
__global__ void __launch_bounds__(256, NT == 1 ? 2 : 1) q8_wide_kernel(const Q8Weight w, const float *__restrict__ x, int rows, float *__restrict__ y) {
  extern __shared__ __align__(16) unsigned char q8_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, qq = lane & 3;
  const int n_in = w.in, G = w.group, ng = n_in / G;
  const int o0 = (blockIdx.x * 8 + warp) * 16;
  const int r0 = min(o0 + g, w.rows - 1), r1 = min(o0 + g + 8, w.rows - 1);
  const uint8_t *w0 = w.w + (size_t)r0 * n_in + 16 * qq, *w1 = w.w + (size_t)r1 * n_in + 16 * qq;
  const uint16_t *s0 = w.scales + (size_t)r0 * ng, *s1 = w.scales + (size_t)r1 * ng;
  const uint16_t *b0 = w.biases + (size_t)r0 * ng, *b1 = w.biases + (size_t)r1 * ng;
  float tot[NT][4], acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; n++)
#pragma unroll
    for (int j = 0; j < 4; j++) tot[n][j] = acc[n][j] = 0.f;
  pdl_launch();
  for (int kb = 0; kb < n_in; kb += Q8_KC) {
    const int kc = min(Q8_KC, n_in - kb), nsteps = kc / 64;  // kc is a multiple of 64
    const int LDX = q8_ldx(min(Q8_KC, n_in));
    __half *xhi = reinterpret_cast<__half *>(q8_smem);
    __half *xlo = xhi + NT * 8 * LDX;
    float *gsum = reinterpret_cast<float *>(xlo + NT * 8 * LDX);  // [NT * 8][kc / 32]: sums of x over 32 inputs
    const int nsum = min(Q8_KC, n_in) / 32;
    // the chunk's first weight bytes are static data: in flight before the activations are staged (and, for the first
    // chunk, before the wait on the kernel that produces them)
    // ... and with them the scale / bias of the group each step belongs to (rows g and g + 8 packed in one register each):
    // loaded where they are used, these two-byte loads cost every step a full memory latency
    uint4 qa[Q8_PF], qb[Q8_PF];
    uint32_t qs[Q8_PF], qz[Q8_PF];
#pragma unroll
    for (int j = 0; j < Q8_PF; j++) {
      if (j < nsteps) {
        qa[j] = __ldcs(reinterpret_cast<const uint4 *>(w0 + kb + j * 64));
        qb[j] = __ldcs(reinterpret_cast<const uint4 *>(w1 + kb + j * 64));
        const int gi = (kb + j * 64) / G;
        qs[j] = (uint32_t)__ldg(s0 + gi) | ((uint32_t)__ldg(s1 + gi) << 16);
        qz[j] = (uint32_t)__ldg(b0 + gi) | ((uint32_t)__ldg(b1 + gi) << 16);
      }
    }
    if (kb == 0) pdl_wait();
    __syncthreads();  // the previous chunk's readers are done
    for (int i = threadIdx.x; i < NT * 8 * (kc / 32); i += 256) {
      const int r = i / (kc / 32), c = i % (kc / 32);
      float sum = 0.f;
      uint4 *dh = reinterpret_cast<uint4 *>(xhi + r * LDX + c * 32), *dl = reinterpret_cast<uint4 *>(xlo + r * LDX + c * 32);
      const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)r * n_in + kb + c * 32);
#pragma unroll
      for (int q = 0; q < 4; q++) {  // 8 inputs per turn
        uint32_t hi[4] = {0u, 0u, 0u, 0u}, lo[4] = {0u, 0u, 0u, 0u};
        if (r < rows) {
#pragma unroll
          for (int j = 0; j < 2; j++) {
            const float4 v = __ldcg(src + 2 * q + j);
            const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const __half2 l01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y), l23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
            const float2 g01 = __half22float2(l01), g23 = __half22float2(l23);
            sum += ((f01.x + g01.x) + (f01.y + g01.y)) + ((f23.x + g23.x) + (f23.y + g23.y));  // of the values the MMAs see
            hi[2 * j] = *reinterpret_cast<const uint32_t *>(&h01); hi[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&h23);
            lo[2 * j] = *reinterpret_cast<const uint32_t *>(&l01); lo[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&l23);
          }
        }
        dh[q] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        dl[q] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
      gsum[r * nsum + c] = sum;
    }
    __syncthreads();
    for (int sb = 0; sb < nsteps; sb += Q8_PF) {
#pragma unroll
      for (int j = 0; j < Q8_PF; j++) {
        const int st = sb + j;
        if (st < nsteps) {  // uniform
          const uint4 ua = qa[j], ub = qb[j];
          const uint32_t us = qs[j], uz = qz[j];
          if (st + Q8_PF < nsteps) {
            qa[j] = __ldcs(reinterpret_cast<const uint4 *>(w0 + kb + (st + Q8_PF) * 64));
            qb[j] = __ldcs(reinterpret_cast<const uint4 *>(w1 + kb + (st + Q8_PF) * 64));
            const int gi = (kb + (st + Q8_PF) * 64) / G;
            qs[j] = (uint32_t)__ldg(s0 + gi) | ((uint32_t)__ldg(s1 + gi) << 16);
            qz[j] = (uint32_t)__ldg(b0 + gi) | ((uint32_t)__ldg(b1 + gi) << 16);
          }
          const uint32_t wa4[4] = {ua.x, ua.y, ua.z, ua.w}, wb4[4] = {ub.x, ub.y, ub.z, ub.w};
          uint32_t fr[4][4];
#pragma unroll
          for (int m = 0; m < 4; m++) {
            fr[m][0] = bytes_to_half2(wa4[m], 0x4140); fr[m][1] = bytes_to_half2(wb4[m], 0x4140);
            fr[m][2] = bytes_to_half2(wa4[m], 0x4342); fr[m][3] = bytes_to_half2(wb4[m], 0x4342);
          }
#pragma unroll
          for (int n = 0; n < NT; n++) {
            const uint4 *ph = reinterpret_cast<const uint4 *>(xhi + (n * 8 + g) * LDX + st * 64 + 16 * qq);
            const uint4 *pl = reinterpret_cast<const uint4 *>(xlo + (n * 8 + g) * LDX + st * 64 + 16 * qq);
            const uint4 h0 = ph[0], h1 = ph[1], l0 = pl[0], l1 = pl[1];
            mma_16816(acc[n], fr[0], h0.x, h0.y); mma_16816(acc[n], fr[1], h0.z, h0.w);
            mma_16816(acc[n], fr[2], h1.x, h1.y); mma_16816(acc[n], fr[3], h1.z, h1.w);
            mma_16816(acc[n], fr[0], l0.x, l0.y); mma_16816(acc[n], fr[1], l0.z, l0.w);
            mma_16816(acc[n], fr[2], l1.x, l1.y); mma_16816(acc[n], fr[3], l1.z, l1.w);
          }
          const int k = kb + st * 64;
          // a group (64, 128 or 256 inputs) ends with this step, or with a later one
          if ((k + 64) % G == 0) {
            const float sc0 = __uint_as_float(us << 16), sc1 = __uint_as_float(us & 0xFFFF0000u);
            const float bi0 = __uint_as_float(uz << 16), bi1 = __uint_as_float(uz & 0xFFFF0000u);
            const int c0 = (k + 64 - G - kb) / 32, nc = G / 32;
#pragma unroll
            for (int n = 0; n < NT; n++) {
              float sa = 0.f, sbb = 0.f;  // sum of x over the group for activation rows 8 n + 2 qq and + 1
              for (int c = 0; c < nc; c++) {
                sa += gsum[(n * 8 + 2 * qq) * nsum + c0 + c];
                sbb += gsum[(n * 8 + 2 * qq + 1) * nsum + c0 + c];
              }
              tot[n][0] += sc0 * acc[n][0] + bi0 * sa;
              tot[n][1] += sc0 * acc[n][1] + bi0 * sbb;
              tot[n][2] += sc1 * acc[n][2] + bi1 * sa;
              tot[n][3] += sc1 * acc[n][3] + bi1 * sbb;
#pragma unroll
              for (int q = 0; q < 4; q++) acc[n][q] = 0.f;
            }
          }
        }
      }
    }
  }
  // tot[n]: (output row g, activation rows 8n + 2qq, +1), (output row g + 8, the same rows): transpose through shared memory
  __syncthreads();
  float(*outt)[NT * 8][17] = reinterpret_cast<float(*)[NT * 8][17]>(q8_smem);
#pragma unroll
  for (int n = 0; n < NT; n++) {
    outt[warp][n * 8 + 2 * qq][g] = tot[n][0];
    outt[warp][n * 8 + 2 * qq + 1][g] = tot[n][1];
    outt[warp][n * 8 + 2 * qq][g + 8] = tot[n][2];
    outt[warp][n * 8 + 2 * qq + 1][g + 8] = tot[n][3];
  }
  __syncwarp();
  for (int i = lane; i < rows * 16; i += 32) {
    const int r = i >> 4, c = i & 15;
    if (o0 + c < w.rows) y[(size_t)r * w.rows + o0 + c] = outt[warp][r][c];
  }
}

// ------------------------------------------------------------------------------------------------ the streaming form
// For Linears of up to Q8_KC inputs (the LM head, the embedding used as a tied head, the hyper-connection up matrix) and up
// to 8 activation rows: persistent CTAs (one per SM), each with one producer warp and eight consumer warps.
//   producer: per row block of 128 output rows the block's scales and biases (contiguous in memory: one bulk copy each into
//     one of two buffers), then per slab of 128 inputs ONE tiled TMA copy of 128 rows x 128 bytes with the 128-byte
//     swizzle into a ring of 16 KB stages (full / empty mbarriers, transaction counts);
//   consumer warp = 16 output rows: per pair of 16-input segments one ldmatrix.x4 on the swizzled stage (conflict-free,
//     each lane gets the 4 bytes of rows g and g + 8 that one MMA needs), bytes -> fp16 (exact), two MMAs per segment against
//     the hi and lo halves of the activations (one ldmatrix.x4; the activations were staged once per CTA, in the input order
//     the byte fragments imply), scale / bias per group in f32.
constexpr int Q8S_ROWS = 128, Q8S_SLAB = 128, Q8S_STAGE_BYTES = Q8S_ROWS * Q8S_SLAB, Q8S_MAX_STAGES = 8;  // (a multiple of Q8S_SETS)
// Consumer sets: set t takes every Q8S_SETS-th slab of the producer's sequence. One warp's work on a slab is a chain of
// dependent steps (barrier, ldmatrix, convert, MMA, scale) about 2000 cycles long during which it issues 150 instructions;
// with one set the SM idles on that latency, with several the chains overlap.
#ifndef Q8S_SETS
#define Q8S_SETS 2
#endif
constexpr int Q8S_CWARPS = 8 * Q8S_SETS, Q8S_THREADS = (Q8S_CWARPS + 1) * 32;

struct Q8StreamLayout {
  int stages, kpad, ldx, ng;
  __host__ __device__ size_t bar_off() const { return (size_t)stages * Q8S_STAGE_BYTES; }
  __host__ __device__ size_t x_off() const { return bar_off() + 256; }
  __host__ __device__ size_t gsum_off() const { return x_off() + (size_t)2 * 8 * ldx * 2; }
  __host__ __device__ size_t xch_off() const { return (gsum_off() + (size_t)8 * (kpad / 32) * 4 + 15) & ~(size_t)15; }
  __host__ __device__ size_t sc_off() const { return xch_off() + (size_t)2 * (Q8S_SETS - 1) * 8 * 32 * 16; }  // partial totals of sets 1.., two buffers
  __host__ __device__ size_t sc_buf_bytes() const { return ((size_t)2 * Q8S_ROWS * ng * 2 + 15) & ~(size_t)15; }  // scales, then biases
  __host__ __device__ size_t total() const { return sc_off() + 2 * sc_buf_bytes(); }
};

struct Q8StreamParams {
  alignas(64) CUtensorMap map;  // weight bytes [rows][in], box 128 x 128, 128-byte swizzle
  Q8Weight w;
  Q8StreamLayout lay;
  int nblocks;
};

// Staged activation rows hold each 16-input segment in the order the byte fragments imply: MMA k index 2 qq + e holds input
// 4 qq + e, k index 8 + 2 qq + e holds input 4 qq + 2 + e (the lane's four bytes are its fragment's two k pairs).

// F = min(group, 128): inputs per run with one scale / bias (a 256-input group is two runs with the same pair)
template <int F>
__global__ void __launch_bounds__(Q8S_THREADS, 1) q8_stream_kernel(const __grid_constant__ Q8StreamParams P, const float *__restrict__ x, int rows,
                                                                   float *__restrict__ y, int *status) {
  extern __shared__ __align__(16) unsigned char q8s_raw[];
  unsigned char *q8s = q8s_raw + ((1024u - (smem_u32(q8s_raw) & 1023u)) & 1023u);  // the swizzled stages want 1024-byte alignment
  const Q8StreamLayout &L = P.lay;
  uint64_t *full = reinterpret_cast<uint64_t *>(q8s + L.bar_off());
  uint64_t *empty = full + Q8S_MAX_STAGES;
  uint64_t *sfull = empty + Q8S_MAX_STAGES;  // [2] scale buffers
  uint64_t *sempty = sfull + 2;
  __half *xhi = reinterpret_cast<__half *>(q8s + L.x_off());
  __half *xlo = xhi + 8 * L.ldx;
  float *gsum = reinterpret_cast<float *>(q8s + L.gsum_off());
  float4 *xch = reinterpret_cast<float4 *>(q8s + L.xch_off());  // [2][SETS - 1][8 warps][32 lanes]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_in = P.w.in, ng = L.ng, nslabs = L.kpad / Q8S_SLAB;
  if (threadIdx.x == 0) {
    for (int i = 0; i < L.stages; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], 8); }
    for (int i = 0; i < 2; i++) { mbar_init(&sfull[i], 1); mbar_init(&sempty[i], Q8S_CWARPS); }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch();
  if (warp == Q8S_CWARPS) {
    // ---------------------------------------------------------------- producer
    const uint64_t pol = l2_evict_first_policy();
    uint32_t stage = 0, phase = 0;
    int sb = 0;
    uint32_t sphase = 0;
    for (int rb = blockIdx.x; rb < P.nblocks; rb += gridDim.x) {
      {  // the block's scales and biases
        if (!mbar_wait(&sempty[sb], sphase ^ 1u, status, 5)) return;
        const int nr = min(Q8S_ROWS, P.w.rows - rb * Q8S_ROWS);
        const uint32_t bytes = (uint32_t)nr * ng * 2, bulk = bytes & ~15u;
        unsigned char *dst = q8s + L.sc_off() + (size_t)sb * L.sc_buf_bytes();
        const unsigned char *ssrc = reinterpret_cast<const unsigned char *>(P.w.scales) + (size_t)rb * Q8S_ROWS * ng * 2;
        const unsigned char *bsrc = reinterpret_cast<const unsigned char *>(P.w.biases) + (size_t)rb * Q8S_ROWS * ng * 2;
        unsigned char *bdst = dst + (size_t)Q8S_ROWS * ng * 2;
        for (uint32_t i = bulk + 2 * lane; i < bytes; i += 64) {  // a tail shorter than 16 bytes (ragged row counts)
          *reinterpret_cast<uint16_t *>(dst + i) = *reinterpret_cast<const uint16_t *>(ssrc + i);
          *reinterpret_cast<uint16_t *>(bdst + i) = *reinterpret_cast<const uint16_t *>(bsrc + i);
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_expect_tx(&sfull[sb], 2 * bulk);
          if (bulk) {
            bulk_g2s(dst, ssrc, bulk, &sfull[sb]);
            bulk_g2s(bdst, bsrc, bulk, &sfull[sb]);
          }
        }
        sb ^= 1;
        if (sb == 0) sphase ^= 1u;
      }
      for (int sl = 0; sl < nslabs; sl++) {
        if (!mbar_wait(&empty[stage], phase ^ 1u, status, 1)) return;
        if (lane == 0) {
          mbar_arrive_expect_tx(&full[stage], Q8S_STAGE_BYTES);
          tma_load_2d(smem_u32(q8s + (size_t)stage * Q8S_STAGE_BYTES), &P.map, sl * Q8S_SLAB, rb * Q8S_ROWS, smem_u32(&full[stage]), pol);
        }
        if (++stage == (uint32_t)L.stages) { stage = 0; phase ^= 1u; }
      }
    }
    return;
  }
  // ------------------------------------------------------------------ consumers: stage the activations once
  pdl_wait();
  for (int i = threadIdx.x; i < 8 * (L.kpad / F); i += Q8S_CWARPS * 32) {  // one run of F inputs of one row per turn
    const int r = i / (L.kpad / F), c = i % (L.kpad / F);
    float sum = 0.f;
#pragma unroll
    for (int sgm = 0; sgm < F / 16; sgm++) {  // 16-input segments
      __half *dh = xhi + r * L.ldx + c * F + sgm * 16, *dl = xlo + r * L.ldx + c * F + sgm * 16;
      const int k0 = c * F + sgm * 16;
      uint32_t hw[8], lw[8];  // the segment in staged order, two halfs per word
#pragma unroll
      for (int q = 0; q < 4; q++) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows && k0 + 4 * q < n_in) v = __ldcg(reinterpret_cast<const float4 *>(x + (size_t)r * n_in + k0) + q);
        // inputs 4 q + {0, 1} sit at positions 2 q + {0, 1}, inputs 4 q + {2, 3} at 8 + 2 q + {0, 1}
        const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
        const __half2 l01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y), l23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
        const float2 g01 = __half22float2(l01), g23 = __half22float2(l23);
        sum += ((f01.x + g01.x) + (f01.y + g01.y)) + ((f23.x + g23.x) + (f23.y + g23.y));  // of the values the MMAs see
        hw[q] = *reinterpret_cast<const uint32_t *>(&h01); hw[4 + q] = *reinterpret_cast<const uint32_t *>(&h23);
        lw[q] = *reinterpret_cast<const uint32_t *>(&l01); lw[4 + q] = *reinterpret_cast<const uint32_t *>(&l23);
      }
      reinterpret_cast<uint4 *>(dh)[0] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
      reinterpret_cast<uint4 *>(dh)[1] = make_uint4(hw[4], hw[5], hw[6], hw[7]);
      reinterpret_cast<uint4 *>(dl)[0] = make_uint4(lw[0], lw[1], lw[2], lw[3]);
      reinterpret_cast<uint4 *>(dl)[1] = make_uint4(lw[4], lw[5], lw[6], lw[7]);
    }
    gsum[r * (L.kpad / F) + c] = sum;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(Q8S_CWARPS * 32) : "memory");  // the consumer warps
  const int set = warp >> 3, rw = warp & 7;  // consumer set, row group (16 output rows) inside the block
  const int g = lane >> 2, qq = lane & 3;
  const int nsum = L.kpad / F, gshift = P.w.group > F ? 1 : 0;  // runs per group: 1, or 2 for groups of 256
  // ldmatrix addresses. A (weight bytes, swizzled stage): lane i gives row 16 rw + (i & 7) + 8 ((i >> 3) & 1), 16-byte chunk
  // c + (i >> 4) of the slab, stored at chunk ^ (row & 7). B (activations): lanes 0-7 hi k 0-7, 8-15 hi k 8-15, 16-23 lo, 24-31 lo.
  const uint32_t a_rowoff = (uint32_t)((16 * rw + (lane & 7) + 8 * ((lane >> 3) & 1)) * Q8S_SLAB);
  const uint32_t a_sw = (uint32_t)(lane & 7), a_hi = (uint32_t)(lane >> 4);
  const uint32_t b_addr = smem_u32(lane < 16 ? xhi : xlo) + (uint32_t)(((lane & 7) * L.ldx + ((lane >> 3) & 1) * 8) * 2);
  const uint32_t ring = smem_u32(q8s);
  // position in the producer's slab sequence (all row blocks of this CTA): whose turn it is, ring stage and its parity
  int turn = 0;
  uint32_t stage = 0, phase = 0;
  int sb = 0, xb = 0;
  bool ok = true;  // false once a bounded wait gave up: the warp then only keeps its barrier appointments (results are void)
  uint32_t sphase = 0;
  for (int rb = blockIdx.x; rb < P.nblocks; rb += gridDim.x) {
    if (ok && !mbar_wait(&sfull[sb], sphase, status, 6)) ok = false;
    const uint16_t *scs = reinterpret_cast<const uint16_t *>(q8s + L.sc_off() + (size_t)sb * L.sc_buf_bytes());
    const uint16_t *bis = scs + (size_t)Q8S_ROWS * ng;
    const uint16_t *s0 = scs + (16 * rw + g) * ng, *s1 = s0 + 8 * ng, *z0 = bis + (16 * rw + g) * ng, *z1 = z0 + 8 * ng;
    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    for (int sl = 0; sl < nslabs; sl++) {
      const bool mine = turn == set;
      const uint32_t st = stage, ph = phase;
      if (++turn == Q8S_SETS) turn = 0;
      if (++stage == (uint32_t)L.stages) { stage = 0; phase ^= 1u; }
      if (!mine) continue;  // another set's slab
      if (ok && !mbar_wait_a(smem_u32(&full[st]), ph, status, 2)) ok = false;
      if (!ok) continue;
#ifndef Q8S_SKIP
      const uint32_t sbase = ring + st * (uint32_t)Q8S_STAGE_BYTES + a_rowoff;
      uint32_t a[4][4];
#pragma unroll
      for (int c = 0; c < 8; c += 2) ldmatrix_x4(a[c >> 1], sbase + (((uint32_t)c + a_hi) ^ a_sw) * 16u);
      // the warp's share of the slab is in registers: hand the stage back now (the arrive is made to depend on the loaded
      // values), so that the ring is refilled while the MMAs run instead of after them
      asm volatile("" ::"r"(a[0][0]), "r"(a[1][0]), "r"(a[2][0]), "r"(a[3][0]) : "memory");
      if (lane == 0) mbar_arrive(&empty[st]);
      // one accumulator per 32 inputs (four chained MMAs: two segments x hi, lo), started from zero by its first MMA
      float acc[4][4];
#pragma unroll
      for (int c = 0; c < 8; c++) {
        const uint32_t ug = a[c >> 1][2 * (c & 1)], ug8 = a[c >> 1][2 * (c & 1) + 1];
        const uint32_t fr[4] = {bytes_to_half2(ug, 0x4140), bytes_to_half2(ug8, 0x4140), bytes_to_half2(ug, 0x4342), bytes_to_half2(ug8, 0x4342)};
        uint32_t b[4];
        ldmatrix_x4(b, b_addr + (uint32_t)((sl * Q8S_SLAB + c * 16) * 2));
        if ((c & 1) == 0) mma_16816_zero(acc[c >> 1], fr, b[0], b[1]);
        else mma_16816(acc[c >> 1], fr, b[0], b[1]);
        mma_16816(acc[c >> 1], fr, b[2], b[3]);
      }
      // per run of F inputs: y += scale * (q . x) + bias * sum(x)
      constexpr int NRUN = Q8S_SLAB / F, QPR = F / 32;  // runs per slab, accumulators per run
      const int run0 = sl * NRUN;
#pragma unroll
      for (int rn = 0; rn < NRUN; rn++) {
        if ((run0 + rn) * F < n_in) {  // (beyond the inputs the padded slab holds zeros and no group)
          const int gi = (run0 + rn) >> gshift;
          const float sc0 = bf16f(s0[gi]), sc1 = bf16f(s1[gi]), bi0 = bf16f(z0[gi]), bi1 = bf16f(z1[gi]);
          const float sa = gsum[(2 * qq) * nsum + run0 + rn], sbb = gsum[(2 * qq + 1) * nsum + run0 + rn];
          float d[4];
#pragma unroll
          for (int q = 0; q < 4; q++) {
            d[q] = acc[rn * QPR][q];
#pragma unroll
            for (int t = 1; t < QPR; t++) d[q] += acc[rn * QPR + t][q];
          }
          tot[0] += sc0 * d[0] + bi0 * sa;
          tot[1] += sc0 * d[1] + bi0 * sbb;
          tot[2] += sc1 * d[2] + bi1 * sa;
          tot[3] += sc1 * d[3] + bi1 * sbb;
        }
      }
#else
      if (lane == 0) mbar_arrive(&empty[st]);
#endif
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sempty[sb]);
    sb ^= 1;
    if (sb == 0) sphase ^= 1u;
    // the sets' partial totals of a row group meet in set 0 (fixed order: deterministic)
    if (Q8S_SETS > 1) {
      if (set > 0) xch[((xb * (Q8S_SETS - 1) + set - 1) * 8 + rw) * 32 + lane] = make_float4(tot[0], tot[1], tot[2], tot[3]);
      asm volatile("bar.sync %0, %1;" ::"r"(2 + rw), "n"(Q8S_SETS * 32) : "memory");  // the warps of this row group
      if (set > 0) { xb ^= 1; continue; }
#pragma unroll
      for (int t = 1; t < Q8S_SETS; t++) {
        const float4 o = xch[((xb * (Q8S_SETS - 1) + t - 1) * 8 + rw) * 32 + lane];
        tot[0] += o.x; tot[1] += o.y; tot[2] += o.z; tot[3] += o.w;
      }
      xb ^= 1;
    }
    // tot: (output row g, activation rows 2 qq, 2 qq + 1), (output row g + 8, the same)
    const int o = rb * Q8S_ROWS + 16 * rw + g;
    if (2 * qq < rows) {
      if (o < P.w.rows) y[(size_t)(2 * qq) * P.w.rows + o] = tot[0];
      if (o + 8 < P.w.rows) y[(size_t)(2 * qq) * P.w.rows + o + 8] = tot[2];
    }
    if (2 * qq + 1 < rows) {
      if (o < P.w.rows) y[(size_t)(2 * qq + 1) * P.w.rows + o] = tot[1];
      if (o + 8 < P.w.rows) y[(size_t)(2 * qq + 1) * P.w.rows + o + 8] = tot[3];
    }
  }
}

__global__ void __launch_bounds__(256) q8_embed_kernel(const Q8Weight w, const int *__restrict__ tokens, float *__restrict__ x, int round_bf16) {
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  int t = tokens[r];
  if (t < 0 || t >= w.rows) t = 0;
  const int ng = w.in / w.group;
  for (int c = threadIdx.x; c < w.in; c += 256) {
    const int gi = c / w.group;
    float v = bf16f(w.scales[(size_t)t * ng + gi]) * (float)w.w[(size_t)t * w.in + c] + bf16f(w.biases[(size_t)t * ng + gi]);
    if (round_bf16) {
      const uint32_t u = __float_as_uint(v);
      v = __uint_as_float((u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u);
    }
    x[(size_t)r * w.in + c] = v;
  }
}

}  // namespace

void check_q8_weight(const Q8Weight &w) {
  IJ_CHECK(w.w && w.scales && w.biases, "8-bit affine weight: null tensor");
  IJ_CHECK(w.rows > 0 && w.in > 0, "8-bit affine weight [%d][%d]", w.rows, w.in);
  IJ_CHECK(w.group >= 32 && (w.group & (w.group - 1)) == 0 && w.group <= 256 && w.in % w.group == 0,
           "8-bit affine group size %d must be 32, 64, 128 or 256 and divide the inputs (%d)", w.group, w.in);
}

template <int NT>
static void launch_q8_nt(const Q8Weight &w, const float *x, int rows, float *y, cudaStream_t st) {
  const size_t smem = std::max(q8_smem_bytes(NT, std::min(Q8_KC, w.in)), (size_t)8 * NT * 8 * 17 * 4);
  IJ_CUDA(cudaFuncSetAttribute(q8_wide_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  launch_pdl(q8_wide_kernel<NT>, dim3((w.rows + 127) / 128), dim3(256), smem, st, w, x, rows, y);
}

static void make_q8_map(CUtensorMap *out, const Q8Weight &w) {
  typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static encode_fn encode = nullptr;  // the driver's cuTensorMapEncodeTiled, looked up through the runtime (no link against libcuda)
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    IJ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    IJ_CHECK(fn != nullptr && q == cudaDriverEntryPointSuccess, "the driver does not provide cuTensorMapEncodeTiled");
    encode = reinterpret_cast<encode_fn>(fn);
  }
  const cuuint64_t dims[2] = {(cuuint64_t)w.in, (cuuint64_t)w.rows};
  const cuuint64_t strides[1] = {(cuuint64_t)w.in};
  const cuuint32_t box[2] = {(cuuint32_t)Q8S_SLAB, (cuuint32_t)Q8S_ROWS};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult rc = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w.w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  IJ_CHECK(rc == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for an 8-bit weight of %d x %d", (int)rc, w.rows, w.in);
}

// the streaming form applies: few enough inputs to stage the activations once, aligned tensors
static bool q8_streamable(const Q8Weight &w) {
  return w.in <= Q8_KC && w.in % 16 == 0 && w.group >= 32 && (((uintptr_t)w.w | (uintptr_t)w.scales | (uintptr_t)w.biases) & 15) == 0;
}

static void launch_q8_stream(const Q8Weight &w, const float *x, int rows, float *y, int *status, cudaStream_t st) {
  Q8StreamParams P{};
  make_q8_map(&P.map, w);
  P.w = w;
  P.nblocks = (w.rows + Q8S_ROWS - 1) / Q8S_ROWS;
  Q8StreamLayout &L = P.lay;
  L.kpad = (w.in + Q8S_SLAB - 1) / Q8S_SLAB * Q8S_SLAB;
  L.ldx = L.kpad + 8;
  L.ng = w.in / w.group;
  L.stages = Q8S_MAX_STAGES;
  const size_t budget = 226 * 1024 - 1024;
  // a multiple of the consumer sets: the previous fill of a stage must have gone to the same set, or a set could run two
  // fills ahead of the barrier's parity
  while (L.stages > Q8S_SETS && L.total() > budget) L.stages -= Q8S_SETS;
  IJ_CHECK(L.total() <= budget, "8-bit Linear of %d inputs in groups of %d does not fit shared memory", w.in, w.group);
  const size_t smem = L.total() + 1024;
  const dim3 grid(std::min(sm_count(), P.nblocks)), block(Q8S_THREADS);
  auto go = [&](auto kernel) {
    IJ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_pdl(kernel, grid, block, smem, st, P, x, rows, y, status);
  };
  if (w.group == 32) go(q8_stream_kernel<32>);
  else if (w.group == 64) go(q8_stream_kernel<64>);
  else go(q8_stream_kernel<128>);
}

void launch_q8_linear(const Q8Weight &w, const float *x, int rows, float *y, int *status, cudaStream_t st) {
  check_q8_weight(w);
  IJ_CHECK(rows >= 1 && rows <= 64, "rows %d outside 1..64", rows);
  IJ_CHECK(((uintptr_t)x & 15) == 0 && w.in % 16 == 0, "x must be 16-byte aligned, the inputs a multiple of 16");
  if (q8_streamable(w)) {
    for (int r0 = 0; r0 < rows; r0 += 8)  // 8 rows per pass over the weights
      launch_q8_stream(w, x + (size_t)r0 * w.in, std::min(8, rows - r0), y + (size_t)r0 * w.rows, status, st);
    return;
  }
  IJ_CHECK(w.group >= 64 && w.in % 64 == 0 && ((uintptr_t)w.w & 15) == 0,
           "ne_q8_linear: more than %d inputs or unaligned tensors need groups of 64, 128 or 256, a multiple of 64 inputs and 16-byte aligned weight bytes",
           Q8_KC);
  for (int r0 = 0; r0 < rows; r0 += 16) {  // at most 16 rows per pass over the weights (the staged activations' shared memory)
    const int nr = std::min(16, rows - r0);
    const float *xr = x + (size_t)r0 * w.in;
    float *yr = y + (size_t)r0 * w.rows;
    if (nr <= 8) launch_q8_nt<1>(w, xr, nr, yr, st);
    else launch_q8_nt<2>(w, xr, nr, yr, st);
  }
}

int q8_linear_launches(const Q8Weight &w, int rows) { return q8_streamable(w) ? (rows + 7) / 8 : (rows + 15) / 16; }

void launch_q8_embed(const Q8Weight &w, const int *tokens, int rows, float *x, bool round_bf16, cudaStream_t st) {
  check_q8_weight(w);
  launch_pdl(q8_embed_kernel, dim3(rows), dim3(256), 0, st, w, tokens, x, round_bf16 ? 1 : 0);
}

}  // namespace ijah
