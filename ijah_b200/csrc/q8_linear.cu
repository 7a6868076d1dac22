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

constexpr int Q8_KB = 256;  // inputs staged per pass (a multiple of every supported group size)

__device__ __forceinline__ float bf16f(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }

// bytes (b0, b1) of `u` selected by `sel` -> half2(b0, b1): 0x6400 | b is the half 1024 + b; subtracting 1024 is exact
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t u, uint32_t sel) {
  const uint32_t h = __byte_perm(u, 0x64646464u, sel);
  const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half((unsigned short)0x6400)));
  return *reinterpret_cast<const uint32_t *>(&r);
}

template <int NT>
__global__ void __launch_bounds__(256) q8_linear_kernel(const Q8Weight w, const float *__restrict__ x, int rows, float *__restrict__ y) {
  constexpr int LDX = Q8_KB + 8;  // halfs per staged row (+16 bytes: the lanes' 16-byte reads of 8 rows fall on distinct banks)
  constexpr int XS_HALFS = NT * 8 * LDX;
  constexpr int STAGE_BYTES = 2 * XS_HALFS * 2 + NT * 8 * (Q8_KB / 16) * 4, OUT_BYTES = 8 * NT * 8 * 17 * 4;
  __shared__ __align__(16) unsigned char buf[STAGE_BYTES > OUT_BYTES ? STAGE_BYTES : OUT_BYTES];
  __half *xhi = reinterpret_cast<__half *>(buf);
  __half *xlo = xhi + XS_HALFS;
  float *gsum = reinterpret_cast<float *>(xlo + XS_HALFS);  // [NT * 8][Q8_KB / 16]: sums of x over 16 inputs (a group is a multiple of 16)
  float(*outt)[NT * 8][17] = reinterpret_cast<float(*)[NT * 8][17]>(buf);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, qq = lane & 3;
  const int n_in = w.in, G = w.group, ng = n_in / G;
  const int o0 = (blockIdx.x * 8 + warp) * 16;
  const int r0 = min(o0 + g, w.rows - 1), r1 = min(o0 + g + 8, w.rows - 1);
  const uint8_t *w0 = w.w + (size_t)r0 * n_in + 8 * qq, *w1 = w.w + (size_t)r1 * n_in + 8 * qq;
  const uint16_t *s0 = w.scales + (size_t)r0 * ng, *s1 = w.scales + (size_t)r1 * ng;
  const uint16_t *b0 = w.biases + (size_t)r0 * ng, *b1 = w.biases + (size_t)r1 * ng;
  float tot[NT][4];
#pragma unroll
  for (int n = 0; n < NT; n++)
#pragma unroll
    for (int j = 0; j < 4; j++) tot[n][j] = 0.f;
  pdl_launch();
  // the first pass's weight bytes are static data: in flight before the wait on the kernel that produces x
  uint2 wa[Q8_KB / 32], wb[Q8_KB / 32];
#pragma unroll
  for (int ks = 0; ks < Q8_KB / 32; ks++) {
    wa[ks] = __ldcs(reinterpret_cast<const uint2 *>(w0 + ks * 32));
    wb[ks] = __ldcs(reinterpret_cast<const uint2 *>(w1 + ks * 32));
  }
  pdl_wait();
  for (int kb = 0; kb < n_in; kb += Q8_KB) {
    const int kn = min(Q8_KB, n_in - kb);  // a multiple of 32
    __syncthreads();
    // stage x[rows][kb .. kb + kn) as hi / lo halves, and its sums over 16 inputs (from the values the MMAs see: hi + lo)
    for (int i = threadIdx.x; i < NT * 8 * (Q8_KB / 16); i += 256) {
      const int r = i / (Q8_KB / 16), c = i % (Q8_KB / 16);
      float s = 0.f;
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int j = 0; j < 8; j++) hi[j] = lo[j] = 0u;
      if (r < rows && c * 16 < kn) {
        const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)r * n_in + kb + c * 16);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const float4 v = __ldcg(src + j);
          const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
          const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
          const __half2 l01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y), l23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
          const float2 g01 = __half22float2(l01), g23 = __half22float2(l23);
          s += ((f01.x + g01.x) + (f01.y + g01.y)) + ((f23.x + g23.x) + (f23.y + g23.y));
          hi[2 * j] = *reinterpret_cast<const uint32_t *>(&h01); hi[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&h23);
          lo[2 * j] = *reinterpret_cast<const uint32_t *>(&l01); lo[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&l23);
        }
      }
      uint4 *dh = reinterpret_cast<uint4 *>(xhi + r * LDX + c * 16), *dl = reinterpret_cast<uint4 *>(xlo + r * LDX + c * 16);
      dh[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]); dh[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
      dl[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]); dl[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
      gsum[r * (Q8_KB / 16) + c] = s;
    }
    __syncthreads();
    float acc[NT][4];
#pragma unroll
    for (int ks = 0; ks < Q8_KB / 32; ks++) {
      if (ks * 32 < kn) {  // uniform
        const int k = kb + ks * 32;
        if (k % G == 0) {
#pragma unroll
          for (int n = 0; n < NT; n++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[n][j] = 0.f;
        }
        // the lane's 8 bytes of rows g and g + 8 -> fragments of two MMAs (inputs 8 qq + 0..3, then 8 qq + 4..7)
        const uint32_t a00 = bytes_to_half2(wa[ks].x, 0x4140), a01 = bytes_to_half2(wa[ks].x, 0x4342);
        const uint32_t a02 = bytes_to_half2(wa[ks].y, 0x4140), a03 = bytes_to_half2(wa[ks].y, 0x4342);
        const uint32_t a10 = bytes_to_half2(wb[ks].x, 0x4140), a11 = bytes_to_half2(wb[ks].x, 0x4342);
        const uint32_t a12 = bytes_to_half2(wb[ks].y, 0x4140), a13 = bytes_to_half2(wb[ks].y, 0x4342);
        const uint32_t fa[4] = {a00, a10, a01, a11}, fb[4] = {a02, a12, a03, a13};
#pragma unroll
        for (int n = 0; n < NT; n++) {
          const uint4 h = *reinterpret_cast<const uint4 *>(xhi + (n * 8 + g) * LDX + ks * 32 + 8 * qq);
          const uint4 l = *reinterpret_cast<const uint4 *>(xlo + (n * 8 + g) * LDX + ks * 32 + 8 * qq);
          mma_16816(acc[n], fa, h.x, h.y);
          mma_16816(acc[n], fb, h.z, h.w);
          mma_16816(acc[n], fa, l.x, l.y);
          mma_16816(acc[n], fb, l.z, l.w);
        }
        if ((k + 32) % G == 0) {  // the group is complete: scale, add the bias term
          const int gi = k / G;
          const float sc0 = bf16f(s0[gi]), sc1 = bf16f(s1[gi]), bi0 = bf16f(b0[gi]), bi1 = bf16f(b1[gi]);
          const int c0 = (k + 32 - G - kb) / 16, nc = G / 16;
#pragma unroll
          for (int n = 0; n < NT; n++) {
            float sa = 0.f, sb = 0.f;  // sum of x over the group for activation rows 8 n + 2 qq and + 1
            for (int c = 0; c < nc; c++) {
              sa += gsum[(n * 8 + 2 * qq) * (Q8_KB / 16) + c0 + c];
              sb += gsum[(n * 8 + 2 * qq + 1) * (Q8_KB / 16) + c0 + c];
            }
            tot[n][0] += sc0 * acc[n][0] + bi0 * sa;
            tot[n][1] += sc0 * acc[n][1] + bi0 * sb;
            tot[n][2] += sc1 * acc[n][2] + bi1 * sa;
            tot[n][3] += sc1 * acc[n][3] + bi1 * sb;
          }
        }
      }
    }
    // the next pass's weight bytes go out before its activations are staged
    if (kb + Q8_KB < n_in) {
#pragma unroll
      for (int ks = 0; ks < Q8_KB / 32; ks++) {
        const int k = kb + Q8_KB + ks * 32;
        if (k < n_in) {
          wa[ks] = __ldcs(reinterpret_cast<const uint2 *>(w0 + k));
          wb[ks] = __ldcs(reinterpret_cast<const uint2 *>(w1 + k));
        }
      }
    }
  }
  // tot[n]: (output row g, activation rows 8n + 2qq, +1), (output row g + 8, the same rows): transpose through shared memory
  __syncthreads();
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
  IJ_CHECK(w.rows > 0 && w.in > 0 && w.in % 32 == 0, "8-bit affine weight [%d][%d]: inputs must be a multiple of 32", w.rows, w.in);
  IJ_CHECK(w.group >= 32 && w.group % 32 == 0 && Q8_KB % w.group == 0 && w.in % w.group == 0,
           "8-bit affine group size %d must be 32, 64, 128 or 256 and divide the inputs", w.group);
  IJ_CHECK(((uintptr_t)w.w & 7) == 0, "8-bit affine weight bytes must be 8-byte aligned");
}

void launch_q8_linear(const Q8Weight &w, const float *x, int rows, float *y, cudaStream_t st) {
  check_q8_weight(w);
  IJ_CHECK(rows >= 1 && rows <= 64, "rows %d outside 1..64", rows);
  IJ_CHECK(((uintptr_t)x & 15) == 0 && w.in % 16 == 0, "x must be 16-byte aligned");
  const dim3 grid((w.rows + 127) / 128), block(256);
  for (int r0 = 0; r0 < rows; r0 += 32) {  // at most 32 rows per pass over the weights (the staged activations' shared memory)
    const int nr = std::min(32, rows - r0);
    const float *xr = x + (size_t)r0 * w.in;
    float *yr = y + (size_t)r0 * w.rows;
    if (nr <= 8) launch_pdl(q8_linear_kernel<1>, grid, block, 0, st, w, xr, nr, yr);
    else if (nr <= 16) launch_pdl(q8_linear_kernel<2>, grid, block, 0, st, w, xr, nr, yr);
    else launch_pdl(q8_linear_kernel<4>, grid, block, 0, st, w, xr, nr, yr);
  }
}

void launch_q8_embed(const Q8Weight &w, const int *tokens, int rows, float *x, bool round_bf16, cudaStream_t st) {
  check_q8_weight(w);
  launch_pdl(q8_embed_kernel, dim3(rows), dim3(256), 0, st, w, tokens, x, round_bf16 ? 1 : 0);
}

}  // namespace ijah
