// Hyper-connection read: two launches. hc_pre: a cluster of four CTAs per block of eight output rows, one CTA per
// residual stream, the four per-stream partial dot products summed in a fixed order through distributed shared memory.
// hc_mix: one warp per output column. Both are small (6.6 MB of 8-bit weights at the reference's sizes) and bound by
// launch latency and L2, not by HBM.
#include <cooperative_groups.h>

#include "common.hpp"
#include "hc_read.cuh"

namespace cg = cooperative_groups;

namespace ijah {
namespace {

constexpr int HC_RC = 8;          // rows per pass (accumulators per lane)
constexpr float HC_EPS = 1e-6f;   // reference kernels/fn_trunk.metal:74

__device__ __forceinline__ float bf16f(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }
__device__ __forceinline__ float sigm(float v) { return 1.0f / (1.0f + __expf(-v)); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// sum_i q_i * x_i and sum_i x_i over the four bytes of one word
__device__ __forceinline__ void dot4q(uint32_t u, float4 x, float &qx, float &sx) {
  qx += (float)(u & 0xFF) * x.x + (float)((u >> 8) & 0xFF) * x.y + (float)((u >> 16) & 0xFF) * x.z + (float)(u >> 24) * x.w;
  sx += (x.x + x.y) + (x.z + x.w);
}

// grid (HC, LR / 8 + 1), cluster (HC, 1, 1), 256 threads. blockIdx.x = stream, blockIdx.y = block of eight rows of W_down;
// the last block holds the HC rows of W_inject. dynamic shared memory: HC_RC * H floats.
__global__ void __cluster_dims__(HC_STREAMS, 1, 1) __launch_bounds__(256)
hc_pre_kernel(const HcWeights w, const float *__restrict__ h, int rows, float *__restrict__ mix, float *__restrict__ inj) {
  extern __shared__ __align__(16) float xs[];  // [HC_RC][H]: h * norm weight of this stream (not yet scaled by 1/rms)
  __shared__ float red[HC_RC][8];
  __shared__ float part[8][HC_RC];
  cg::cluster_group cluster = cg::this_cluster();
  const int H = w.H, HCD = HC_STREAMS * H, LR = w.LR, G = w.down.group;
  const int s = blockIdx.x, blk = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool injb = blk == (int)gridDim.y - 1;
  const int row = blk * 8 + warp;
  for (int r0 = 0; r0 < rows; r0 += HC_RC) {
    const int nr = min(HC_RC, rows - r0);
    for (int r = 0; r < nr; r++) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < H; i += 256) {
        const float v = h[(size_t)(r0 + r) * HCD + s * H + i];
        ss += v * v;
        xs[r * H + i] = v * bf16f(w.norm[s * H + i]);
      }
      ss = warp_sum(ss);
      if (lane == 0) red[r][warp] = ss;
    }
    __syncthreads();
    float inv[HC_RC], acc[HC_RC];
#pragma unroll
    for (int r = 0; r < HC_RC; r++) {
      float t = 0.f;
      if (r < nr)
        for (int g = 0; g < 8; g++) t += red[r][g];
      inv[r] = rsqrtf(t / (float)H + HC_EPS);
      acc[r] = 0.f;
    }
    if (blk == 0 && threadIdx.x == 0) {
#pragma unroll
      for (int r = 0; r < HC_RC; r++)
        if (r < nr) inj[(size_t)(r0 + r) * 2 * HC_STREAMS + HC_STREAMS + s] = inv[r];
    }
    if (!injb) {
      const uint4 *w4 = reinterpret_cast<const uint4 *>(w.down.w + (size_t)row * HCD + (size_t)s * H);
      const uint16_t *sc = w.down.scales + (size_t)row * (HCD / G) + s * (H / G);
      const uint16_t *bi = w.down.biases + (size_t)row * (HCD / G) + s * (H / G);
      for (int c = lane; c < H / 16; c += 32) {
        const uint4 u = __ldg(w4 + c);
        const int g = 16 * c / G;
        const float sg = bf16f(sc[g]), bg = bf16f(bi[g]);
#pragma unroll
        for (int r = 0; r < HC_RC; r++) {
          if (r >= nr) break;
          const float4 *x4 = reinterpret_cast<const float4 *>(xs + r * H) + 4 * c;
          float qx = 0.f, sx = 0.f;
          dot4q(u.x, x4[0], qx, sx);
          dot4q(u.y, x4[1], qx, sx);
          dot4q(u.z, x4[2], qx, sx);
          dot4q(u.w, x4[3], qx, sx);
          acc[r] += sg * qx + bg * sx;
        }
      }
    } else if (warp < HC_STREAMS) {
      const uint4 *w4 = reinterpret_cast<const uint4 *>(w.inject + (size_t)warp * HCD + (size_t)s * H);
      for (int c = lane; c < H / 8; c += 32) {
        const uint4 u = __ldg(w4 + c);
#pragma unroll
        for (int r = 0; r < HC_RC; r++) {
          if (r >= nr) break;
          const float4 *x4 = reinterpret_cast<const float4 *>(xs + r * H) + 2 * c;
          const float4 a = x4[0], b = x4[1];
          acc[r] += __uint_as_float(u.x << 16) * a.x + __uint_as_float(u.x & 0xFFFF0000u) * a.y + __uint_as_float(u.y << 16) * a.z +
                    __uint_as_float(u.y & 0xFFFF0000u) * a.w + __uint_as_float(u.z << 16) * b.x + __uint_as_float(u.z & 0xFFFF0000u) * b.y +
                    __uint_as_float(u.w << 16) * b.z + __uint_as_float(u.w & 0xFFFF0000u) * b.w;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < HC_RC; r++) {
      const float v = warp_sum(acc[r]) * inv[r];
      if (lane == 0) part[warp][r] = v;
    }
    cluster.sync();
    if (cluster.block_rank() == 0 && threadIdx.x < 8 * HC_RC) {
      const int wr = threadIdx.x / HC_RC, r = threadIdx.x % HC_RC;
      if (r < nr) {
        float p[HC_STREAMS];
#pragma unroll
        for (int q = 0; q < HC_STREAMS; q++) p[q] = cluster.map_shared_rank(&part[0][0], q)[wr * HC_RC + r];
        const float v = (((p[0] + p[1]) + p[2]) + p[3]) * (1.0f / HC_STREAMS);
        if (!injb) mix[(size_t)(r0 + r) * LR + blk * 8 + wr] = v * sigm(v);
        else if (wr < HC_STREAMS) inj[(size_t)(r0 + r) * 2 * HC_STREAMS + wr] = 2.0f * sigm(v);
      }
    }
    cluster.sync();  // the partials stay readable until rank 0 has summed them; also fences xs / red for the next pass
  }
}

// grid ceil(H / 8), 256 threads: warp = output column c, eight lanes per stream row s * H + c of W_up (LR 8-bit inputs).
// dynamic shared memory: HC_RC * LR floats (the mix rows of one pass).
__global__ void __launch_bounds__(256)
hc_mix_kernel(const HcWeights w, const float *__restrict__ h, const float *__restrict__ mix, const float *__restrict__ inj, int rows,
              float *__restrict__ out) {
  extern __shared__ __align__(16) float ms[];  // [HC_RC][LR]
  const int H = w.H, HCD = HC_STREAMS * H, LR = w.LR, G = w.up.group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 8 + warp, s = lane >> 3, l8 = lane & 7;
  const bool live = c < H;
  const size_t row = (size_t)s * H + (live ? c : 0);
  const uint2 *w2 = reinterpret_cast<const uint2 *>(w.up.w + row * LR);
  const uint16_t *sc = w.up.scales + row * (LR / G), *bi = w.up.biases + row * (LR / G);
  const float nw = bf16f(w.norm[row]);
  for (int r0 = 0; r0 < rows; r0 += HC_RC) {
    const int nr = min(HC_RC, rows - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < nr * LR; i += 256) ms[i] = mix[(size_t)r0 * LR + i];
    __syncthreads();
    float acc[HC_RC];
#pragma unroll
    for (int r = 0; r < HC_RC; r++) acc[r] = 0.f;
    for (int ch = l8; ch < LR / 8; ch += 8) {
      const uint2 u = __ldg(w2 + ch);
      const int g = 8 * ch / G;
      const float sg = bf16f(sc[g]), bg = bf16f(bi[g]);
#pragma unroll
      for (int r = 0; r < HC_RC; r++) {
        if (r >= nr) break;
        const float4 *m4 = reinterpret_cast<const float4 *>(ms + r * LR) + 2 * ch;
        float qx = 0.f, sx = 0.f;
        dot4q(u.x, m4[0], qx, sx);
        dot4q(u.y, m4[1], qx, sx);
        acc[r] += sg * qx + bg * sx;
      }
    }
#pragma unroll
    for (int r = 0; r < HC_RC; r++) {
      if (r >= nr) break;  // uniform over the warp
      float a = acc[r];
      a += __shfl_xor_sync(0xffffffffu, a, 1);
      a += __shfl_xor_sync(0xffffffffu, a, 2);
      a += __shfl_xor_sync(0xffffffffu, a, 4);
      const size_t rr = r0 + r;
      float v = sigm(a) * (h[rr * HCD + row] * inj[rr * 2 * HC_STREAMS + HC_STREAMS + s] * nw);
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      if (lane == 0 && live) out[rr * H + c] = v * (1.0f / HC_STREAMS);
    }
  }
}

}  // namespace

void check_hc_weights(const HcWeights &w) {
  IJ_CHECK(w.H > 0 && w.H % 16 == 0 && w.LR > 0 && w.LR % 8 == 0, "hyper-connection dims: H %d (multiple of 16), LR %d (multiple of 8)", w.H, w.LR);
  IJ_CHECK(w.down.rows == w.LR && w.down.in == HC_STREAMS * w.H, "hc down is [%d][%d], expected [%d][%d]", w.down.rows, w.down.in, w.LR, HC_STREAMS * w.H);
  IJ_CHECK(w.up.rows == HC_STREAMS * w.H && w.up.in == w.LR, "hc up is [%d][%d], expected [%d][%d]", w.up.rows, w.up.in, HC_STREAMS * w.H, w.LR);
  IJ_CHECK(w.down.group == w.up.group && w.down.group % 16 == 0 && w.H % w.down.group == 0 && w.LR % w.down.group == 0,
           "hc group size %d / %d must be a multiple of 16 dividing H and LR", w.down.group, w.up.group);
  IJ_CHECK((size_t)HC_RC * w.H * 4 <= 200 * 1024 && (size_t)HC_RC * w.LR * 4 <= 200 * 1024, "hyper-connection dims too large for shared memory");
  for (const void *p : {(const void *)w.norm, (const void *)w.inject, (const void *)w.down.w, (const void *)w.up.w})
    IJ_CHECK(p != nullptr && ((uintptr_t)p & 15) == 0, "hyper-connection weights must be 16-byte aligned");
  for (const void *p : {(const void *)w.down.scales, (const void *)w.down.biases, (const void *)w.up.scales, (const void *)w.up.biases})
    IJ_CHECK(p != nullptr && ((uintptr_t)p & 1) == 0, "hyper-connection scales missing");
}

void launch_hc_pre(const HcWeights &w, const float *h, int rows, float *mix, float *inj, cudaStream_t st) {
  IJ_CHECK(rows >= 1 && ((uintptr_t)h & 15) == 0, "bad rows / alignment");
  const size_t smem = (size_t)HC_RC * w.H * 4;
  IJ_CUDA(cudaFuncSetAttribute(hc_pre_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  hc_pre_kernel<<<dim3(HC_STREAMS, w.LR / 8 + 1), 256, smem, st>>>(w, h, rows, mix, inj);
  IJ_CUDA(cudaGetLastError());
}

void launch_hc_mix(const HcWeights &w, const float *h, const float *mix, const float *inj, int rows, float *out, cudaStream_t st) {
  IJ_CHECK(rows >= 1, "bad rows");
  const size_t smem = (size_t)HC_RC * w.LR * 4;
  IJ_CUDA(cudaFuncSetAttribute(hc_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  hc_mix_kernel<<<(w.H + 7) / 8, 256, smem, st>>>(w, h, mix, inj, rows, out);
  IJ_CUDA(cudaGetLastError());
}

}  // namespace ijah
