// Glue kernels of the decoder stack. See stack.cuh.
#include <algorithm>
#include <cmath>

#include "common.hpp"
#include "launch.cuh"
#include "stack.cuh"

namespace ijah {

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {  // round to nearest even (finite inputs)
  const uint32_t u = __float_as_uint(f);
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

// =============================================================================================== embedding, norm
__global__ void embed_kernel(const int *__restrict__ tokens, const uint16_t *__restrict__ embed, int vocab, int H, float *__restrict__ x) {
  const int r = blockIdx.y;
  pdl_launch();
  pdl_wait();
  int t = tokens[r];
  t = (t < 0 || t >= vocab) ? 0 : t;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) x[(size_t)r * H + i] = bf16_bits_to_float(embed[(size_t)t * H + i]);
}

void launch_embed(const int *tokens, const uint16_t *embed_bf16, int vocab, int H, int rows, float *x, cudaStream_t st) {
  launch_pdl(embed_kernel, dim3((H + 255) / 256, rows), dim3(256), 0, st, tokens, embed_bf16, vocab, H, x);
}

__global__ void __launch_bounds__(256) rms_add_kernel(float *__restrict__ x, const float *__restrict__ add, float *__restrict__ xn,
                                                      const uint16_t *__restrict__ w, int H, float eps) {
  __shared__ float red[8];
  const int r = blockIdx.x;
  float *xr = x + (size_t)r * H;
  float ss = 0.0f;
  pdl_launch();
  pdl_wait();
  for (int i = threadIdx.x; i < H; i += 256) {
    float v = xr[i];
    if (add) { v += add[(size_t)r * H + i]; xr[i] = v; }
    ss += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; i++) tot += red[i];
  const float sc = rsqrtf(tot / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += 256) xn[(size_t)r * H + i] = xr[i] * sc * (w ? bf16_bits_to_float(w[i]) : 1.0f);
}

void launch_rms_add(float *x, const float *add, float *xn, const uint16_t *w_bf16, int rows, int H, float eps, cudaStream_t st) {
  launch_pdl(rms_add_kernel, dim3(rows), dim3(256), 0, st, x, add, xn, w_bf16, H, eps);
}

// =============================================================================================== attention stand-in
// partial: one CTA per (block of PB = 64, 128 or 256 cached positions, KV head). K and V of the block are staged once in
// shared memory and used for every query vector of the head group (rows x heads / kv_heads of them), 16 at a time; two
// groups of four warps take alternate tiles of 16 query vectors (each group with its own P buffer, reductions and named
// barrier):
//   S = Q K^T (warp w of the group: positions w PB/4 .. (w + 1) PB/4 - 1), block max and sum over the four warps,
//   P = exp(S - max) as fp16, O = P V (warp w: a quarter of the head dimension).
// Per (query vector, block) it leaves max, sum and the unnormalised O; the merge kernel combines the blocks. The launcher
// takes the largest block that divides the cache length, fits shared memory and still fills the GPU: the partial results
// (one [head dim + 2] float record per query vector and block) are as many bytes as the K / V cache itself at 64 positions
// per block and 8 rows, a quarter of that at 256.
constexpr int AT_PB_MIN = 64;  // smallest block: the cache length is a multiple of it

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

constexpr int AT_QCAP = 64;  // query vectors staged at a time (fp16, scaled)

constexpr int AT_THREADS = 256;
template <int HD, int PB>
__global__ void __launch_bounds__(AT_THREADS) attn_partial_kernel(const float *__restrict__ q, const __half *__restrict__ kc, const __half *__restrict__ vc, int rows,
                                                           int heads, int kv_heads, int nsplit, float *__restrict__ part, float *__restrict__ ml) {
  constexpr int LD = HD + 8;          // padded row length in halfs (ldmatrix rows on distinct banks)
  constexpr int LDP = PB + 8;
  constexpr int PW = PB / 4;   // positions per warp of a group
  constexpr int PT = PW / 16;  // 16-position tiles per warp
  extern __shared__ __align__(16) unsigned char at_smem[];
  __half *Ks = reinterpret_cast<__half *>(at_smem);
  __half *Vs = Ks + PB * LD;
  __half *Qs = Vs + PB * LD;
  const int grp = threadIdx.x >> 7;  // warp group: tiles grp, grp + 2, ...
  __half *Ps = Qs + AT_QCAP * LD + grp * 16 * LDP;
  float *red = reinterpret_cast<float *>(Qs + AT_QCAP * LD + 2 * 16 * LDP) + grp * 128;  // [2][4][16]: per-warp max, per-warp sum
  const int split = blockIdx.x, kvh = blockIdx.y, G = heads / kv_heads, NQ = rows * G;
  const int warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31, g = lane >> 2, qq = lane & 3;
  auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory"); };
  // K and V of the block: asynchronous 16-byte copies, all in flight at once (static data: before the wait on the
  // preceding kernel, so the copies overlap its tail)
  {
    const size_t rstride = (size_t)kv_heads * HD;
    const __half *ksrc = kc + ((size_t)split * PB) * rstride + (size_t)kvh * HD;
    const __half *vsrc = vc + ((size_t)split * PB) * rstride + (size_t)kvh * HD;
    const uint32_t Kd = smem_u32(Ks), Vd = smem_u32(Vs);
#pragma unroll 4
    for (int i = threadIdx.x; i < PB * (HD / 8); i += AT_THREADS) {
      const int p = i / (HD / 8), c = i % (HD / 8);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(Kd + (uint32_t)((p * LD + c * 8) * 2)), "l"(ksrc + p * rstride + c * 8) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(Vd + (uint32_t)((p * LD + c * 8) * 2)), "l"(vsrc + p * rstride + c * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  pdl_launch();
  pdl_wait();
  const float scale = rsqrtf((float)HD);
  const uint32_t Qa0 = smem_u32(Qs), Ka = smem_u32(Ks), Va = smem_u32(Vs), Pa = smem_u32(Ps);
  for (int qc = 0; qc < NQ; qc += AT_QCAP) {
    __syncthreads();  // the previous chunk's readers of Qs are done
    // the chunk's query vectors: fp32 -> scaled fp16, four independent 16-byte loads per thread per pass
    for (int i0 = 0; i0 < AT_QCAP * (HD / 4); i0 += AT_THREADS * 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = i0 + u * AT_THREADS + threadIdx.x, j = i / (HD / 4), c = i % (HD / 4), qi = qc + j;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (qi < NQ) v[u] = __ldcg(reinterpret_cast<const float4 *>(q + ((size_t)(qi / G) * heads + kvh * G + qi % G) * HD + c * 4));
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = i0 + u * AT_THREADS + threadIdx.x, j = i / (HD / 4), c = i % (HD / 4);
        __half2 *dst = reinterpret_cast<__half2 *>(Qs + j * LD + c * 4);
        dst[0] = __floats2half2_rn(v[u].x * scale, v[u].y * scale);
        dst[1] = __floats2half2_rn(v[u].z * scale, v[u].w * scale);
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    for (int qt = grp; qt * 16 < min(AT_QCAP, NQ - qc); qt += 2) {
      const uint32_t Qa = Qa0 + (uint32_t)(qt * 16 * LD * 2);
      // ---- S = Q K^T for this warp's PW positions
      float s[PT][2][4];
#pragma unroll
      for (int pt = 0; pt < PT; pt++)
#pragma unroll
        for (int j = 0; j < 4; j++) s[pt][0][j] = s[pt][1][j] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        uint32_t a[4];
        ldsm_x4(a, Qa + (uint32_t)(((lane & 15) * LD + kk * 16 + (lane >> 4) * 8) * 2));
        const int m = lane >> 3;
#pragma unroll
        for (int pt = 0; pt < PT; pt++) {
          uint32_t b[4];
          ldsm_x4(b, Ka + (uint32_t)(((warp * PW + pt * 16 + (lane & 7) + (m >> 1) * 8) * LD + kk * 16 + (m & 1) * 8) * 2));
          mma_16816(s[pt][0], a, b[0], b[1]);
          mma_16816(s[pt][1], a, b[2], b[3]);
        }
      }
      // ---- block max and sum per query row (rows g and g + 8 of the tile)
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int pt = 0; pt < PT; pt++) {
        mx0 = fmaxf(mx0, fmaxf(fmaxf(s[pt][0][0], s[pt][0][1]), fmaxf(s[pt][1][0], s[pt][1][1])));
        mx1 = fmaxf(mx1, fmaxf(fmaxf(s[pt][0][2], s[pt][0][3]), fmaxf(s[pt][1][2], s[pt][1][3])));
      }
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, o));
      }
      group_sync();  // the group's previous tile: its readers of red and Ps are done
      if (qq == 0) { red[warp * 16 + g] = mx0; red[warp * 16 + g + 8] = mx1; }
      group_sync();
      float m0 = red[g], m1 = red[g + 8];
#pragma unroll
      for (int w = 1; w < 4; w++) { m0 = fmaxf(m0, red[w * 16 + g]); m1 = fmaxf(m1, red[w * 16 + g + 8]); }
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int pt = 0; pt < PT; pt++) {
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
          const float p0 = __expf(s[pt][nt][0] - m0), p1 = __expf(s[pt][nt][1] - m0), p2 = __expf(s[pt][nt][2] - m1), p3 = __expf(s[pt][nt][3] - m1);
          const __half2 h01 = __floats2half2_rn(p0, p1), h23 = __floats2half2_rn(p2, p3);
          // the sums use the rounded values the tensor core will multiply with
          l0 += __low2float(h01) + __high2float(h01);
          l1 += __low2float(h23) + __high2float(h23);
          *reinterpret_cast<__half2 *>(Ps + g * LDP + warp * PW + pt * 16 + nt * 8 + 2 * qq) = h01;
          *reinterpret_cast<__half2 *>(Ps + (g + 8) * LDP + warp * PW + pt * 16 + nt * 8 + 2 * qq) = h23;
        }
      }
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, o);
        l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, o);
      }
      if (qq == 0) { red[64 + warp * 16 + g] = l0; red[64 + warp * 16 + g + 8] = l1; }
      group_sync();
      // ---- O = P V for this warp's quarter of the head dimension
      constexpr int NTW = HD / 4 / 8;  // n-tiles per warp
      float o_acc[NTW][4];
#pragma unroll
      for (int n = 0; n < NTW; n++)
#pragma unroll
        for (int j = 0; j < 4; j++) o_acc[n][j] = 0.f;
#pragma unroll
      for (int ks = 0; ks < PB / 16; ks++) {
        uint32_t a[4];
        ldsm_x4(a, Pa + (uint32_t)(((lane & 15) * LDP + ks * 16 + (lane >> 4) * 8) * 2));
#pragma unroll
        for (int n2 = 0; n2 < NTW / 2; n2++) {
          uint32_t b[4];
          const int m = lane >> 3, n0 = warp * (HD / 4) + n2 * 16;
          ldsm_x4_trans(b, Va + (uint32_t)(((ks * 16 + (lane & 7) + (m & 1) * 8) * LD + n0 + (m >> 1) * 8) * 2));
          mma_16816(o_acc[2 * n2], a, b[0], b[1]);
          mma_16816(o_acc[2 * n2 + 1], a, b[2], b[3]);
        }
      }
      // ---- partial results of the tile's live query vectors
      const int q0 = qc + qt * 16 + g, q1 = q0 + 8;
      if (warp == 0 && qq == 0) {
        float la = 0.f, lb = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) { la += red[64 + w * 16 + g]; lb += red[64 + w * 16 + g + 8]; }
        if (q0 < NQ) { ml[(((size_t)kvh * NQ + q0) * nsplit + split) * 2] = m0; ml[(((size_t)kvh * NQ + q0) * nsplit + split) * 2 + 1] = la; }
        if (q1 < NQ) { ml[(((size_t)kvh * NQ + q1) * nsplit + split) * 2] = m1; ml[(((size_t)kvh * NQ + q1) * nsplit + split) * 2 + 1] = lb; }
      }
#pragma unroll
      for (int n = 0; n < NTW; n++) {
        const int d = warp * (HD / 4) + n * 8 + 2 * qq;
        if (q0 < NQ) *reinterpret_cast<float2 *>(part + (((size_t)kvh * NQ + q0) * nsplit + split) * HD + d) = make_float2(o_acc[n][0], o_acc[n][1]);
        if (q1 < NQ) *reinterpret_cast<float2 *>(part + (((size_t)kvh * NQ + q1) * nsplit + split) * HD + d) = make_float2(o_acc[n][2], o_acc[n][3]);
      }
    }
  }
}

// merge: one CTA per query vector (row, head), 1024 threads. The block maxima and sums of all position blocks are loaded in
// parallel (one per thread), reduced to the global maximum and the weights exp(m_s - M) in shared memory; then 1024 / hd
// thread groups each sum a slice of the blocks for every dimension with independent loads (eight in flight) and the slices
// are added through shared memory, so the kernel costs a few memory round trips instead of one per block. The row's own
// (k, v) enters as one more position.
constexpr int AT_MAXSPLIT = 1024;
constexpr int AT_MT = 1024;  // merge threads
__global__ void __launch_bounds__(AT_MT) attn_merge_kernel(const float *__restrict__ q, const float *__restrict__ knew, const float *__restrict__ vnew,
                                                           const float *__restrict__ part, const float *__restrict__ ml, int rows, int heads, int kv_heads,
                                                           int hd, int nsplit, float *__restrict__ out) {
  __shared__ float red[32], red2[32];
  __shared__ float wsh[AT_MAXSPLIT];
  __shared__ float acc[AT_MT];
  __shared__ float s_M, s_den, s_wself;
  const int r = blockIdx.x / heads, h = blockIdx.x % heads, G = heads / kv_heads, kvh = h / G, NQ = rows * G, qi = r * G + h % G;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  pdl_launch();
  pdl_wait();
  const float *mlq = ml + ((size_t)kvh * NQ + qi) * nsplit * 2;
  // every thread's block statistics (threads beyond nsplit: neutral), and the dot product q . k_new
  const float m_own = t < nsplit ? mlq[2 * t] : -INFINITY, l_own = t < nsplit ? mlq[2 * t + 1] : 0.f;
  float m_loc = m_own;
  float dot = t < hd ? q[((size_t)r * heads + h) * hd + t] * knew[((size_t)r * kv_heads + kvh) * hd + t] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    m_loc = fmaxf(m_loc, __shfl_xor_sync(0xFFFFFFFFu, m_loc, o));
    dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
  }
  if (lane == 0) { red[warp] = m_loc; red2[warp] = dot; }
  __syncthreads();
  if (warp == 0) {
    float M = red[lane], dsum = red2[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
      dsum += __shfl_xor_sync(0xFFFFFFFFu, dsum, o);
    }
    if (lane == 0) {
      const float s_self = dsum * rsqrtf((float)hd);
      M = fmaxf(M, s_self);
      s_M = M;
      s_wself = __expf(s_self - M);
    }
  }
  __syncthreads();
  const float w_own = t < nsplit ? __expf(m_own - s_M) : 0.f;
  if (t < nsplit) wsh[t] = w_own;
  float den_loc = w_own * l_own;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) den_loc += __shfl_xor_sync(0xFFFFFFFFu, den_loc, o);
  if (lane == 0) red[warp] = den_loc;
  __syncthreads();
  if (warp == 0) {
    float den = red[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xFFFFFFFFu, den, o);
    if (lane == 0) s_den = den + s_wself;
  }
  // thread (d, grp): dimension d over the blocks grp, grp + ngrp, ...
  const int ngrp = AT_MT / hd, d = t % hd, grp = t / hd;
  const float *pq = part + ((size_t)kvh * NQ + qi) * nsplit * hd + d;
  float num = 0.f;
  int s = grp;
  for (; s + 7 * ngrp < nsplit; s += 8 * ngrp) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = __ldcg(pq + (size_t)(s + j * ngrp) * hd);
#pragma unroll
    for (int j = 0; j < 8; j++) num += wsh[s + j * ngrp] * v[j];
  }
  for (; s < nsplit; s += ngrp) num += wsh[s] * __ldcg(pq + (size_t)s * hd);
  acc[t] = num;
  __syncthreads();
  if (t < hd) {
    float tot = s_wself * vnew[((size_t)r * kv_heads + kvh) * hd + t];
    for (int gI = 0; gI < ngrp; gI++) tot += acc[gI * hd + t];
    out[((size_t)r * heads + h) * hd + t] = tot / s_den;
  }
}

size_t attn_scratch_bytes(int rows, int heads, int hd, int T) {
  const size_t nsplit = T / AT_PB_MIN;  // the smallest block = the most partial results
  return (size_t)rows * heads * nsplit * (hd + 2) * 4 + 256;
}

static size_t attn_smem_bytes(int hd, int pb) { return (size_t)(2 * pb * (hd + 8) + AT_QCAP * (hd + 8) + 2 * 16 * (pb + 8)) * 2 + 2 * 128 * 4; }

// positions per block: the largest of 256, 128, 64 that divides the cache length, fits shared memory and leaves at least
// 120 CTAs (most of the GPU's SMs) unless a smaller block does not either
static int attn_block(int T, int hd, int kv_heads) {
  for (int pb = 256; pb > AT_PB_MIN; pb >>= 1)
    if (T % pb == 0 && attn_smem_bytes(hd, pb) <= 200 * 1024 && (T / pb) * kv_heads >= 120) return pb;
  return AT_PB_MIN;
}

template <int HD, int PB>
static void launch_attn_partial(const float *q, const __half *kc, const __half *vc, int rows, int heads, int kv_heads, int nsplit, float *part, float *ml,
                                cudaStream_t st) {
  const size_t smem = attn_smem_bytes(HD, PB);
  IJ_CUDA(cudaFuncSetAttribute(attn_partial_kernel<HD, PB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  launch_pdl(attn_partial_kernel<HD, PB>, dim3(nsplit, kv_heads), dim3(AT_THREADS), smem, st, q, kc, vc, rows, heads, kv_heads, nsplit, part, ml);
}
template <int HD>
static void launch_attn_partial_pb(int pb, const float *q, const __half *kc, const __half *vc, int rows, int heads, int kv_heads, int nsplit, float *part,
                                   float *ml, cudaStream_t st) {
  if constexpr (HD <= 128) {
    if (pb == 256) return launch_attn_partial<HD, 256>(q, kc, vc, rows, heads, kv_heads, nsplit, part, ml, st);
  }
  if (pb == 128) return launch_attn_partial<HD, 128>(q, kc, vc, rows, heads, kv_heads, nsplit, part, ml, st);
  IJ_CHECK(pb == 64, "attention stand-in: block of %d positions", pb);
  launch_attn_partial<HD, 64>(q, kc, vc, rows, heads, kv_heads, nsplit, part, ml, st);
}

void launch_attn_standin(const float *q, const float *knew, const float *vnew, const __half *kc, const __half *vc, int rows, int heads, int kv_heads,
                         int hd, int T, float *out, void *scratch, cudaStream_t st) {
  IJ_CHECK(T % AT_PB_MIN == 0 && T >= AT_PB_MIN && T / AT_PB_MIN <= AT_MAXSPLIT, "attention stand-in: cache length %d must be a multiple of %d, at most %d",
           T, AT_PB_MIN, AT_PB_MIN * AT_MAXSPLIT);
  IJ_CHECK(heads % kv_heads == 0 && (hd == 64 || hd == 128 || hd == 256), "attention stand-in: heads %d / %d, head dim %d not supported", heads, kv_heads, hd);
  const int pb = attn_block(T, hd, kv_heads), nsplit = T / pb;
  float *part = (float *)scratch;
  float *ml = part + (size_t)rows * heads * nsplit * hd;
  switch (hd) {
    case 64: launch_attn_partial_pb<64>(pb, q, kc, vc, rows, heads, kv_heads, nsplit, part, ml, st); break;
    case 128: launch_attn_partial_pb<128>(pb, q, kc, vc, rows, heads, kv_heads, nsplit, part, ml, st); break;
    default: launch_attn_partial_pb<256>(pb, q, kc, vc, rows, heads, kv_heads, nsplit, part, ml, st); break;
  }
  launch_pdl(attn_merge_kernel, dim3(rows * heads), dim3(AT_MT), 0, st, q, knew, vnew, (const float *)part, (const float *)ml, rows, heads, kv_heads, hd,
             nsplit, out);
}

// =============================================================================================== LM head
__global__ void to_bf16_kernel(const float *__restrict__ x, uint16_t *__restrict__ y, size_t n) {
  pdl_launch();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) y[i] = float_to_bf16_bits(x[i]);
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One warp per 16 vocabulary rows, 8 warps per CTA. The head is streamed from global memory straight into the A fragments
// (each lane reads 16 contiguous bytes of rows g and g + 8 per 32 k: the k order inside a step is permuted the same way
// for both operands, which a dot product does not mind); the activations (bf16) are staged per block of 256 k in shared
// memory for all rows. NT = 8-row groups of activations.
constexpr int LH_KB = 256;
template <int NT>
__global__ void __launch_bounds__(256) lm_head_kernel(const uint16_t *__restrict__ xb, const uint16_t *__restrict__ head, int vocab, int H, int rows,
                                                      float *__restrict__ logits) {
  constexpr int LDX = LH_KB + 8;  // halfs per staged row (+16 bytes: the lanes' 16-byte reads of 8 rows fall on distinct banks)
  constexpr int XS_BYTES = NT * 8 * LDX * 2, OUT_BYTES = 8 * NT * 8 * 17 * 4;
  __shared__ __align__(16) unsigned char lh_buf[XS_BYTES > OUT_BYTES ? XS_BYTES : OUT_BYTES];  // staged activations, later the output transpose
  uint16_t *xs = reinterpret_cast<uint16_t *>(lh_buf);
  float(*outt)[NT * 8][17] = reinterpret_cast<float(*)[NT * 8][17]>(lh_buf);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, qq = lane & 3;
  const int v0 = (blockIdx.x * 8 + warp) * 16;
  const uint16_t *w0 = head + (size_t)min(v0 + g, vocab - 1) * H + 8 * qq;
  const uint16_t *w1 = head + (size_t)min(v0 + g + 8, vocab - 1) * H + 8 * qq;
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; n++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[n][j] = 0.f;
  pdl_launch();
  pdl_wait();
  for (int kb = 0; kb < H; kb += LH_KB) {
    __syncthreads();
    for (int i = threadIdx.x; i < NT * 8 * (LH_KB / 8); i += 256) {
      const int r = i / (LH_KB / 8), c = i % (LH_KB / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < rows) v = *reinterpret_cast<const uint4 *>(xb + (size_t)r * H + kb + c * 8);
      *reinterpret_cast<uint4 *>(xs + r * LDX + c * 8) = v;
    }
    __syncthreads();
    uint4 wa[LH_KB / 32], wb[LH_KB / 32];
#pragma unroll
    for (int ks = 0; ks < LH_KB / 32; ks++) {
      wa[ks] = __ldg(reinterpret_cast<const uint4 *>(w0 + kb + ks * 32));
      wb[ks] = __ldg(reinterpret_cast<const uint4 *>(w1 + kb + ks * 32));
    }
#pragma unroll
    for (int ks = 0; ks < LH_KB / 32; ks++) {
#pragma unroll
      for (int n = 0; n < NT; n++) {
        const uint4 b = *reinterpret_cast<const uint4 *>(xs + (n * 8 + g) * LDX + ks * 32 + 8 * qq);
        mma_bf16_16816(acc[n], wa[ks].x, wb[ks].x, wa[ks].y, wb[ks].y, b.x, b.y);
        mma_bf16_16816(acc[n], wa[ks].z, wb[ks].z, wa[ks].w, wb[ks].w, b.z, b.w);
      }
    }
  }
  // acc[n]: (vocab row g, activation rows 8n + 2qq, +1), (vocab row g + 8, the same rows): transpose through shared memory
  __syncthreads();  // every warp is done with the staged activations
#pragma unroll
  for (int n = 0; n < NT; n++) {
    outt[warp][n * 8 + 2 * qq][g] = acc[n][0];
    outt[warp][n * 8 + 2 * qq + 1][g] = acc[n][1];
    outt[warp][n * 8 + 2 * qq][g + 8] = acc[n][2];
    outt[warp][n * 8 + 2 * qq + 1][g + 8] = acc[n][3];
  }
  __syncwarp();
  for (int i = lane; i < rows * 16; i += 32) {
    const int r = i >> 4, c = i & 15;
    if (v0 + c < vocab) logits[(size_t)r * vocab + v0 + c] = outt[warp][r][c];
  }
}

size_t lm_head_scratch_bytes(int rows, int H) { return (size_t)rows * H * 2 + 256; }

void launch_lm_head(const float *xn, const uint16_t *head_bf16, int vocab, int H, int rows, float *logits, void *scratch, cudaStream_t st) {
  IJ_CHECK(rows >= 1 && rows <= 64 && H % LH_KB == 0, "LM head: rows %d outside 1..64 or hidden %d not a multiple of %d", rows, H, LH_KB);
  uint16_t *xb = (uint16_t *)scratch;
  launch_pdl(to_bf16_kernel, dim3(std::min(64, (rows * H + 255) / 256)), dim3(256), 0, st, xn, xb, (size_t)rows * H);
  const dim3 grid((vocab + 127) / 128), block(256);
  const uint16_t *xc = xb;
  if (rows <= 8) launch_pdl(lm_head_kernel<1>, grid, block, 0, st, xc, head_bf16, vocab, H, rows, logits);
  else if (rows <= 16) launch_pdl(lm_head_kernel<2>, grid, block, 0, st, xc, head_bf16, vocab, H, rows, logits);
  else if (rows <= 32) launch_pdl(lm_head_kernel<4>, grid, block, 0, st, xc, head_bf16, vocab, H, rows, logits);
  else launch_pdl(lm_head_kernel<8>, grid, block, 0, st, xc, head_bf16, vocab, H, rows, logits);
}

// =============================================================================================== greedy sampling
__global__ void __launch_bounds__(256) argmax_part_kernel(const float *__restrict__ logits, int vocab, float *__restrict__ pv, int *__restrict__ pi) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int r = blockIdx.y, per = (vocab + ARGMAX_BLOCKS - 1) / ARGMAX_BLOCKS, lo = blockIdx.x * per, hi = min(vocab, lo + per);
  float best = -INFINITY;
  int bi = 0x7FFFFFFF;
  pdl_launch();
  pdl_wait();
  for (int i = lo + threadIdx.x; i < hi; i += 256) {
    const float v = logits[(size_t)r * vocab + i];
    if (v > best) { best = v; bi = i; }  // ascending i: the first maximum wins
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
    const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    pv[r * ARGMAX_BLOCKS + blockIdx.x] = best;
    pi[r * ARGMAX_BLOCKS + blockIdx.x] = bi;
  }
}
__global__ void argmax_final_kernel(const float *__restrict__ pv, const int *__restrict__ pi, int *__restrict__ next) {
  const int r = blockIdx.x, lane = threadIdx.x;
  float best = -INFINITY;
  int bi = 0x7FFFFFFF;
  pdl_launch();
  pdl_wait();
  for (int i = lane; i < ARGMAX_BLOCKS; i += 32) {
    const float v = pv[r * ARGMAX_BLOCKS + i];
    const int id = pi[r * ARGMAX_BLOCKS + i];
    if (v > best || (v == best && id < bi)) { best = v; bi = id; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
    const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) next[r] = bi;
}

void launch_argmax(const float *logits, int vocab, int rows, int *next, void *scratch, cudaStream_t st) {
  float *pv = (float *)scratch;
  int *pi = (int *)(pv + (size_t)rows * ARGMAX_BLOCKS);
  launch_pdl(argmax_part_kernel, dim3(ARGMAX_BLOCKS, rows), dim3(256), 0, st, logits, vocab, pv, pi);
  launch_pdl(argmax_final_kernel, dim3(rows), dim3(32), 0, st, (const float *)pv, (const int *)pi, next);
}

// =============================================================================================== synthetic weights
__device__ __forceinline__ uint64_t mix64(uint64_t z) {  // splitmix64 finaliser
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float unit_normal(uint64_t h) {  // Box-Muller on the two halves of a hash
  const float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f), u2 = (float)(uint32_t)((h >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
  return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}
template <int MODE>  // 0 trellis words (4 per hash), 1 signs f16, 2 scales f16, 3 normal bf16, 4 normal f16
__global__ void fill_kernel(uint16_t *dst, size_t n, float scale, uint64_t seed, size_t first) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  if constexpr (MODE == 0) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i * 4 < n; i += stride) {
      const uint64_t h = mix64(seed ^ ((first / 4 + i) * 0xD1B54A32D192ED03ull));
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (i * 4 + j < n) dst[i * 4 + j] = (uint16_t)(h >> (16 * j));
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const uint64_t h = mix64(seed ^ ((first + i) * 0xD1B54A32D192ED03ull));
      if (MODE == 1) dst[i] = (h & 1) ? 0x3C00u : 0xBC00u;
      else if (MODE == 2) dst[i] = __half_as_ushort(__float2half_rn(((h & 1) ? 1.0f : -1.0f) * fabsf(unit_normal(h)) * scale));
      else if (MODE == 3) dst[i] = float_to_bf16_bits(unit_normal(h) * scale);
      else dst[i] = __half_as_ushort(__float2half_rn(unit_normal(h) * scale));
    }
  }
}
template <int MODE>
static void fill(void *dst, size_t n, float scale, uint64_t seed, cudaStream_t st, size_t first) {
  if (n == 0) return;
  IJ_CHECK(MODE != 0 || first % 4 == 0, "trellis fill offset must be a multiple of 4 words");
  const size_t work = MODE == 0 ? (n + 3) / 4 : n;
  fill_kernel<MODE><<<(unsigned)std::min<size_t>((work + 255) / 256, 148 * 16), 256, 0, st>>>((uint16_t *)dst, n, scale, seed, first);
  IJ_CUDA(cudaGetLastError());
}
void fill_trellis(void *dst, size_t n_u16, uint64_t seed, cudaStream_t st, size_t first) { fill<0>(dst, n_u16, 0.f, seed, st, first); }
void fill_signs_f16(void *dst, size_t n, uint64_t seed, cudaStream_t st, size_t first) { fill<1>(dst, n, 0.f, seed, st, first); }
void fill_scales_f16(void *dst, size_t n, float scale, uint64_t seed, cudaStream_t st, size_t first) { fill<2>(dst, n, scale, seed, st, first); }
void fill_normal_bf16(void *dst, size_t n, float scale, uint64_t seed, cudaStream_t st, size_t first) { fill<3>(dst, n, scale, seed, st, first); }
void fill_normal_f16(void *dst, size_t n, float scale, uint64_t seed, cudaStream_t st, size_t first) { fill<4>(dst, n, scale, seed, st, first); }

}  // namespace ijah
