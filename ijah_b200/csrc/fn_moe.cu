// Decode MoE block kernels. See fn_moe.cuh.
#include <algorithm>
#include <cmath>

#include "common.hpp"
#include "fn_moe.cuh"
#include "launch.cuh"

namespace ijah {

// =============================================================================================== router + top-k + plan
// Reference: kernels/fn_moe.metal:26-134 (logits = x . W in fp32 from bf16 weights, shared-gate logit as row E;
// the last CTA to arrive selects top-k on the logits, ties -> lowest index, w = exp(l - l_max) / sum over the k).
constexpr int RT_WARPS = 8;    // expert rows per CTA (one per warp): every CTA stages all activation rows, so fewer, fuller CTAs read them less often
constexpr int RT_THREADS = 256;
constexpr int RT_RC = 8;       // activation rows per pass
constexpr int RT_EMAX = 1024;  // experts the finisher covers (32 logits per lane)
constexpr int RT_PMAX = 2048;  // (row, slot) pairs the finisher covers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// k-split partial sums of NP * 4 elements per lane (element j of pointer q: base[q][lane + 32 j] + s * sstride), added in
// split order, four splits' loads in flight at a time (a rolled loop of dependent adds would pay one L2 round trip per split)
template <int NP>
__device__ __forceinline__ void sum_splits(const float *const (&base)[NP], size_t sstride, int S, int lane, float (&acc)[NP][4]) {
#pragma unroll
  for (int q = 0; q < NP; q++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[q][j] = 0.0f;
  for (int s0 = 0; s0 < S; s0 += 4) {
    float t[4][NP][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int q = 0; q < NP; q++)
#pragma unroll
        for (int j = 0; j < 4; j++) t[i][q][j] = s0 + i < S ? __ldcg(base[q] + (size_t)(s0 + i) * sstride + lane + 32 * j) : 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int q = 0; q < NP; q++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[q][j] += t[i][q][j];
  }
}

// float -> unsigned key with the same order (for redux.sync max); -0 was folded into +0 before
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float order_key_inv(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

// Warp-wide selection of the k largest of 32 * NV (value, id) candidates held in registers (NV per lane; unused entries
// are -inf with id INT_MAX). Order: larger value first, ties -> lower id. Per round: two warp reductions (largest value,
// then lowest id among its holders) and a rescan by the winning lane only. Lane t < k returns the t-th winner.
template <int NV>
__device__ __forceinline__ void topk_regs(float (&v)[NV], int (&id)[NV], int k, int lane, float &myv, int &myi) {
  float best = -INFINITY;
  int bid = 0x7FFFFFFF;
#pragma unroll
  for (int j = 0; j < NV; j++)
    if (v[j] > best || (v[j] == best && id[j] < bid)) { best = v[j]; bid = id[j]; }
  for (int t = 0; t < k; t++) {
    const uint32_t key = order_key(best);
    const uint32_t kmax = __reduce_max_sync(0xFFFFFFFFu, key);
    const int cand = key == kmax ? bid : 0x7FFFFFFF;
    const int wi = __reduce_min_sync(0xFFFFFFFFu, cand);
    if (lane == t) { myv = order_key_inv(kmax); myi = wi; }
    if (cand == wi && wi != 0x7FFFFFFF) {  // the winner drops its entry and rescans its registers
      best = -INFINITY; bid = 0x7FFFFFFF;
#pragma unroll
      for (int j = 0; j < NV; j++) {
        if (id[j] == wi) { v[j] = -INFINITY; id[j] = 0x7FFFFFFF; }
        if (v[j] > best || (v[j] == best && id[j] < bid)) { best = v[j]; bid = id[j]; }
      }
    }
  }
}

// candidates n0 .. n0 + n of `vals` (ids: `ids[i]`, or i itself when ids == nullptr), lane-strided, -0 folded into +0
template <int NV>
__device__ __forceinline__ void topk_span(const float *vals, const int *ids, int n0, int n, int k, int lane, float &myv, int &myi) {
  float v[NV];
  int id[NV];
#pragma unroll
  for (int j = 0; j < NV; j++) {
    const int i = j * 32 + lane;
    v[j] = i < n ? (ids ? vals[n0 + i] : __ldcg(vals + n0 + i)) + 0.0f : -INFINITY;  // ids != nullptr: shared memory
    id[j] = i < n ? (ids ? ids[n0 + i] : n0 + i) : 0x7FFFFFFF;
  }
  topk_regs<NV>(v, id, k, lane, myv, myi);
}

__device__ __forceinline__ void topk_any(const float *vals, const int *ids, int n0, int n, int k, int lane, float &myv, int &myi) {
  const int nv = (n + 31) >> 5;
  if (nv <= 1) topk_span<1>(vals, ids, n0, n, k, lane, myv, myi);
  else if (nv <= 2) topk_span<2>(vals, ids, n0, n, k, lane, myv, myi);
  else if (nv <= 4) topk_span<4>(vals, ids, n0, n, k, lane, myv, myi);
  else if (nv <= 8) topk_span<8>(vals, ids, n0, n, k, lane, myv, myi);
  else if (nv <= 16) topk_span<16>(vals, ids, n0, n, k, lane, myv, myi);
  else topk_span<32>(vals, ids, n0, n, k, lane, myv, myi);
}

// lanes t < k hold the row's winners in order: softmax over them, write route[r] (ids, then weights) and sid[r * k ..]
__device__ __forceinline__ void route_row(const MoeParams &p, int r, int *sid, int lane, float myv, int myi) {
  const int k = p.topk;
  const float top = __shfl_sync(0xFFFFFFFFu, myv, 0);
  const float pr = lane < k ? expf(myv - top) : 0.0f;
  const float sum = warp_sum(pr);
  if (lane < k) {
    p.route[(size_t)r * p.ldr + lane] = (uint32_t)myi;
    p.route[(size_t)r * p.ldr + k + lane] = __float_as_uint(pr / sum);
    sid[r * k + lane] = myi;
  }
}

// bitonic sort across the 32 lanes of a warp, descending (lane 0 ends with the largest key): 15 exchange steps
template <class T>
__device__ __forceinline__ T warp_sort_desc(T key, int lane) {
#pragma unroll
  for (int k2 = 2; k2 <= 32; k2 <<= 1) {
#pragma unroll
    for (int j = k2 >> 1; j > 0; j >>= 1) {
      const T other = __shfl_xor_sync(0xFFFFFFFFu, key, j);
      const bool take_max = ((lane & j) == 0) == ((lane & k2) == 0);
      key = take_max ? (key > other ? key : other) : (key < other ? key : other);
    }
  }
  return key;
}

// One warp selects the k <= 32 largest logits of row r (ties -> lowest index) with few dependent warp-wide steps:
// the k-th largest of the 32 per-lane maxima is a lower bound T of the k-th largest logit, so only logits >= T can win.
// Those (normally a handful more than k) are compacted into `list` as 64-bit keys (ordered value, inverted index) and one
// more warp sort puts the winners, in order, into lanes 0 .. k-1. More than 32 candidates (heavy ties): the round-based
// selection takes over. `list`: 32 entries of shared memory owned by the warp.
template <int NV>
__device__ void topk_row(const MoeParams &p, int r, int *sid, unsigned long long *list, int lane) {
  const int E = p.E, k = p.topk, nv = E >> 5;
  const float *lg = p.logits + (size_t)r * (E + 1);
  // all loads go out before the first use (clamped addresses instead of predicates: a guarded load per iteration would
  // serialise one L2 round trip per 32 logits)
  float f[NV];
#pragma unroll
  for (int j = 0; j < NV; j++) f[j] = __ldcg(lg + min(j * 32 + lane, E - 1));
  uint32_t key[NV];
  uint32_t m = 0u;
#pragma unroll
  for (int j = 0; j < NV; j++) {
    key[j] = j < nv ? order_key(f[j] + 0.0f) : 0u;
    m = max(m, key[j]);
  }
  const uint32_t T = __shfl_sync(0xFFFFFFFFu, warp_sort_desc<uint32_t>(m, lane), k - 1);
  // compaction (order is irrelevant, the list is sorted next): per-lane count, exclusive scan over lanes, then each lane
  // writes its own candidates
  int mine = 0;
#pragma unroll
  for (int j = 0; j < NV; j++) mine += (j < nv && key[j] >= T) ? 1 : 0;
  int inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += a;
  }
  const int count = __shfl_sync(0xFFFFFFFFu, inc, 31);
  int pos = inc - mine;
  if (mine > 0) {
#pragma unroll
    for (int j = 0; j < NV; j++) {
      if (j < nv && key[j] >= T) {
        if (pos < 32) list[pos] = ((unsigned long long)key[j] << 32) | (0xFFFFFFFFu - (uint32_t)(j * 32 + lane));
        pos++;
      }
    }
  }
  __syncwarp();
  float myv = 0.0f;
  int myi = 0;
  if (count <= 32) {
    const unsigned long long c = warp_sort_desc<unsigned long long>(lane < count ? list[lane] : 0ull, lane);
    myv = order_key_inv((uint32_t)(c >> 32));
    myi = (int)(0xFFFFFFFFu - (uint32_t)c);
  } else {
    topk_any(lg, nullptr, 0, E, k, lane, myv, myi);
  }
  __syncwarp();
  route_row(p, r, sid, lane, myv, myi);
}

// The local experts that the rows*topk (row, slot) pairs use, in expert order, each with its pairs in row order, cut into
// entries of at most PLAN_ROWS rows: one entry = one pass of the stream kernels over that expert's weights (an expert that
// more than PLAN_ROWS rows selected is streamed once per entry, which at decode widths is rare). One CTA (blockDim a
// multiple of 32, <= 1024); `buf` is 16 KB of shared memory, sid[P] the pairs' expert ids (shared).
__device__ void build_plan_block(const MoeParams &p, unsigned char *buf, const int *sid) {
  unsigned long long *mask = reinterpret_cast<unsigned long long *>(buf);  // [E] rows that use expert e
  int *uidx = reinterpret_cast<int *>(buf + 8 * RT_EMAX);                  // [E] index among present experts
  int *firs = uidx + RT_EMAX;                                              // [E] offset of its pairs
  __shared__ int wtot[32];
  const int tid = threadIdx.x, T = blockDim.x, E = p.E, k = p.topk, P = p.P;
  const int lane = tid & 31, warp = tid >> 5;
  PlanView pv{p.plan, P};
  for (int e = tid; e < E; e += T) mask[e] = 0ull;
  __syncthreads();
  for (int i = tid; i < P; i += T) {
    const int e = sid[i];
    if (e >= p.e0 && e < p.e0 + p.ecount) atomicOr(&mask[e], 1ull << (i / k));
  }
  __syncthreads();
  // exclusive scan over experts of (entries, pair count), packed as (entries << 16) | count (count <= 2048):
  // thread t covers experts [t * per, (t + 1) * per)
  const int per = (E + T - 1) / T, e_lo = tid * per;
  int mine = 0, distinct = 0;
  for (int e = e_lo; e < min(E, e_lo + per); e++) {
    const int c = __popcll(mask[e]);
    mine += (((c + PLAN_ROWS - 1) / PLAN_ROWS) << 16) + c;
    distinct += c > 0 ? 1 : 0;
  }
  int inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += a;
  }
  if (lane == 31) wtot[warp] = inc;
  __syncthreads();
  int run = inc - mine;
  for (int w = 0; w < warp; w++) run += wtot[w];
  if (tid == T - 1) *pv.nu() = (run + mine) >> 16;
  if (tid == 0) *pv.distinct() = 0;
  for (int e = e_lo; e < min(E, e_lo + per); e++) {
    const int c = __popcll(mask[e]);
    if (c > 0) {
      const int u = run >> 16, f = run & 0xFFFF, ng = (c + PLAN_ROWS - 1) / PLAN_ROWS;
      firs[e] = f;
      for (int g = 0; g < ng; g++) {
        pv.expert()[u + g] = e;
        pv.nrows()[u + g] = min(PLAN_ROWS, c - g * PLAN_ROWS);
        pv.first()[u + g] = f + g * PLAN_ROWS;
      }
      run += (ng << 16) + c;
    }
  }
  (void)uidx;
  __syncthreads();
  if (distinct) atomicAdd(pv.distinct(), distinct);
  __syncthreads();
  for (int i = tid; i < P; i += T) {
    const int r = i / k, e = sid[i];
    if (e >= p.e0 && e < p.e0 + p.ecount) pv.pairs()[firs[e] + __popcll(mask[e] & ((1ull << r) - 1ull))] = i;
  }
}

// acc[t] = W row (16 x 8 bf16 per lane, chunk j covers elements [8 (32 j + lane), +8)) . activation row t of the staged pass,
// for NR rows at once (rows >= nr repeat row nr - 1: no branches between the shared-memory loads)
template <int NR>
__device__ __forceinline__ void router_dot(const uint4 (&wreg)[16], const float *dyn, int H, int lane, int nr, float (&acc)[RT_RC]) {
#pragma unroll
  for (int t = 0; t < RT_RC; t++) acc[t] = 0.0f;
  const float4 *x4 = reinterpret_cast<const float4 *>(dyn);
  const int q = H / 4, h8 = H / 8;
#pragma unroll
  for (int j = 0; j < 16; j++) {
    const int c = j * 32 + lane;
    if (j * 32 < h8) {  // uniform (H is a multiple of 256)
      const uint4 u = wreg[j];
      const float w0 = __uint_as_float(u.x << 16), w1 = __uint_as_float(u.x & 0xFFFF0000u);
      const float w2 = __uint_as_float(u.y << 16), w3 = __uint_as_float(u.y & 0xFFFF0000u);
      const float w4_ = __uint_as_float(u.z << 16), w5 = __uint_as_float(u.z & 0xFFFF0000u);
      const float w6 = __uint_as_float(u.w << 16), w7 = __uint_as_float(u.w & 0xFFFF0000u);
#pragma unroll
      for (int t = 0; t < NR; t++) {
        const int tt = min(t, nr - 1);
        const float4 a = x4[tt * q + c], b = x4[tt * q + h8 + c];
        acc[t] += a.x * w0 + a.y * w1 + a.z * w2 + a.w * w3 + b.x * w4_ + b.y * w5 + b.z * w6 + b.w * w7;
      }
    }
  }
}

// Dynamic shared memory: first the activation rows of one pass (RT_RC rows x H floats, shared by the CTA's expert
// rows), later reused by the finisher (the plan's tables, then the pairs' expert ids).
__global__ void __launch_bounds__(RT_THREADS) moe_router_kernel(const MoeParams p, int build_plan) {
  extern __shared__ __align__(16) float dyn[];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * RT_WARPS + warp;
  const int H = p.H, E = p.E;
  const uint16_t *wr = warp >= RT_WARPS ? nullptr : row < E ? p.router + (size_t)row * H : (row == E ? p.sgate : nullptr);
  // the expert's weight row stays in registers for all passes: H / 256 x 8 bf16 per lane (H <= 4096)
  // (clamped addresses, no predicates: all 16 loads are in flight at once; the dot loop skips the chunks past H / 8)
  uint4 wreg[16];
  const uint4 *wsrc = reinterpret_cast<const uint4 *>(wr != nullptr ? wr : p.router);
#pragma unroll
  for (int j = 0; j < 16; j++) wreg[j] = __ldg(wsrc + min(j * 32 + lane, H / 8 - 1));
  pdl_launch();
  pdl_wait();  // the router weights above are static; the activations may be the preceding kernel's output
  for (int r0 = 0; r0 < p.rows; r0 += RT_RC) {
    const int nr = min(RT_RC, p.rows - r0);
    __syncthreads();
    {  // asynchronous 16-byte copies: every thread's share is in flight at once
      const uint32_t dst = smem_u32(dyn);
      const float4 *src = reinterpret_cast<const float4 *>(p.x + (size_t)r0 * H);
      // row t, floats [8c, 8c+4) go to float4 slot t * H/4 + c, floats [8c+4, 8c+8) to slot t * H/4 + H/8 + c: a warp's
      // 16-byte reads of either half are then contiguous (no bank conflicts)
      const int q = H / 4, h8 = H / 8;
      for (int t = 0; t < nr; t++)
        for (int w = threadIdx.x; w < q; w += blockDim.x) {
          const int slot = t * q + (w & 1) * h8 + (w >> 1);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)slot * 16u), "l"(src + t * q + w) : "memory");
        }
      asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (wr == nullptr) continue;
    float acc[RT_RC];
    if (nr == 1) router_dot<1>(wreg, dyn, H, lane, nr, acc);
    else if (nr == 2) router_dot<2>(wreg, dyn, H, lane, nr, acc);
    else if (nr <= 4) router_dot<4>(wreg, dyn, H, lane, nr, acc);
    else router_dot<8>(wreg, dyn, H, lane, nr, acc);
#pragma unroll
    for (int t = 0; t < RT_RC; t++) {
      if (t < nr) {  // uniform
        const float v = warp_sum(acc[t]);
        if (lane == 0 && row <= E) p.logits[(size_t)(r0 + t) * (E + 1) + row] = v;
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.counter, 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!s_last) return;  // the finisher reads the other CTAs' logits with L2 loads (ld.global.cg), past their fences
  unsigned char *tables = reinterpret_cast<unsigned char *>(dyn);
  int *sid = reinterpret_cast<int *>(tables + 16 * RT_EMAX);
  unsigned long long *lists = reinterpret_cast<unsigned long long *>(tables + 16 * RT_EMAX + 4 * RT_PMAX);
  for (int r = warp; r < p.rows; r += RT_THREADS / 32) {
    if (p.E <= 512) topk_row<16>(p, r, sid, lists + warp * 32, lane);
    else topk_row<32>(p, r, sid, lists + warp * 32, lane);
  }
  __syncthreads();
  if (build_plan) build_plan_block(p, tables, sid);
  if (threadIdx.x == 0) *p.counter = 0u;
}

void launch_moe_router(const MoeParams &p, bool build_plan, cudaStream_t st) {
  IJ_CHECK(p.E <= RT_EMAX && p.E % 32 == 0 && p.H % 256 == 0 && p.topk <= 32, "router: unsupported dims E %d H %d k %d", p.E, p.H, p.topk);
  IJ_CHECK(p.H <= 4096, "router: hidden %d > 4096", p.H);
  IJ_CHECK(p.P <= RT_PMAX, "router: %d (row, slot) pairs > %d", p.P, RT_PMAX);
  const int grid = (p.E + 1 + RT_WARPS - 1) / RT_WARPS;
  const size_t smem = std::max((size_t)std::min(p.rows, RT_RC) * p.H * 4, (size_t)16 * RT_EMAX + (size_t)RT_PMAX * 4 + 2048);  // tables, pair ids, candidate lists
  IJ_CUDA(cudaFuncSetAttribute(moe_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_RC * 4096 * 4));  // per device: every launch
  launch_pdl(moe_router_kernel, dim3(grid), dim3(RT_THREADS), smem, st, p, build_plan ? 1 : 0);
}

// =============================================================================================== operand prep
// xh_gu[pair][proj][H] = fp16(H128(x[row(pair)] * suh_proj[expert(pair)])) for every local (row, slot) pair, and
// xh_sgu[row][proj][H] for the shared expert (reference kernels/fn_moe.metal:304-311, prefill twin
// kernels/prefill/pf_moe.metal:88-104). One warp per (operand row, 128-element chunk). With build_plan, one extra CTA
// (the last blockIdx.y) builds the expert plan of the stream kernels meanwhile: the plan needs the routes, not the operands.
__global__ void __launch_bounds__(128) moe_prep_kernel(const MoeParams p, int build_plan) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x * 4 + warp, job = blockIdx.y;  // job < P: routed pair; else shared row
  const int H = p.H, k = p.topk;
  pdl_wait();
  pdl_launch();
  if (build_plan && blockIdx.y == gridDim.y - 1) {
    __shared__ __align__(16) unsigned char tables[16 * RT_EMAX];
    __shared__ int sid[RT_PMAX];
    if (blockIdx.x != 0) return;
    for (int i = threadIdx.x; i < p.P; i += blockDim.x) sid[i] = (int)p.route[(size_t)(i / k) * p.ldr + (i % k)];
    __syncthreads();
    build_plan_block(p, tables, sid);
    return;
  }
  if (chunk * 128 >= H) return;
  const float hs = 0.08838834764831845f;
  int r;
  const __half *sg, *su;
  __half *dst;
  if (job < p.P) {
    r = job / k;
    const int e = (int)p.route[(size_t)r * p.ldr + (job - r * k)] - p.e0;
    if (e < 0 || e >= p.ecount) return;
    sg = p.gate.suh + (size_t)e * H;
    su = p.up.suh + (size_t)e * H;
    dst = p.xh_gu + (size_t)job * 2 * H * A_HALFS_PER_INPUT;
  } else {
    r = job - p.P;
    sg = p.sgt.suh;
    su = p.sup.suh;
    dst = p.xh_sgu + (size_t)r * 2 * H * A_HALFS_PER_INPUT;
  }
  const int o = chunk * 128 + lane;
  float xv[4], v[4];
#pragma unroll
  for (int j = 0; j < 4; j++) xv[j] = p.x[(size_t)r * p.ldx + o + 32 * j];
#pragma unroll
  for (int j = 0; j < 4; j++) v[j] = xv[j] * __half2float(sg[o + 32 * j]);
  fwht_chunk(v, lane, 128, hs);
#pragma unroll
  for (int j = 0; j < 4; j++) store_a(dst, o + 32 * j, v[j], p.dup);
#pragma unroll
  for (int j = 0; j < 4; j++) v[j] = xv[j] * __half2float(su[o + 32 * j]);
  fwht_chunk(v, lane, 128, hs);
#pragma unroll
  for (int j = 0; j < 4; j++) store_a(dst + H * A_HALFS_PER_INPUT, o + 32 * j, v[j], p.dup);
}

// xh_d[pair][I] = fp16(H128(silu(g) * u * suh_down)), g = H128(sum_s raw gate) * svh_gate, u likewise
// (reference kernels/fn_moe.metal:370-384, kernels/prefill/pf_moe.metal:107-125). One warp per (pair | shared row,
// 128-element chunk of the intermediate).
__global__ void __launch_bounds__(128) moe_mid_kernel(const MoeParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x * 4 + warp, job = blockIdx.y;
  const int I = p.I, k = p.topk;
  pdl_launch();  // the down kernel's CTAs may take the places the gate/up kernel's CTAs leave and stream their first weights
  pdl_wait();
  if (chunk * 128 >= I) return;
  const float hs = 0.08838834764831845f;
  const bool shared = job >= p.P;
  // the partial sums' addresses do not depend on the routing: their loads go out first, together with the route entry
  const float *raw = shared ? p.raw_sgu + (size_t)(job - p.P) * 2 * I : p.raw_gu + (size_t)job * 2 * I;
  const size_t sstride = shared ? (size_t)p.rows * 2 * I : (size_t)p.P * 2 * I;
  const int o = chunk * 128 + lane;
  const float *const src[2] = {raw + chunk * 128, raw + I + chunk * 128};
  float gu[2][4];
  sum_splits<2>(src, sstride, p.S_gu, lane, gu);
  const __half *svg, *svu, *sud;
  __half *dst;
  if (!shared) {
    const int r = job / k, e = (int)p.route[(size_t)r * p.ldr + (job - r * k)] - p.e0;
    if (e < 0 || e >= p.ecount) return;
    svg = p.gate.svh + (size_t)e * I; svu = p.up.svh + (size_t)e * I; sud = p.down.suh + (size_t)e * I;
    dst = p.xh_d + (size_t)job * I * A_HALFS_PER_INPUT;
  } else {
    svg = p.sgt.svh; svu = p.sup.svh; sud = p.sdn.suh;
    dst = p.xh_sd + (size_t)(job - p.P) * I * A_HALFS_PER_INPUT;
  }
  float gv[4], uv[4], hh[4], s_g[4], s_u[4], s_d[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    gv[j] = gu[0][j]; uv[j] = gu[1][j];
    s_g[j] = __half2float(svg[o + 32 * j]); s_u[j] = __half2float(svu[o + 32 * j]); s_d[j] = __half2float(sud[o + 32 * j]);
  }
  fwht_chunk(gv, lane, 128, hs);
  fwht_chunk(uv, lane, 128, hs);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    gv[j] *= s_g[j];
    uv[j] *= s_u[j];
    hh[j] = gv[j] / (1.0f + expf(-gv[j])) * uv[j] * s_d[j];
  }
  if (shared) {  // finished shared gate | up, kept for inspection ("shared_gu")
    const int r = job - p.P;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      p.gush[(size_t)r * 2 * I + o + 32 * j] = gv[j];
      p.gush[(size_t)r * 2 * I + I + o + 32 * j] = uv[j];
    }
  }
  fwht_chunk(hh, lane, 128, hs);
#pragma unroll
  for (int j = 0; j < 4; j++) store_a(dst, o + 32 * j, hh[j], p.dup);
}

// =============================================================================================== gate / up
// Unit order: for each distinct expert u: proj (gate, up) x k-split x column group; then the shared expert's.
struct MoeGateUpProblem {
  // The plan is final at launch when the router kernel wrote it (the operand prep in between only lets this launch go
  // once the router has completed); when the prep kernel itself builds the plan (routes from outside) it is not.
  __device__ bool units_final() const { return plan_final != 0; }
  struct Unit : UnitBase {
    int s, k0, g, proj, shared, e, first;
  };
  alignas(64) CUtensorMap maps[4];  // gate, up, shared gate, shared up
  MoeParams p;
  int IT, OT, NG, S, kc, plan_final;

  __device__ const CUtensorMap *tmap(int i) const { return &maps[i]; }

  __device__ int shared_groups() const { return p.has_shared ? (p.sh_rows + PLAN_ROWS - 1) / PLAN_ROWS : 0; }
  __device__ int num_units() const { return (*PlanView{p.plan, p.P}.nu() + shared_groups()) * 2 * S * NG; }
  __device__ Unit unit(int u) const {
    const PlanView pv{p.plan, p.P};
    Unit un;
    const int per = 2 * S * NG, q = u / per, rem = u - q * per;
    un.proj = rem / (S * NG);
    un.s = (rem / NG) % S;
    un.g = rem % NG;
    un.k0 = un.s * kc;
    un.kc = min(kc, IT - un.k0);
    un.ntiles = min(SG_WARPS, OT - un.g * SG_WARPS);
    un.shared = q >= *pv.nu();
    if (un.shared) {  // only the rows whose shared expert runs here, PLAN_ROWS at a time
      un.e = 0; un.first = (q - *pv.nu()) * PLAN_ROWS; un.nrows = min(PLAN_ROWS, p.sh_rows - un.first); un.K = p.Ks;
      un.map = 2 + un.proj;
    } else {
      un.e = pv.expert()[q] - p.e0; un.first = pv.first()[q]; un.nrows = pv.nrows()[q]; un.K = p.Kx;
      un.map = un.proj;
    }
    un.x = un.g * SG_WARPS * 4 * un.K; un.y = un.k0; un.z = un.e;
    return un;
  }
  // row index = the (row, slot) pair for routed units, the activation row for the shared expert
  __device__ int row_index(const Unit &un, int i) const {
    return un.shared ? p.sh_row0 + un.first + i : PlanView{p.plan, p.P}.pairs()[un.first + i];
  }
  __device__ const __half *a_row(const Unit &un, int idx) const {
    return (un.shared ? p.xh_sgu : p.xh_gu) + (((size_t)idx * 2 + un.proj) * p.H + un.k0 * 16) * A_HALFS_PER_INPUT;
  }
  __device__ float *out_base(const Unit &un) const {
    return (un.shared ? p.raw_sgu + ((size_t)un.s * p.rows * 2 + un.proj) * p.I : p.raw_gu + ((size_t)un.s * p.P * 2 + un.proj) * p.I) + un.g * 128;
  }
  __device__ int out_row_off(const Unit &, int idx) const { return idx * 2 * p.I; }
};

// =============================================================================================== down
struct MoeDownProblem {
  // the plan was complete before the gate/up kernel started, i.e. before the predecessor (mid) could release this launch
  __device__ bool units_final() const { return true; }
  struct Unit : UnitBase {
    int s, k0, g, shared, e, first;
  };
  alignas(64) CUtensorMap maps[2];  // down, shared down
  MoeParams p;
  int IT, OT, NG, S, kc;  // IT = I/16, OT = H/16

  __device__ const CUtensorMap *tmap(int i) const { return &maps[i]; }

  __device__ int shared_groups() const { return p.has_shared ? (p.sh_rows + PLAN_ROWS - 1) / PLAN_ROWS : 0; }
  __device__ int num_units() const { return (*PlanView{p.plan, p.P}.nu() + shared_groups()) * S * NG; }
  __device__ Unit unit(int u) const {
    const PlanView pv{p.plan, p.P};
    Unit un;
    const int per = S * NG, q = u / per, rem = u - q * per;
    un.s = rem / NG;
    un.g = rem % NG;
    un.k0 = un.s * kc;
    un.kc = min(kc, IT - un.k0);
    un.ntiles = min(SG_WARPS, OT - un.g * SG_WARPS);
    un.shared = q >= *pv.nu();
    if (un.shared) { un.e = 0; un.first = (q - *pv.nu()) * PLAN_ROWS; un.nrows = min(PLAN_ROWS, p.sh_rows - un.first); un.K = p.Ks; }
    else { un.e = pv.expert()[q] - p.e0; un.first = pv.first()[q]; un.nrows = pv.nrows()[q]; un.K = p.Kx; }
    un.map = un.shared ? 1 : 0;
    un.x = un.g * SG_WARPS * 4 * un.K; un.y = un.k0; un.z = un.e;
    return un;
  }
  __device__ int row_index(const Unit &un, int i) const {
    return un.shared ? p.sh_row0 + un.first + i : PlanView{p.plan, p.P}.pairs()[un.first + i];
  }
  __device__ const __half *a_row(const Unit &un, int idx) const {
    return (un.shared ? p.xh_sd : p.xh_d) + ((size_t)idx * p.I + un.k0 * 16) * A_HALFS_PER_INPUT;
  }
  __device__ float *out_base(const Unit &un) const {
    return (un.shared ? p.raw_sd + (size_t)un.s * p.rows * p.H : p.raw_d + (size_t)un.s * p.P * p.H) + un.g * 128;
  }
  __device__ int out_row_off(const Unit &, int idx) const { return idx * p.H; }
};

// =============================================================================================== combine
// One CTA per (row, 128-column block), one warp per slot plus one for the shared expert (reference
// kernels/fn_moe.metal:411-451, kernels/prefill/pf_moe.metal:129-161): every slot's raw down output gets
// H * svh_down * w_k into shared memory; warp 0 then sums the slots in slot order, adds
// sigmoid(shared-gate logit) * shared down and applies the optional hyper-connection write.
constexpr int CB_MAXK = 16;
__global__ void __launch_bounds__(32 * (CB_MAXK + 1)) moe_combine_kernel(const MoeParams p, int routed_only) {
  __shared__ float vals[CB_MAXK + 1][128];
  __shared__ int used[CB_MAXK + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int blk = blockIdx.x, r = blockIdx.y;
  const int H = p.H, k = p.topk;
  pdl_launch();
  pdl_wait();
  const float hs = 0.08838834764831845f;
  if (warp < k) {
    // the partial sums' addresses do not depend on the routing: their loads go out together with the route entry
    const float *const src[1] = {p.raw_d + (size_t)(r * k + warp) * H + blk * 128};
    float part[1][4];
    sum_splits<1>(src, (size_t)p.P * H, p.S_d, lane, part);
    const int e = (int)p.route[(size_t)r * p.ldr + warp];
    const float wk = __uint_as_float(p.route[(size_t)r * p.ldr + k + warp]);
    const bool local = e >= p.e0 && e < p.e0 + p.ecount;
    if (lane == 0) used[warp] = local ? 1 : 0;
    if (local) {
      const __half *sv = p.down.svh + (size_t)(e - p.e0) * H + blk * 128;
      float v[4], sc[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        sc[j] = __half2float(sv[lane + 32 * j]);
        v[j] = part[0][j];
      }
      fwht_chunk(v, lane, 128, hs);
#pragma unroll
      for (int j = 0; j < 4; j++) vals[warp][lane + 32 * j] = v[j] * sc[j] * wk;
    }
  } else if (warp == k) {
    const bool on = !routed_only && (p.has_shared || p.shared_pre) && r >= p.sh_row0 && r < p.sh_row0 + p.sh_rows;
    if (lane == 0) used[k] = on ? 1 : 0;
    if (on && p.shared_pre) {  // finished by other kernels (8-bit affine shared expert): only the sigmoid gate is applied here
      const float lg = p.logits[(size_t)(r - p.lg_row0) * (p.E + 1) + p.E];
      const float sg = 1.0f / (1.0f + expf(-lg));
#pragma unroll
      for (int j = 0; j < 4; j++) vals[k][lane + 32 * j] = sg * p.sho[(size_t)r * H + blk * 128 + lane + 32 * j];
    } else if (on) {
      const float *const src[1] = {p.raw_sd + (size_t)r * H + blk * 128};
      float part[1][4], v[4];
      sum_splits<1>(src, (size_t)p.rows * H, p.S_d, lane, part);
      const float lg = p.logits[(size_t)(r - p.lg_row0) * (p.E + 1) + p.E];
#pragma unroll
      for (int j = 0; j < 4; j++) v[j] = part[0][j];
      fwht_chunk(v, lane, 128, hs);
      const float sg = 1.0f / (1.0f + expf(-lg));
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int c = blk * 128 + lane + 32 * j;
        v[j] *= __half2float(p.sdn.svh[c]);
        p.sho[(size_t)r * H + c] = v[j];
        vals[k][lane + 32 * j] = sg * v[j];
      }
    }
  }
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int c = blk * 128 + lane + 32 * j;
    float acc = 0.0f;
    for (int t = 0; t <= k; t++)
      if (used[t]) acc += vals[t][lane + 32 * j];
    if (p.ep != nullptr) {  // straight into the memory of the rank that owns row r (peer store over NVLink)
      const int dest = r / p.ep_rows;
      p.ep->part[dest][((size_t)p.ep->rank * p.ep->rows_cap + (r - dest * p.ep_rows)) * H + c] = acc;
    } else {
      p.y[(size_t)r * H + c] = acc;
    }
    if (p.h_mid != nullptr)
      for (int s = 0; s < p.HC; s++)
        p.h_out[((size_t)r * p.HC + s) * H + c] = p.h_mid[((size_t)r * p.HC + s) * H + c] + acc * p.inj[(size_t)r * 2 * p.HC + s];
  }
  if (p.ep != nullptr) {  // the last CTA to get here tells every peer that this rank's partial rows are in place
    __threadfence_system();
    __syncwarp();
    if (lane == 0 && atomicAdd(p.ep->counter, 1u) == gridDim.x * gridDim.y - 1) {
      *p.ep->counter = 0u;
      __threadfence_system();
      const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(p.ep->epoch);
      for (int d = 0; d < p.ep->world; d++)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ep->pflag[d] + p.ep->rank), "r"(epoch) : "memory");
    }
  }
}

// =============================================================================================== host side
MoeSplits plan_moe(int H, int I, int E, int topk, int Kx, int Ks, int rows, bool has_shared) {
  IJ_CHECK(H % 256 == 0 && I % 128 == 0, "MoE dims: hidden %d must be a multiple of 256, intermediate %d of 128", H, I);
  IJ_CHECK(rows >= 1 && rows <= 64, "rows %d outside 1..64", rows);
  IJ_CHECK(Kx >= 4 && Kx <= 8 && (!has_shared || (Ks >= 4 && Ks <= 8)), "bits per weight outside 4..8");
  MoeSplits s{};
  s.MT = 1;  // every unit has at most PLAN_ROWS = 8 rows (the plan cuts experts with more rows into several entries)
  const int kmax = std::max(Kx, has_shared ? Ks : 0);
  const int ctas = stream_ctas(std::min(rows, PLAN_ROWS), kmax);
  s.grid = ctas * sm_count();
  const int urows = std::min(rows, PLAN_ROWS);
  // expected number of distinct experts under uniform routing; any actual count works, this only tunes the k-split
  const double nu = E * (1.0 - std::pow(1.0 - (double)topk / E, rows));
  const double rpu = std::min((double)urows, std::max(1.0, rows * (double)topk / std::max(nu, 1.0)));
  const double nsh = has_shared ? (rows + PLAN_ROWS - 1) / PLAN_ROWS : 0;
  const int kcap = kc_cap(urows, kmax, ctas);
  // at most 16 splits (bounds the partial-sum scratch)
  choose_split(H / 16, (int)std::lround((nu + nsh) * 2 * (I / 128)), kcap, s.grid, rpu, &s.S_gu, &s.kc_gu);
  if (s.S_gu > 16) { s.kc_gu = (H / 16 + 15) / 16; s.kc_gu = (s.kc_gu + SG_KS - 1) / SG_KS * SG_KS; s.S_gu = (H / 16 + s.kc_gu - 1) / s.kc_gu; }
  choose_split(I / 16, (int)std::lround((nu + nsh) * (H / 128)), kcap, s.grid, rpu, &s.S_d, &s.kc_d);
  if (s.S_d > 16) { s.kc_d = (I / 16 + 15) / 16; s.kc_d = (s.kc_d + SG_KS - 1) / SG_KS * SG_KS; s.S_d = (I / 16 + s.kc_d - 1) / s.kc_d; }
  s.lay_gu = make_layout(kmax, s.kc_gu, urows, ctas);
  s.lay_d = make_layout(kmax, s.kc_d, urows, ctas);
  return s;
}

void launch_moe_prep(const MoeParams &p, bool build_plan, cudaStream_t st) {
  IJ_CHECK(p.P <= RT_PMAX && p.E <= RT_EMAX, "plan: %d pairs / %d experts exceed %d / %d", p.P, p.E, RT_PMAX, RT_EMAX);
  dim3 grid((p.H / 128 + 3) / 4, p.P + (p.has_shared ? p.rows : 0) + (build_plan ? 1 : 0));
  launch_pdl(moe_prep_kernel, grid, dim3(128), 0, st, p, build_plan ? 1 : 0);
}

void launch_moe_mid(const MoeParams &p, cudaStream_t st) {
  dim3 grid((p.I / 128 + 3) / 4, p.P + (p.has_shared ? p.rows : 0));
  launch_pdl(moe_mid_kernel, grid, dim3(128), 0, st, p);
}

void launch_moe_gateup(const MoeParams &p, const MoeMaps &maps, const MoeSplits &s, bool plan_final, int *status, cudaStream_t st) {
  MoeGateUpProblem pr;
  pr.maps[0] = maps.gate; pr.maps[1] = maps.up; pr.maps[2] = maps.sgt; pr.maps[3] = maps.sup;
  pr.p = p;
  pr.plan_final = plan_final ? 1 : 0;
  pr.IT = p.H / 16; pr.OT = p.I / 16; pr.NG = (pr.OT + SG_WARPS - 1) / SG_WARPS;
  pr.S = s.S_gu; pr.kc = s.kc_gu;
  launch_stream(pr, s.MT, s.lay_gu, s.grid, status, st);
}

void launch_moe_down(const MoeParams &p, const MoeMaps &maps, const MoeSplits &s, int *status, cudaStream_t st) {
  MoeDownProblem pr;
  pr.maps[0] = maps.down; pr.maps[1] = maps.sdn;
  pr.p = p;
  pr.IT = p.I / 16; pr.OT = p.H / 16; pr.NG = (pr.OT + SG_WARPS - 1) / SG_WARPS;
  pr.S = s.S_d; pr.kc = s.kc_d;
  launch_stream(pr, s.MT, s.lay_d, s.grid, status, st);
}

__global__ void __launch_bounds__(256) swiglu_rows_kernel(const float *__restrict__ g, const float *__restrict__ u, int rows, int I,
                                                          float *__restrict__ gush, float *__restrict__ act) {
  pdl_launch();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * I; i += gridDim.x * blockDim.x) {
    const int r = i / I, c = i - r * I;
    const float gv = g[i], uv = u[i];
    gush[(size_t)r * 2 * I + c] = gv;
    gush[(size_t)r * 2 * I + I + c] = uv;
    act[i] = gv / (1.0f + expf(-gv)) * uv;
  }
}

void launch_swiglu_rows(const float *g, const float *u, int rows, int I, float *gush, float *act, cudaStream_t st) {
  launch_pdl(swiglu_rows_kernel, dim3((rows * I + 255) / 256), dim3(256), 0, st, g, u, rows, I, gush, act);
}

void launch_moe_combine(const MoeParams &p, bool routed_only, cudaStream_t st) {
  IJ_CHECK(p.topk <= CB_MAXK, "combine: top_k %d > %d", p.topk, CB_MAXK);
  dim3 grid(p.H / 128, p.rows);
  launch_pdl(moe_combine_kernel, grid, dim3(32 * (p.topk + 1)), 0, st, p, routed_only ? 1 : 0);
}

}  // namespace ijah
