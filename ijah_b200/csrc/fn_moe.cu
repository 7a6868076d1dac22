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
constexpr int RT_WARPS = 8;
constexpr int RT_RC = 8;      // activation rows per pass
constexpr int RT_EMAX = 1024;  // experts the finisher's shared memory covers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

__device__ void topk_row(const MoeParams &p, int r, float *s, int lane) {
  const int E = p.E, k = p.topk;
  for (int i = lane; i < E; i += 32) s[i] = __ldcg(&p.logits[(size_t)r * (E + 1) + i]);
  __syncwarp();
  float myv = 0.0f, top = 0.0f;
  int myi = 0;
  for (int t = 0; t < k; t++) {
    float best = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = lane; i < E; i += 32) {
      const float v = s[i];
      if (v > best || bi == 0x7FFFFFFF) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (t == 0) top = best;
    if (lane == t) { myv = best; myi = bi; }
    if ((bi & 31) == lane) s[bi] = -INFINITY;
    __syncwarp();
  }
  const float pr = lane < k ? expf(myv - top) : 0.0f;
  const float sum = warp_sum(pr);
  if (lane < k) {
    p.route[(size_t)r * 2 * k + lane] = (uint32_t)myi;
    p.route[(size_t)r * 2 * k + k + lane] = __float_as_uint(pr / sum);
  }
}

// Distinct local experts of the rows*topk (row, slot) pairs, in expert order, each with its pairs in row order.
// One CTA; `buf` is >= 16 KB of shared memory.
__device__ void build_plan_block(const MoeParams &p, unsigned char *buf) {
  unsigned long long *mask = reinterpret_cast<unsigned long long *>(buf);  // [E] rows that use expert e
  int *uidx = reinterpret_cast<int *>(buf + 8 * RT_EMAX);                  // [E] index among present experts
  int *firs = uidx + RT_EMAX;                                              // [E] offset of its pairs
  const int tid = threadIdx.x, T = blockDim.x, E = p.E, k = p.topk, P = p.P;
  PlanView pv{p.plan, P};
  for (int e = tid; e < E; e += T) mask[e] = 0ull;
  __syncthreads();
  for (int i = tid; i < P; i += T) {
    const int r = i / k, e = (int)p.route[(size_t)r * 2 * k + (i - r * k)];
    if (e >= p.e0 && e < p.e0 + p.ecount) atomicOr(&mask[e], 1ull << r);
  }
  __syncthreads();
  if (tid < 32) {
    int run_u = 0, run_f = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + tid;
      const int c = e < E ? __popcll(mask[e]) : 0, pr = c > 0 ? 1 : 0;
      int su = pr, sf = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int a = __shfl_up_sync(0xFFFFFFFFu, su, o), b = __shfl_up_sync(0xFFFFFFFFu, sf, o);
        if (tid >= o) { su += a; sf += b; }
      }
      if (e < E) { uidx[e] = run_u + su - pr; firs[e] = run_f + sf - c; }
      run_u += __shfl_sync(0xFFFFFFFFu, su, 31);
      run_f += __shfl_sync(0xFFFFFFFFu, sf, 31);
    }
    if (tid == 0) *pv.nu() = run_u;
  }
  __syncthreads();
  for (int e = tid; e < E; e += T) {
    const int c = __popcll(mask[e]);
    if (c > 0) {
      const int u = uidx[e];
      pv.expert()[u] = e;
      pv.nrows()[u] = c;
      pv.first()[u] = firs[e];
    }
  }
  for (int i = tid; i < P; i += T) {
    const int r = i / k, e = (int)p.route[(size_t)r * 2 * k + (i - r * k)];
    if (e >= p.e0 && e < p.e0 + p.ecount) pv.pairs()[firs[e] + __popcll(mask[e] & ((1ull << r) - 1ull))] = i;
  }
}

// Dynamic shared memory: first the activation rows of one pass (RT_RC rows x H floats, shared by the CTA's 8 expert
// rows), later reused by the finisher (per-warp logit rows, then the plan's tables).
__global__ void __launch_bounds__(32 * RT_WARPS) moe_router_kernel(const MoeParams p, int build_plan) {
  extern __shared__ __align__(16) float dyn[];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * RT_WARPS + warp;
  const int H = p.H, E = p.E;
  const uint16_t *wr = row < E ? p.router + (size_t)row * H : (row == E ? p.sgate : nullptr);
  // the expert's weight row stays in registers for all passes: H / 256 x 8 bf16 per lane (H <= 4096)
  uint4 wreg[16];
#pragma unroll
  for (int j = 0; j < 16; j++)
    wreg[j] = (wr != nullptr && j * 32 + lane < H / 8) ? __ldg(reinterpret_cast<const uint4 *>(wr) + j * 32 + lane) : make_uint4(0, 0, 0, 0);
  pdl_wait();  // the router weights above are static; the activations may be the preceding kernel's output
  pdl_launch();
  for (int r0 = 0; r0 < p.rows; r0 += RT_RC) {
    const int nr = min(RT_RC, p.rows - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < nr * H / 4; i += blockDim.x)
      reinterpret_cast<float4 *>(dyn)[i] = reinterpret_cast<const float4 *>(p.x + (size_t)r0 * H)[i];
    __syncthreads();
    float acc[RT_RC];
#pragma unroll
    for (int t = 0; t < RT_RC; t++) acc[t] = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int c = j * 32 + lane;
      if (c < H / 8) {
        const uint4 u = wreg[j];
        const float w0 = __uint_as_float(u.x << 16), w1 = __uint_as_float(u.x & 0xFFFF0000u);
        const float w2 = __uint_as_float(u.y << 16), w3 = __uint_as_float(u.y & 0xFFFF0000u);
        const float w4_ = __uint_as_float(u.z << 16), w5 = __uint_as_float(u.z & 0xFFFF0000u);
        const float w6 = __uint_as_float(u.w << 16), w7 = __uint_as_float(u.w & 0xFFFF0000u);
#pragma unroll
        for (int t = 0; t < RT_RC; t++) {
          if (t < nr) {
            const float4 *x4 = reinterpret_cast<const float4 *>(dyn + (size_t)t * H) + 2 * c;
            const float4 a = x4[0], b = x4[1];
            acc[t] += a.x * w0 + a.y * w1 + a.z * w2 + a.w * w3 + b.x * w4_ + b.y * w5 + b.z * w6 + b.w * w7;
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < RT_RC; t++) {
      const float v = warp_sum(acc[t]);
      if (lane == 0 && t < nr && row <= E) p.logits[(size_t)(r0 + t) * (E + 1) + row] = v;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.counter, 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int r = warp; r < p.rows; r += RT_WARPS) topk_row(p, r, dyn + (size_t)warp * RT_EMAX, lane);
  __syncthreads();
  if (build_plan) build_plan_block(p, reinterpret_cast<unsigned char *>(dyn));
  if (threadIdx.x == 0) *p.counter = 0u;
}

__global__ void __launch_bounds__(256) moe_plan_kernel(const MoeParams p) {
  __shared__ __align__(16) unsigned char buf[16 * RT_EMAX];
  pdl_wait();
  pdl_launch();
  build_plan_block(p, buf);
}

void launch_moe_router(const MoeParams &p, bool build_plan, cudaStream_t st) {
  IJ_CHECK(p.E <= RT_EMAX && p.E % 32 == 0 && p.H % 256 == 0 && p.topk <= 32, "router: unsupported dims E %d H %d k %d", p.E, p.H, p.topk);
  IJ_CHECK(p.H <= 4096, "router: hidden %d > 4096", p.H);
  const int grid = (p.E + 1 + RT_WARPS - 1) / RT_WARPS;
  const size_t smem = std::max((size_t)std::min(p.rows, RT_RC) * p.H * 4, (size_t)RT_WARPS * RT_EMAX * 4);
  static bool ready = false;
  if (!ready) {
    IJ_CUDA(cudaFuncSetAttribute(moe_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_RC * 4096 * 4));
    ready = true;
  }
  launch_pdl(moe_router_kernel, dim3(grid), dim3(32 * RT_WARPS), smem, st, p, build_plan ? 1 : 0);
}

void launch_moe_plan(const MoeParams &p, cudaStream_t st) {
  launch_pdl(moe_plan_kernel, dim3(1), dim3(256), 0, st, p);
}

// =============================================================================================== operand prep
// xh_gu[pair][proj][H] = fp16(H128(x[row(pair)] * suh_proj[expert(pair)])) for every local (row, slot) pair, and
// xh_sgu[row][proj][H] for the shared expert (reference kernels/fn_moe.metal:304-311, prefill twin
// kernels/prefill/pf_moe.metal:88-104). One warp per (operand row, 128-element chunk).
__global__ void __launch_bounds__(128) moe_prep_kernel(const MoeParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x * 4 + warp, job = blockIdx.y;  // job < P: routed pair; else shared row
  const int H = p.H, k = p.topk;
  pdl_wait();
  pdl_launch();
  if (chunk * 128 >= H) return;
  const float hs = 0.08838834764831845f;
  int r;
  const __half *sg, *su;
  __half *dst;
  if (job < p.P) {
    r = job / k;
    const int e = (int)p.route[(size_t)r * 2 * k + (job - r * k)] - p.e0;
    if (e < 0 || e >= p.ecount) return;
    sg = p.gate.suh + (size_t)e * H;
    su = p.up.suh + (size_t)e * H;
    dst = p.xh_gu + (size_t)job * 2 * H;
  } else {
    r = job - p.P;
    sg = p.sgt.suh;
    su = p.sup.suh;
    dst = p.xh_sgu + (size_t)r * 2 * H;
  }
  const int o = chunk * 128 + lane;
  float xv[4], v[4];
#pragma unroll
  for (int j = 0; j < 4; j++) xv[j] = p.x[(size_t)r * H + o + 32 * j];
#pragma unroll
  for (int j = 0; j < 4; j++) v[j] = xv[j] * __half2float(sg[o + 32 * j]);
  fwht_chunk(v, lane, 128, hs);
#pragma unroll
  for (int j = 0; j < 4; j++) dst[o + 32 * j] = __float2half_rn(v[j]);
#pragma unroll
  for (int j = 0; j < 4; j++) v[j] = xv[j] * __half2float(su[o + 32 * j]);
  fwht_chunk(v, lane, 128, hs);
#pragma unroll
  for (int j = 0; j < 4; j++) dst[H + o + 32 * j] = __float2half_rn(v[j]);
}

// xh_d[pair][I] = fp16(H128(silu(g) * u * suh_down)), g = H128(sum_s raw gate) * svh_gate, u likewise
// (reference kernels/fn_moe.metal:370-384, kernels/prefill/pf_moe.metal:107-125). One warp per (pair | shared row,
// 128-element chunk of the intermediate).
__global__ void __launch_bounds__(128) moe_mid_kernel(const MoeParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x * 4 + warp, job = blockIdx.y;
  const int I = p.I, k = p.topk;
  pdl_wait();
  pdl_launch();
  if (chunk * 128 >= I) return;
  const float hs = 0.08838834764831845f;
  const float *raw;
  size_t sstride;
  const __half *svg, *svu, *sud;
  __half *dst;
  const bool shared = job >= p.P;
  if (!shared) {
    const int r = job / k, e = (int)p.route[(size_t)r * 2 * k + (job - r * k)] - p.e0;
    if (e < 0 || e >= p.ecount) return;
    raw = p.raw_gu + (size_t)job * 2 * I;
    sstride = (size_t)p.P * 2 * I;
    svg = p.gate.svh + (size_t)e * I; svu = p.up.svh + (size_t)e * I; sud = p.down.suh + (size_t)e * I;
    dst = p.xh_d + (size_t)job * I;
  } else {
    const int r = job - p.P;
    raw = p.raw_sgu + (size_t)r * 2 * I;
    sstride = (size_t)p.rows * 2 * I;
    svg = p.sgt.svh; svu = p.sup.svh; sud = p.sdn.suh;
    dst = p.xh_sd + (size_t)r * I;
  }
  const int o = chunk * 128 + lane;
  float gv[4], uv[4], hh[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    float a = 0.0f, b = 0.0f;
    for (int s = 0; s < p.S_gu; s++) {  // k-split partials in split order
      a += raw[s * sstride + o + 32 * j];
      b += raw[s * sstride + I + o + 32 * j];
    }
    gv[j] = a; uv[j] = b;
  }
  fwht_chunk(gv, lane, 128, hs);
  fwht_chunk(uv, lane, 128, hs);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    gv[j] *= __half2float(svg[o + 32 * j]);
    uv[j] *= __half2float(svu[o + 32 * j]);
    hh[j] = gv[j] / (1.0f + expf(-gv[j])) * uv[j] * __half2float(sud[o + 32 * j]);
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
  for (int j = 0; j < 4; j++) dst[o + 32 * j] = __float2half_rn(hh[j]);
}

// =============================================================================================== gate / up
// Unit order: for each distinct expert u: proj (gate, up) x k-split x column group; then the shared expert's.
struct MoeGateUpProblem {
  static constexpr bool kUnitsFinalAtLaunch = false;  // the plan is written by the router kernel just before
  struct Unit : UnitBase {
    int s, k0, g, proj, shared, e, first;
  };
  MoeParams p;
  int IT, OT, NG, S, kc;

  __device__ int num_units() const { return (*PlanView{p.plan, p.P}.nu() + (p.has_shared ? 1 : 0)) * 2 * S * NG; }
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
    const Exl3Stack *w;
    if (un.shared) {
      un.e = 0; un.first = 0; un.nrows = p.rows; un.K = p.Ks;
      w = un.proj ? &p.sup : &p.sgt;
    } else {
      un.e = pv.expert()[q] - p.e0; un.first = pv.first()[q]; un.nrows = pv.nrows()[q]; un.K = p.Kx;
      w = un.proj ? &p.up : &p.gate;
    }
    const size_t tile = 32u * un.K;
    un.kstride = (uint32_t)(OT * tile);
    un.w = w->trellis + ((size_t)un.e * IT * OT + (size_t)un.k0 * OT + (size_t)un.g * SG_WARPS) * tile;
    return un;
  }
  // row index = the (row, slot) pair for routed units, the activation row for the shared expert
  __device__ int row_index(const Unit &un, int i) const { return un.shared ? i : PlanView{p.plan, p.P}.pairs()[un.first + i]; }
  __device__ const __half *a_row(const Unit &un, int idx) const {
    return (un.shared ? p.xh_sgu : p.xh_gu) + ((size_t)idx * 2 + un.proj) * p.H + un.k0 * 16;
  }
  __device__ void store(const Unit &un, int idx, int col, float v) const {
    float *dst = un.shared ? p.raw_sgu + (((size_t)un.s * p.rows + idx) * 2 + un.proj) * p.I
                           : p.raw_gu + (((size_t)un.s * p.P + idx) * 2 + un.proj) * p.I;
    dst[un.g * 128 + col] = v;
  }
};

// =============================================================================================== down
struct MoeDownProblem {
  // the plan was complete before the gate/up kernel started, i.e. before the predecessor (mid) could release this launch
  static constexpr bool kUnitsFinalAtLaunch = true;
  struct Unit : UnitBase {
    int s, k0, g, shared, e, first;
  };
  MoeParams p;
  int IT, OT, NG, S, kc;  // IT = I/16, OT = H/16

  __device__ int num_units() const { return (*PlanView{p.plan, p.P}.nu() + (p.has_shared ? 1 : 0)) * S * NG; }
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
    if (un.shared) { un.e = 0; un.first = 0; un.nrows = p.rows; un.K = p.Ks; }
    else { un.e = pv.expert()[q] - p.e0; un.first = pv.first()[q]; un.nrows = pv.nrows()[q]; un.K = p.Kx; }
    const size_t tile = 32u * un.K;
    un.kstride = (uint32_t)(OT * tile);
    un.w = (un.shared ? p.sdn.trellis : p.down.trellis) + ((size_t)un.e * IT * OT + (size_t)un.k0 * OT + (size_t)un.g * SG_WARPS) * tile;
    return un;
  }
  __device__ int row_index(const Unit &un, int i) const { return un.shared ? i : PlanView{p.plan, p.P}.pairs()[un.first + i]; }
  __device__ const __half *a_row(const Unit &un, int idx) const {
    return (un.shared ? p.xh_sd : p.xh_d) + (size_t)idx * p.I + un.k0 * 16;
  }
  __device__ void store(const Unit &un, int idx, int col, float v) const {
    float *dst = un.shared ? p.raw_sd + ((size_t)un.s * p.rows + idx) * p.H : p.raw_d + ((size_t)un.s * p.P + idx) * p.H;
    dst[un.g * 128 + col] = v;
  }
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
  pdl_wait();
  pdl_launch();
  const float hs = 0.08838834764831845f;
  if (warp < k) {
    const int e = (int)p.route[(size_t)r * 2 * k + warp];
    const bool local = e >= p.e0 && e < p.e0 + p.ecount;
    if (lane == 0) used[warp] = local ? 1 : 0;
    if (local) {
      const float wk = __uint_as_float(p.route[(size_t)r * 2 * k + k + warp]);
      const float *raw = p.raw_d + (size_t)(r * k + warp) * H + blk * 128;
      const __half *sv = p.down.svh + (size_t)(e - p.e0) * H + blk * 128;
      float v[4], sc[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        sc[j] = __half2float(sv[lane + 32 * j]);
        float a = 0.0f;
        for (int s = 0; s < p.S_d; s++) a += raw[(size_t)s * p.P * H + lane + 32 * j];
        v[j] = a;
      }
      fwht_chunk(v, lane, 128, hs);
#pragma unroll
      for (int j = 0; j < 4; j++) vals[warp][lane + 32 * j] = v[j] * sc[j] * wk;
    }
  } else if (warp == k) {
    const bool on = !routed_only && p.has_shared && r >= p.sh_row0 && r < p.sh_row0 + p.sh_rows;
    if (lane == 0) used[k] = on ? 1 : 0;
    if (on) {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float a = 0.0f;
        for (int s = 0; s < p.S_d; s++) a += p.raw_sd[((size_t)s * p.rows + r) * H + blk * 128 + lane + 32 * j];
        v[j] = a;
      }
      fwht_chunk(v, lane, 128, hs);
      const float sg = 1.0f / (1.0f + expf(-p.logits[(size_t)r * (p.E + 1) + p.E]));
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
    p.y[(size_t)r * H + c] = acc;
    if (p.h_mid != nullptr)
      for (int s = 0; s < p.HC; s++)
        p.h_out[((size_t)r * p.HC + s) * H + c] = p.h_mid[((size_t)r * p.HC + s) * H + c] + acc * p.inj[(size_t)r * 2 * p.HC + s];
  }
}

// =============================================================================================== host side
MoeSplits plan_moe(int H, int I, int E, int topk, int Kx, int Ks, int rows, bool has_shared) {
  IJ_CHECK(H % 256 == 0 && I % 128 == 0, "MoE dims: hidden %d must be a multiple of 256, intermediate %d of 128", H, I);
  IJ_CHECK(rows >= 1 && rows <= 64, "rows %d outside 1..64", rows);
  IJ_CHECK(Kx >= 4 && Kx <= 8 && (!has_shared || (Ks >= 4 && Ks <= 8)), "bits per weight outside 4..8");
  MoeSplits s{};
  s.MT = rows <= 8 ? 1 : rows <= 16 ? 2 : rows <= 32 ? 4 : 8;
  s.grid = 2 * sm_count();
  // expected number of distinct experts under uniform routing; any actual count works, this only tunes the k-split
  const double nu = E * (1.0 - std::pow(1.0 - (double)topk / E, rows));
  const double rpu = std::max(1.0, rows * (double)topk / std::max(nu, 1.0));
  const int kcap = kc_cap(rows);
  // at most 16 splits (bounds the partial-sum scratch)
  choose_split(H / 16, (int)std::lround((nu + (has_shared ? 1 : 0)) * 2 * (I / 128)), kcap, s.grid, rpu, &s.S_gu, &s.kc_gu);
  if (s.S_gu > 16) { s.kc_gu = (H / 16 + 15) / 16; s.kc_gu = (s.kc_gu + SG_KS - 1) / SG_KS * SG_KS; s.S_gu = (H / 16 + s.kc_gu - 1) / s.kc_gu; }
  choose_split(I / 16, (int)std::lround((nu + (has_shared ? 1 : 0)) * (H / 128)), kcap, s.grid, rpu, &s.S_d, &s.kc_d);
  if (s.S_d > 16) { s.kc_d = (I / 16 + 15) / 16; s.kc_d = (s.kc_d + SG_KS - 1) / SG_KS * SG_KS; s.S_d = (I / 16 + s.kc_d - 1) / s.kc_d; }
  const int kmax = std::max(Kx, has_shared ? Ks : 0);
  s.lay_gu = make_layout(kmax, s.kc_gu, rows, 2);
  s.lay_d = make_layout(kmax, s.kc_d, rows, 2);
  return s;
}

void launch_moe_prep(const MoeParams &p, cudaStream_t st) {
  dim3 grid((p.H / 128 + 3) / 4, p.P + (p.has_shared ? p.rows : 0));
  launch_pdl(moe_prep_kernel, grid, dim3(128), 0, st, p);
}

void launch_moe_mid(const MoeParams &p, cudaStream_t st) {
  dim3 grid((p.I / 128 + 3) / 4, p.P + (p.has_shared ? p.rows : 0));
  launch_pdl(moe_mid_kernel, grid, dim3(128), 0, st, p);
}

void launch_moe_gateup(const MoeParams &p, const MoeSplits &s, int *status, cudaStream_t st) {
  MoeGateUpProblem pr;
  pr.p = p;
  pr.IT = p.H / 16; pr.OT = p.I / 16; pr.NG = (pr.OT + SG_WARPS - 1) / SG_WARPS;
  pr.S = s.S_gu; pr.kc = s.kc_gu;
  launch_stream(pr, s.MT, s.lay_gu, s.grid, status, st);
}

void launch_moe_down(const MoeParams &p, const MoeSplits &s, int *status, cudaStream_t st) {
  MoeDownProblem pr;
  pr.p = p;
  pr.IT = p.I / 16; pr.OT = p.H / 16; pr.NG = (pr.OT + SG_WARPS - 1) / SG_WARPS;
  pr.S = s.S_d; pr.kc = s.kc_d;
  launch_stream(pr, s.MT, s.lay_d, s.grid, status, st);
}

void launch_moe_combine(const MoeParams &p, bool routed_only, cudaStream_t st) {
  IJ_CHECK(p.topk <= CB_MAXK, "combine: top_k %d > %d", p.topk, CB_MAXK);
  dim3 grid(p.H / 128, p.rows);
  launch_pdl(moe_combine_kernel, grid, dim3(32 * (p.topk + 1)), 0, st, p, routed_only ? 1 : 0);
}

}  // namespace ijah
