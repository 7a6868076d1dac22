// EXL3 Linear at decode widths: planning, the finisher, the dequantiser, launchers. See exl3_linear.cuh.
#include <algorithm>

#include "common.hpp"
#include "exl3_linear.cuh"
#include "launch.cuh"

namespace ijah {

// Shared memory a CTA may use when `ctas` CTAs share an SM.
static size_t smem_budget(int ctas) { return (size_t)(228 / ctas - 2) * 1024; }
constexpr int kMinStages = SG_KS >= 16 ? 2 : 3;

StreamLayout make_layout(int Kmax, int kcmax, int arows, int ctas_per_sm) {
  StreamLayout l;
  l.stage_bytes = SG_KS * SG_WARPS * 32 * Kmax;
  l.lda = kcmax * 16 * A_HALFS_PER_INPUT + 8;
  l.arows = std::max(arows, 1);
  const size_t budget = smem_budget(ctas_per_sm);
  const size_t base = l.ring_off() + (size_t)l.lda * 2;
  const size_t want_stages = SG_KS >= 16 ? 3 : 6;
  // three A slots or more let the producer issue the rows of unit u + 2 while the consumers are still on unit u; the widest
  // row counts only fit two (the producer then waits for the consumers to leave unit u - 1 before it sends unit u + 1)
  l.aslots = base + SG_MAX_ASLOTS * l.slot_bytes() + want_stages * (size_t)l.stage_bytes <= budget ? SG_MAX_ASLOTS
             : base + 3 * l.slot_bytes() + kMinStages * (size_t)l.stage_bytes <= budget             ? 3
                                                                                                     : 2;
  const size_t fixed = base + l.aslots * l.slot_bytes();
  IJ_CHECK(fixed + kMinStages * (size_t)l.stage_bytes <= budget, "A operand of %d rows x %d k-tiles does not fit shared memory", arows, kcmax);
  l.stages = (int)std::min<size_t>(SG_MAX_STAGES, (budget - fixed) / l.stage_bytes);
  return l;
}

// Largest k-tile count per unit (a multiple of SG_KS) whose three A slots of `arows` rows leave room for the smallest ring
// of K = Kmax stages when `ctas` CTAs share an SM (two slots with one CTA per SM, if three do not fit); 0 if not even
// SG_KS k-tiles fit.
int kc_cap(int arows, int Kmax, int ctas) {
  const long room = (long)smem_budget(ctas) - 4096 - (long)kMinStages * SG_KS * SG_WARPS * 32 * Kmax;
  auto cap = [&](int slots) {
    const long halfs_per_row = room / slots / std::max(arows, 1) / 2;
    return std::max(0, std::min((int)((halfs_per_row - 8) / (16 * A_HALFS_PER_INPUT)) / SG_KS * SG_KS, 256));
  };
  const int c3 = cap(3);
  return c3 >= SG_KS || ctas > 1 ? c3 : cap(2);
}

// CTAs per SM for units of `arows` rows: the default, or one CTA per SM with all of its shared memory when the default
// cannot hold even the smallest unit (wide row counts at K = 7, 8)
int stream_ctas(int arows, int Kmax) {
  if (kc_cap(arows, Kmax, SG_CTAS) >= SG_KS) return SG_CTAS;
  IJ_CHECK(kc_cap(arows, Kmax, 1) >= SG_KS, "%d activation rows at K%d do not fit the shared memory of an SM", arows, Kmax);
  return 1;
}

// Units are dealt round-robin to a persistent grid; cost of a candidate = rounds * (k-tiles per unit + a per-unit
// overhead that grows with the rows whose partial sums the unit writes) with a small bias towards fewer splits. The fixed
// part of the overhead (descriptor, activation rows, epilogue, the partial sums' round trip through the next kernel) is
// worth about eight k-tiles: fitted to measured gate/up and down times at 4 and 8 rows with the split forced to each value.
void choose_split(int IT, int cols, int kcap, int grid, double rows_per_unit, int *S, int *kc) {
  double best = -1;
  for (int c = SG_KS; c <= std::max(SG_KS, std::min((IT + SG_KS - 1) / SG_KS * SG_KS, kcap)); c += SG_KS) {
    const int s = (IT + c - 1) / c;
    const long rounds = ((long)cols * s + grid - 1) / grid;
    const double cost = rounds * ((double)IT / s + 8.0 + 0.4 * rows_per_unit) + 0.05 * s;  // (the last split of a matrix is shorter: average k-tiles)
    if (best < 0 || cost < best) { best = cost; *S = s; *kc = c; }
  }
}

LinearPlan plan_linear(int in, int out, int K, int rows) {
  IJ_CHECK(in > 0 && out > 0 && in % 16 == 0 && out % 16 == 0, "EXL3 Linear dims must be multiples of 16 (%d -> %d)", in, out);
  IJ_CHECK(K >= 4 && K <= 8, "EXL3 bits per weight %d outside 4..8", K);
  IJ_CHECK(rows >= 1 && rows <= 64, "rows %d outside 1..64", rows);
  LinearPlan p{};
  p.in = in; p.out = out; p.K = K; p.rows = rows;
  p.IT = in / 16; p.OT = out / 16; p.NG = (p.OT + SG_WARPS - 1) / SG_WARPS;
  p.hi = had_size(in); p.ho = had_size(out);
  p.MT = rows <= 8 ? 1 : rows <= 16 ? 2 : rows <= 32 ? 4 : 8;
  const int ctas = stream_ctas(rows, K);
  p.grid = ctas * sm_count();
  choose_split(p.IT, p.NG, kc_cap(rows, K, ctas), p.grid, rows, &p.S, &p.kc);
  p.lay = make_layout(K, p.kc, rows, ctas);
  p.grid = std::min(p.grid, p.NG * p.S);
  return p;
}

__global__ void __launch_bounds__(128) prep_rows_kernel(const float *__restrict__ x, const __half *__restrict__ suh,
                                                        __half *__restrict__ xh, int rows, int n, int hn, float hscale, int dup) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x * 4 + warp, r = blockIdx.y;
  pdl_wait();
  pdl_launch();
  if (chunk * 128 >= n) return;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = chunk * 128 + lane + 32 * j;
    v[j] = i < n ? x[(size_t)r * n + i] * __half2float(suh[i]) : 0.0f;
  }
  fwht_chunk(v, lane, hn, hscale);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = chunk * 128 + lane + 32 * j;
    if (i < n) store_a(xh + (size_t)r * n * A_HALFS_PER_INPUT, i, v[j], dup);
  }
}

void launch_prep_rows(const float *x, const __half *suh, __half *xh, int rows, int n, cudaStream_t st) {
  const int hn = had_size(n);
  dim3 grid(((n + 127) / 128 + 3) / 4, rows);
  launch_pdl(prep_rows_kernel, grid, dim3(128), 0, st, x, suh, xh, rows, n, hn, (float)(1.0 / sqrt((double)hn)), g_summand_product);
}

// y[r][c] = (H_ho(sum_s raw[s][r]))[c] * svh[c]; one warp per (row, 128-column chunk), splits summed in index order
__global__ void linear_finish_kernel(const float *__restrict__ raw, const __half *__restrict__ svh, float *__restrict__ y,
                                     int rows, int out, int S, int ho, float hscale) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x * (blockDim.x >> 5) + warp, r = blockIdx.y;
  pdl_wait();
  pdl_launch();
  if (chunk * 128 >= out) return;
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int s0 = 0; s0 < S; s0 += 4) {  // splits in index order, four splits' loads in flight at a time
    float t[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int c = chunk * 128 + lane + 32 * j;
        t[i][j] = (c < out && s0 + i < S) ? __ldcg(&raw[((size_t)(s0 + i) * rows + r) * out + c]) : 0.0f;
      }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) v[j] += t[i][j];
  }
  fwht_chunk(v, lane, ho, hscale);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int c = chunk * 128 + lane + 32 * j;
    if (c < out) y[(size_t)r * out + c] = v[j] * __half2float(svh[c]);
  }
}

// ---- several Linears on the same rows
struct MlPtrs {
  const __half *suh[ML_MAX], *svh[ML_MAX];
  __half *xh[ML_MAX];
  const float *raw[ML_MAX];
  float *y[ML_MAX];
  int out[ML_MAX], ho[ML_MAX];
  float hs[ML_MAX];  // 1 / sqrt(ho), rounded once on the host like everywhere else
  int dup;           // store_a's pair form: the product mode in force when the call was enqueued
};

__global__ void __launch_bounds__(128) prep_rows_multi_kernel(const float *__restrict__ x, const MlPtrs a, int rows, int n, int hn, float hscale) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x * 4 + warp, r = blockIdx.y, m = blockIdx.z;
  pdl_wait();
  pdl_launch();
  if (chunk * 128 >= n) return;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = chunk * 128 + lane + 32 * j;
    v[j] = i < n ? x[(size_t)r * n + i] * __half2float(a.suh[m][i]) : 0.0f;
  }
  fwht_chunk(v, lane, hn, hscale);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = chunk * 128 + lane + 32 * j;
    if (i < n) store_a(a.xh[m] + (size_t)r * n * A_HALFS_PER_INPUT, i, v[j], a.dup);
  }
}

__global__ void __launch_bounds__(128) linear_finish_multi_kernel(const MlPtrs a, int rows, int S) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x * 4 + warp, r = blockIdx.y, m = blockIdx.z, out = a.out[m], ho = a.ho[m];
  pdl_wait();
  pdl_launch();
  if (chunk * 128 >= out) return;
  const float *raw = a.raw[m];
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int s0 = 0; s0 < S; s0 += 4) {
    float t[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int c = chunk * 128 + lane + 32 * j;
        t[i][j] = (c < out && s0 + i < S) ? __ldcg(&raw[((size_t)(s0 + i) * rows + r) * out + c]) : 0.0f;
      }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) v[j] += t[i][j];
  }
  fwht_chunk(v, lane, ho, a.hs[m]);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int c = chunk * 128 + lane + 32 * j;
    if (c < out) a.y[m][(size_t)r * out + c] = v[j] * __half2float(a.svh[m][c]);
  }
}

MultiLinearPlan plan_linear_multi(int n, int in, const int *out, const int *K, int rows) {
  IJ_CHECK(n >= 1 && n <= ML_MAX, "%d Linears in one call (1..%d)", n, ML_MAX);
  IJ_CHECK(in > 0 && in % 16 == 0, "EXL3 Linear input width %d must be a multiple of 16", in);
  IJ_CHECK(rows >= 1 && rows <= 64, "rows %d outside 1..64", rows);
  MultiLinearPlan p{};
  p.n = n; p.in = in; p.rows = rows; p.IT = in / 16; p.hi = had_size(in);
  int ng = 0, kmax = 0;
  for (int m = 0; m < n; m++) {
    IJ_CHECK(out[m] > 0 && out[m] % 16 == 0, "EXL3 Linear output width %d must be a multiple of 16", out[m]);
    IJ_CHECK(K[m] >= 4 && K[m] <= 8, "EXL3 bits per weight %d outside 4..8", K[m]);
    p.out[m] = out[m]; p.K[m] = K[m]; p.OT[m] = out[m] / 16; p.NG[m] = (p.OT[m] + SG_WARPS - 1) / SG_WARPS; p.ho[m] = had_size(out[m]);
    ng += p.NG[m];
    kmax = std::max(kmax, K[m]);
  }
  p.MT = rows <= 8 ? 1 : rows <= 16 ? 2 : rows <= 32 ? 4 : 8;
  const int ctas = stream_ctas(rows, kmax);
  p.grid = ctas * sm_count();
  choose_split(p.IT, ng, kc_cap(rows, kmax, ctas), p.grid, rows, &p.S, &p.kc);
  p.lay = make_layout(kmax, p.kc, rows, ctas);
  p.grid = std::min(p.grid, ng * p.S);
  return p;
}

void launch_linear_multi(const MultiLinearPlan &p, const MultiLinearArgs &a, const float *x, void *scratch, int *status, cudaStream_t st) {
  MultiLinearProblem pr{};
  MlPtrs q{};
  q.dup = g_summand_product;
  char *cur = (char *)scratch;
  int maxout = 0;
  pr.n = p.n; pr.in = p.in; pr.rows = p.rows; pr.IT = p.IT; pr.S = p.S; pr.kc = p.kc;
  pr.ubase[0] = 0;
  for (int m = 0; m < p.n; m++) {
    float *raw = (float *)cur;
    cur += (p.raw_floats(m) * 4 + 255) & ~(size_t)255;
    __half *xh = (__half *)cur;
    cur += ((size_t)p.rows * p.in * A_HALFS_PER_INPUT * 2 + 255) & ~(size_t)255;
    make_trellis_map(&pr.maps[m], a.trellis[m], 1, p.IT, p.OT[m], p.K[m], SG_KS);
    pr.xh[m] = xh; pr.raw[m] = raw;
    pr.out[m] = p.out[m]; pr.K[m] = p.K[m]; pr.OT[m] = p.OT[m]; pr.NG[m] = p.NG[m];
    pr.ubase[m + 1] = pr.ubase[m] + p.NG[m] * p.S;
    q.suh[m] = (const __half *)a.suh[m]; q.svh[m] = (const __half *)a.svh[m]; q.xh[m] = xh; q.raw[m] = raw; q.y[m] = a.y[m];
    q.out[m] = p.out[m]; q.ho[m] = p.ho[m]; q.hs[m] = (float)(1.0 / sqrt((double)p.ho[m]));
    maxout = std::max(maxout, p.out[m]);
  }
  launch_pdl(prep_rows_multi_kernel, dim3(((p.in + 127) / 128 + 3) / 4, p.rows, p.n), dim3(128), 0, st, x, q, p.rows, p.in, p.hi,
             (float)(1.0 / sqrt((double)p.hi)));
  launch_stream(pr, p.MT, p.lay, p.grid, status, st);
  launch_pdl(linear_finish_multi_kernel, dim3(((maxout + 127) / 128 + 3) / 4, p.rows, p.n), dim3(128), 0, st, q, p.rows, p.S);
}

void launch_linear(const LinearPlan &p, const void *trellis, const void *suh, const void *svh, const float *x, float *y,
                   void *scratch, int *status, cudaStream_t st) {
  float *raw = (float *)scratch;
  __half *xh = (__half *)((char *)scratch + ((p.raw_floats() * 4 + 255) & ~(size_t)255));
  launch_prep_rows(x, (const __half *)suh, xh, p.rows, p.in, st);
  LinearProblem pr;
  make_trellis_map(&pr.map, trellis, 1, p.IT, p.OT, p.K, SG_KS);
  pr.xh = xh;
  pr.raw = raw;
  pr.in = p.in; pr.out = p.out; pr.K = p.K; pr.rows = p.rows;
  pr.IT = p.IT; pr.OT = p.OT; pr.NG = p.NG; pr.S = p.S; pr.kc = p.kc;
  launch_stream(pr, p.MT, p.lay, p.grid, status, st);
  const int chunks = (p.out + 127) / 128;
  dim3 grid((chunks + 3) / 4, p.rows);
  launch_pdl(linear_finish_kernel, grid, dim3(128), 0, st, raw, (const __half *)svh, y, p.rows, p.out, p.S, p.ho,
             (float)(1.0 / sqrt((double)p.ho)));
}

// one warp per tile, straight from global memory
template <int K>
__global__ void dequant_kernel(const uint32_t *__restrict__ tr, int IT, int OT, __half *__restrict__ w) {
  const int lane = threadIdx.x & 31;
  const long tile = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tile >= (long)IT * OT) return;
  const typename Codec<K>::Lane L = Codec<K>::lane(lane);
  const char *t = reinterpret_cast<const char *>(tr) + tile * Codec<K>::TILE_BYTES;
  uint32_t b[4];
  dec8<K>(*reinterpret_cast<const uint32_t *>(t + L.o0), *reinterpret_cast<const uint32_t *>(t + L.o1),
          *reinterpret_cast<const uint32_t *>(t + L.o2), L.a, McgConst::load(), b);
  const int tk = (int)(tile / OT), tn = (int)(tile % OT), q = lane & 3, c = lane >> 2;
  const int out = OT * 16;
  const __half *h = reinterpret_cast<const __half *>(b);
  const int rows[4] = {2 * q, 2 * q + 1, 2 * q + 8, 2 * q + 9};
#pragma unroll
  for (int j = 0; j < 8; j++) w[(size_t)(tk * 16 + rows[j & 3]) * out + tn * 16 + c + 8 * (j >> 2)] = h[j];
}

void launch_dequant(const void *trellis, int in, int out, int K, __half *w, cudaStream_t st) {
  IJ_CHECK(in % 16 == 0 && out % 16 == 0 && K >= 4 && K <= 8, "bad dequant shape %d x %d K%d", in, out, K);
  const int IT = in / 16, OT = out / 16;
  const long tiles = (long)IT * OT;
  const int blocks = (int)((tiles + 7) / 8);
  const uint32_t *tr = (const uint32_t *)trellis;
  switch (K) {
    case 4: dequant_kernel<4><<<blocks, 256, 0, st>>>(tr, IT, OT, w); break;
    case 5: dequant_kernel<5><<<blocks, 256, 0, st>>>(tr, IT, OT, w); break;
    case 6: dequant_kernel<6><<<blocks, 256, 0, st>>>(tr, IT, OT, w); break;
    case 7: dequant_kernel<7><<<blocks, 256, 0, st>>>(tr, IT, OT, w); break;
    default: dequant_kernel<8><<<blocks, 256, 0, st>>>(tr, IT, OT, w); break;
  }
  IJ_CUDA(cudaGetLastError());
}

}  // namespace ijah
