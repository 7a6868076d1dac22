// One EXL3 Linear at decode widths: y[rows][out] = x[rows][in] @ W, W = diag(suh) H_in W' H_out diag(svh)
// (reference: kernels/trunk6/trunk6.metal:366-429 t6_simd, host plan kernels/trunk6/trunk6.mm:84-168).
//
// Three launches: a prep kernel (xh = fp16(H_in(x * suh)), the A operand), stream_gemm (raw partial products of
// k-splits) and a finisher that sums the splits in index order and applies H_out and svh. Used for the trunk
// projections (K 6/7/8) and as the building block of the tests.
#pragma once
#include "stream_gemm.cuh"

namespace ijah {

struct LinearPlan {
  int in, out, K, rows;
  int IT, OT, NG;     // k-tiles, n-tiles, n-groups of 8 tiles
  int S, kc;          // k-splits and k-tiles per split
  int hi, ho;         // Hadamard sizes
  int MT;             // 8-row groups per unit (1, 2, 4, 8)
  StreamLayout lay;
  int grid;
  size_t raw_floats() const { return (size_t)S * rows * out; }
  size_t xh_halfs() const { return (size_t)rows * in * A_HALFS_PER_INPUT; }
  size_t scratch_bytes() const { return raw_floats() * 4 + ((xh_halfs() * 2 + 255) & ~(size_t)255) + 256; }
};

LinearPlan plan_linear(int in, int out, int K, int rows);

struct LinearProblem {
  __device__ bool units_final() const { return true; }  // the unit list is arithmetic
  struct Unit : UnitBase {
    int g, s, k0;
  };
  alignas(64) CUtensorMap map;  // over the trellis (make_trellis_map)
  const __half *xh;  // [rows][2 in] prepared operand (store_a layout)
  float *raw;
  int in, out, K, rows, IT, OT, NG, S, kc;

  __device__ const CUtensorMap *tmap(int) const { return &map; }
  __device__ int num_units() const { return NG * S; }
  __device__ Unit unit(int u) const {
    Unit un;
    un.g = u % NG;
    un.s = u / NG;
    un.k0 = un.s * kc;
    un.kc = min(kc, IT - un.k0);
    un.ntiles = min(SG_WARPS, OT - un.g * SG_WARPS);
    un.K = K;
    un.nrows = rows;
    un.map = 0; un.x = un.g * SG_WARPS * 4 * K; un.y = un.k0; un.z = 0;
    return un;
  }
  __device__ int row_index(const Unit &, int i) const { return i; }
  __device__ const __half *a_row(const Unit &un, int i) const { return xh + ((size_t)i * in + un.k0 * 16) * A_HALFS_PER_INPUT; }
  __device__ float *out_base(const Unit &un) const { return raw + (size_t)un.s * rows * out + un.g * 128; }
  __device__ int out_row_off(const Unit &, int row) const { return row * out; }
};

// Several Linears that read the same activation rows (the q, k, v projections of a layer; reference: t6::record_multi,
// kernels/trunk6/trunk6.h:78-79, which also takes one input per Linear) as ONE chain of three launches: the units of all matrices share the persistent grid, so
// small matrices (k, v: 0.8 MB) no longer pay a launch chain each nor leave most of the GPU idle.
constexpr int ML_MAX = 4;
struct MultiLinearPlan {
  int n, in, rows, IT, S, kc, MT, grid, hi;
  int out[ML_MAX], K[ML_MAX], OT[ML_MAX], NG[ML_MAX], ho[ML_MAX];
  StreamLayout lay;
  size_t raw_floats(int m) const { return (size_t)S * rows * out[m]; }
  size_t scratch_bytes() const {
    size_t b = 256;
    for (int m = 0; m < n; m++) b += ((raw_floats(m) * 4 + 255) & ~(size_t)255) + (((size_t)rows * in * A_HALFS_PER_INPUT * 2 + 255) & ~(size_t)255);
    return b;
  }
};
MultiLinearPlan plan_linear_multi(int n, int in, const int *out, const int *K, int rows);

struct MultiLinearProblem {
  __device__ bool units_final() const { return true; }  // the unit list is arithmetic
  struct Unit : UnitBase {
    int g, s, k0, m;
  };
  alignas(64) CUtensorMap maps[ML_MAX];  // one per trellis
  const __half *xh[ML_MAX];  // [rows][2 in] prepared operand per matrix (the scale vectors differ)
  float *raw[ML_MAX];
  int out[ML_MAX], K[ML_MAX], OT[ML_MAX], NG[ML_MAX], ubase[ML_MAX + 1];  // ubase[m]: first unit of matrix m
  int n, in, rows, IT, S, kc;

  __device__ const CUtensorMap *tmap(int i) const { return &maps[i]; }
  __device__ int num_units() const { return ubase[n]; }
  __device__ Unit unit(int u) const {
    Unit un;
    int m = 0;
    while (m + 1 < n && u >= ubase[m + 1]) m++;
    const int v = u - ubase[m];
    un.m = m;
    un.g = v % NG[m];
    un.s = v / NG[m];
    un.k0 = un.s * kc;
    un.kc = min(kc, IT - un.k0);
    un.ntiles = min(SG_WARPS, OT[m] - un.g * SG_WARPS);
    un.K = K[m];
    un.nrows = rows;
    un.map = m; un.x = un.g * SG_WARPS * 4 * K[m]; un.y = un.k0; un.z = 0;
    return un;
  }
  __device__ int row_index(const Unit &, int i) const { return i; }
  __device__ const __half *a_row(const Unit &un, int i) const { return xh[un.m] + ((size_t)i * in + un.k0 * 16) * A_HALFS_PER_INPUT; }
  __device__ float *out_base(const Unit &un) const { return raw[un.m] + (size_t)un.s * rows * out[un.m] + un.g * 128; }
  __device__ int out_row_off(const Unit &un, int row) const { return row * out[un.m]; }
};

struct MultiLinearArgs {  // per matrix: device pointers of the caller
  const void *trellis[ML_MAX], *suh[ML_MAX], *svh[ML_MAX];
  float *y[ML_MAX];
};
void launch_linear_multi(const MultiLinearPlan &p, const MultiLinearArgs &a, const float *x, void *scratch, int *status, cudaStream_t st);

// `scratch` holds LinearPlan::scratch_bytes(): the k-split partials, then the prepared operand
void launch_linear(const LinearPlan &p, const void *trellis, const void *suh, const void *svh, const float *x, float *y,
                   void *scratch, int *status, cudaStream_t st);

// xh[r][i] = fp16(H_n(x[r] * suh))[i]: product and butterflies in fp32, one rounding (one warp per 128-element chunk)
void launch_prep_rows(const float *x, const __half *suh, __half *xh, int rows, int n, cudaStream_t st);

// W' as fp16 [in][out] (bit-exact codebook values), for parity checks of the decoder
void launch_dequant(const void *trellis, int in, int out, int K, __half *w, cudaStream_t st);

// shared-memory carve-up for a stream_gemm launch: kcmax k-tiles of A for arows rows, ring sized to what is left
StreamLayout make_layout(int Kmax, int kcmax, int arows, int ctas_per_sm);
// largest k-tile count per unit whose A slots leave room for the ring (0: does not fit), and the CTAs per SM to plan with
int kc_cap(int arows, int Kmax, int ctas);
int stream_ctas(int arows, int Kmax);
// k-split choice for `cols` column groups of IT k-tiles on a persistent grid: returns S and kc (multiple of 4)
void choose_split(int IT, int cols, int kcap, int grid, double rows_per_unit, int *S, int *kc);


}  // namespace ijah
