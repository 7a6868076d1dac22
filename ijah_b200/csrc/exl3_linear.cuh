// One EXL3 Linear at decode widths: y[rows][out] = x[rows][in] @ W, W = diag(suh) H_in W' H_out diag(svh)
// (reference: kernels/trunk6/trunk6.metal:366-429 t6_simd, host plan kernels/trunk6/trunk6.mm:84-168).
//
// Two launches: stream_gemm (raw partial products of k-splits) and a finisher that sums the splits in index order,
// applies H_out and svh. Used for the trunk projections (K 6/7/8) and as the building block of the tests.
#pragma once
#include "stream_gemm.cuh"

namespace ijah {

struct LinearPlan {
  int in, out, K, rows;
  int IT, OT, NG;     // k-tiles, n-tiles, n-groups of 8 tiles
  int S, kc;          // k-splits and k-tiles per split
  int hi, ho;         // Hadamard sizes
  int MT;             // 16-row MMA tiles
  StreamLayout lay;
  int grid;
  size_t raw_floats() const { return (size_t)S * rows * out; }
};

LinearPlan plan_linear(int in, int out, int K, int rows);

struct LinearProblem {
  struct Unit : UnitBase {
    int g, s, k0;
  };
  const char *trellis;
  const __half *suh;
  const float *x;
  float *raw;
  int in, out, K, rows, IT, OT, NG, S, kc, hi;
  float hscale;

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
    un.kstride = (uint32_t)OT * 32u * (uint32_t)K;
    un.w = trellis + ((size_t)un.k0 * OT + (size_t)un.g * SG_WARPS) * (32u * K);
    return un;
  }
  // A[r][i] = half(H_hi(x[r] * suh))[k0*16 + i]: product and butterflies in fp32, one rounding to fp16
  __device__ void prologue(const Unit &un, __half *A, int lda, int warp, int lane) const {
    const int n = un.kc * 16, nch = (n + 127) >> 7;
    for (int job = warp; job < rows * nch; job += SG_WARPS) {
      const int r = job / nch, c = (job - r * nch) << 7;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int i = c + lane + 32 * j, gi = un.k0 * 16 + i;
        v[j] = i < n ? x[(size_t)r * in + gi] * __half2float(suh[gi]) : 0.0f;
      }
      fwht_chunk(v, lane, hi, hscale);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int i = c + lane + 32 * j;
        if (i < n) A[(size_t)r * lda + i] = __float2half_rn(v[j]);
      }
    }
  }
  __device__ void store(const Unit &un, int row, int col, float v0, float v1) const {
    *reinterpret_cast<float2 *>(raw + ((size_t)un.s * rows + row) * out + un.g * 128 + col) = make_float2(v0, v1);
  }
};

void launch_linear(const LinearPlan &p, const void *trellis, const void *suh, const void *svh, const float *x, float *y,
                   float *raw, int *status, cudaStream_t st);

// W' as fp16 [in][out] (bit-exact codebook values), for parity checks of the decoder
void launch_dequant(const void *trellis, int in, int out, int K, __half *w, cudaStream_t st);

// shared-memory carve-up for a stream_gemm launch: kcmax k-tiles of A for arows rows, ring sized to what is left
StreamLayout make_layout(int Kmax, int kcmax, int arows, int ctas_per_sm);


}  // namespace ijah
