// Streaming trellis GEMM for decode widths (1..64 activation rows) on sm_100a.
//
//   raw[rows][cols] (+)= A[rows][k] (fp16, prepared in shared memory)  x  W'[k][cols] (EXL3 tiles, decoded in registers)
//
// One CTA = 8 consumer warps + 1 producer warp and is persistent over a list of work units. A unit is a block of
// <= 8 output tiles (128 columns) x a run of k-tiles of one matrix. The producer thread streams the unit's compressed
// tiles global -> shared with 1-D bulk async copies into a ring of stages (mbarrier transaction counts), running ahead
// across unit boundaries, so HBM stays busy while the consumers build the next unit's A operand. Each consumer warp owns
// one output tile: per k-tile it reads its lane window (3 words) from the ring, decodes 8 weights per lane and issues
// two mma.m16n8k16 per 16 activation rows; accumulators are fp32 registers. Only compressed bytes cross HBM.
//
// The "problem" type P supplies the unit list and the pre/post work:
//   int  P::num_units() const
//   Unit P::unit(int u) const                 // where the tiles are, how many k-steps, K, rows, ...
//   void P::prologue(const Unit&, __half *A, int lda, int warp, int lane) const   // fill A[row][k] (8 warps)
//   void P::store(const Unit&, int row, int col, float v0, float v1) const        // raw output of (row, col..col+1)
#pragma once
#include "exl3_decode.cuh"
#include "pipeline.cuh"

namespace ijah {

constexpr int SG_WARPS = 8;               // consumer warps = output tiles per unit
constexpr int SG_THREADS = 32 * (SG_WARPS + 1);
constexpr int SG_KS = 4;                  // k-steps per ring stage

struct UnitBase {
  const char *w;       // first tile of the unit: tile (k0, n0)
  uint32_t kstride;    // bytes between consecutive k-tiles of the same column tile (= out/16 * 32K)
  int kc;              // k-tiles in this unit
  int ntiles;          // output tiles (1..8)
  int K;               // bits per weight
  int nrows;           // live activation rows (<= 16 * MT)
};

struct StreamLayout {  // dynamic shared memory carve-up (host computes, kernel mirrors)
  int stages;          // ring stages
  int stage_bytes;     // SG_KS * 8 * 32 * Kmax
  int lda;             // A row stride in halfs (k elements + 8 pad)
  int arows;           // A rows held (live rows only; dead MMA rows read the zero row)
  __host__ __device__ size_t ring_off() const { return 256; }
  __host__ __device__ size_t a_off() const { return ring_off() + (size_t)stages * stage_bytes; }
  __host__ __device__ size_t zero_off() const { return a_off() + (size_t)arows * lda * 2; }
  __host__ __device__ size_t total() const { return zero_off() + (size_t)lda * 2; }
};

template <int K, int MT>
__device__ __forceinline__ void consume_stage(const char *stage, int nsteps, int kstep_bytes, int warp, uint32_t a_addr,
                                              const uint32_t (&a_rowoff)[MT], int kbase, const typename Codec<K>::Lane &L,
                                              float (&acc)[MT][2][4]) {
  const char *tile = stage + warp * Codec<K>::TILE_BYTES;
#pragma unroll
  for (int i = 0; i < SG_KS; i++) {
    if (i < nsteps) {
      const char *t = tile + i * kstep_bytes;
      const uint32_t w0 = *reinterpret_cast<const uint32_t *>(t + L.o0);
      const uint32_t w1 = *reinterpret_cast<const uint32_t *>(t + L.o1);
      const uint32_t w2 = *reinterpret_cast<const uint32_t *>(t + L.o2);
      uint32_t b[4];
      dec8<K>(w0, w1, w2, L.a, b);
#pragma unroll
      for (int m = 0; m < MT; m++) {
        uint32_t a[4];
        ldmatrix_x4(a, a_addr + a_rowoff[m] + (uint32_t)(kbase + i) * 32u);
        mma_16816(acc[m][0], a, b[0], b[1]);
        mma_16816(acc[m][1], a, b[2], b[3]);
      }
    }
  }
}

template <class P, int MT>
__global__ void __launch_bounds__(SG_THREADS, 2) stream_gemm_kernel(const P prob, const StreamLayout lay, int *status) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + 16;
  char *ring = reinterpret_cast<char *>(smem + lay.ring_off());
  __half *A = reinterpret_cast<__half *>(smem + lay.a_off());
  __half *zrow = reinterpret_cast<__half *>(smem + lay.zero_off());
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < lay.stages; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], SG_WARPS);
    }
    mbar_fence_init();
    s_abort = 0;
  }
  for (int i = threadIdx.x; i < lay.lda / 2; i += blockDim.x) reinterpret_cast<uint32_t *>(zrow)[i] = 0u;
  __syncthreads();
  const int nunits = prob.num_units();

  if (warp == SG_WARPS) {
    // ---------------------------------------------------------------- producer (one thread)
    if (lane != 0) return;
    int stage = 0;
    uint32_t phase = 0;
    long issued = 0;
    for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
      const typename P::Unit un = prob.unit(u);
      const uint32_t kb = (uint32_t)un.ntiles * 32u * (uint32_t)un.K;
      for (int k = 0; k < un.kc; k += SG_KS) {
        const int n = min(SG_KS, un.kc - k);
        if (issued >= lay.stages && !mbar_wait(&empty[stage], phase ^ 1u, status, 1)) { s_abort = 1; return; }
        if (*reinterpret_cast<volatile int *>(&s_abort)) return;
        mbar_arrive_expect_tx(&full[stage], (uint32_t)n * kb);
        char *dst = ring + (size_t)stage * lay.stage_bytes;
        for (int i = 0; i < n; i++) bulk_g2s(dst + i * kb, un.w + (size_t)(k + i) * un.kstride, kb, &full[stage]);
        issued++;
        if (++stage == lay.stages) { stage = 0; phase ^= 1u; }
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers (8 warps)
  const int g = lane >> 2, q = lane & 3;
  int stage = 0;
  uint32_t phase = 0;
  // ldmatrix row addresses: lanes 0-7 rows 0-7 (k 0-7), 8-15 rows 8-15, 16-23 rows 0-7 (k 8-15), 24-31 rows 8-15
  const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
  const uint32_t lkof = (uint32_t)(lane >> 4) * 16u;
  const uint32_t a_base = smem_u32(A), z_base = smem_u32(zrow);

  for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
    const typename P::Unit un = prob.unit(u);
    asm volatile("bar.sync 1, %0;" ::"n"(32 * SG_WARPS));  // everyone is done reading the previous unit's A
    prob.prologue(un, A, lay.lda, warp, lane);
    asm volatile("bar.sync 1, %0;" ::"n"(32 * SG_WARPS));

    uint32_t a_rowoff[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const int r = m * 16 + lrow;
      // offsets are relative to a_base; dead rows are redirected to the zero row
      a_rowoff[m] = (r < un.nrows ? (uint32_t)r * (uint32_t)lay.lda * 2u : (z_base - a_base)) + lkof;
    }
    float acc[MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
      for (int h = 0; h < 2; h++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[m][h][j] = 0.0f;

    const int kb = un.ntiles * 32 * un.K;
    const bool live = warp < un.ntiles;
    bool ok = true;
    for (int k = 0; k < un.kc && ok; k += SG_KS) {
      const int n = min(SG_KS, un.kc - k);
      ok = mbar_wait(&full[stage], phase, status, 2);
      if (!ok) { s_abort = 1; break; }
      const char *st = ring + (size_t)stage * lay.stage_bytes;
      if (live) {
        switch (un.K) {
          case 4: consume_stage<4, MT>(st, n, kb, warp, a_base, a_rowoff, k, Codec<4>::lane(lane), acc); break;
          case 5: consume_stage<5, MT>(st, n, kb, warp, a_base, a_rowoff, k, Codec<5>::lane(lane), acc); break;
          case 6: consume_stage<6, MT>(st, n, kb, warp, a_base, a_rowoff, k, Codec<6>::lane(lane), acc); break;
          case 7: consume_stage<7, MT>(st, n, kb, warp, a_base, a_rowoff, k, Codec<7>::lane(lane), acc); break;
          default: consume_stage<8, MT>(st, n, kb, warp, a_base, a_rowoff, k, Codec<8>::lane(lane), acc); break;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
      if (++stage == lay.stages) { stage = 0; phase ^= 1u; }
    }
    if (!ok) break;
    if (live) {
      const int col = warp * 16 + 2 * q;
#pragma unroll
      for (int m = 0; m < MT; m++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int r0 = m * 16 + g;
          if (r0 < un.nrows) prob.store(un, r0, col + 8 * h, acc[m][h][0], acc[m][h][1]);
          if (r0 + 8 < un.nrows) prob.store(un, r0 + 8, col + 8 * h, acc[m][h][2], acc[m][h][3]);
        }
    }
  }
}

}  // namespace ijah
