// Streaming trellis GEMM for decode widths (1..64 activation rows) on sm_100a.
//
//   raw[rows][cols] = A[rows][k] (fp16, prepared beforehand in global memory)  x  W'[k][cols] (EXL3 tiles, decoded in
//   registers)
//
// One CTA = 8 consumer warps + 1 producer warp and is persistent over a list of work units. A unit is a block of
// <= 8 output tiles (128 columns) x a run of k-tiles of one matrix. The producer thread moves everything with 1-D bulk
// async copies (global -> shared, mbarrier transaction counts): the unit's A rows into one of a few A slots, and the
// unit's compressed tiles into a ring of stages. It runs ahead across unit boundaries, so HBM stays busy and the
// consumers never wait for an operand that could have been fetched earlier. Each consumer warp owns one output tile:
// per k-tile it reads its lane window (3 words) from the ring, decodes 8 weights per lane and issues two
// mma.m16n8k16 per 16 activation rows; accumulators are fp32 registers. Only compressed bytes cross HBM.
//
// The "problem" type P supplies the unit list and the operand / result addresses:
//   int  P::num_units() const
//   Unit P::unit(int u) const                         // where the tiles are, how many k-steps, K, rows, ...
//   int  P::row_index(const Unit&, int i) const       // which operand / result row the unit's i-th row is
//   const __half *P::a_row(const Unit&, int idx) const  // global address of that row's first element of the unit's k range
//   void P::store(const Unit&, int idx, int col, float v) const   // raw output element (row idx, col)
#pragma once
#include "exl3_decode.cuh"
#include "pipeline.cuh"

// SG_DBG: timing-only builds that answer "is it the decode, the MMA or the bytes" (results are wrong on purpose):
// 1 = decode but no MMA, 2 = MMA on the undecoded words. 0 = the product.
#ifndef SG_DBG
#define SG_DBG 0
#endif

namespace ijah {

constexpr int SG_WARPS = 8;               // consumer warps = output tiles per unit
constexpr int SG_THREADS = 32 * (SG_WARPS + 1);
constexpr int SG_KS = 8;                  // k-steps per ring stage
constexpr int SG_MAX_STAGES = 16;
constexpr int SG_MAX_ASLOTS = 4;
constexpr int SG_DESC_UNIT_BYTES = 128;   // shared-memory room for one unit descriptor
constexpr int SG_DESC_BYTES = SG_DESC_UNIT_BYTES + 64 * 4;  // + the row indices of up to 64 rows

struct UnitBase {
  const char *w;       // first tile of the unit: tile (k0, n0)
  uint32_t kstride;    // bytes between consecutive k-tiles of the same column tile (= out/16 * 32K)
  int kc;              // k-tiles in this unit
  int ntiles;          // output tiles (1..8)
  int K;               // bits per weight
  int nrows;           // live activation rows (<= 8 * MT)
};

struct StreamLayout {  // dynamic shared memory carve-up (host computes, kernel mirrors)
  int stages;          // ring stages
  int stage_bytes;     // SG_KS * 8 * 32 * Kmax
  int lda;             // A row stride in halfs (k elements + 8 pad: keeps ldmatrix rows on distinct banks)
  int arows;           // rows per A slot
  int aslots;          // A slots (units the producer may run ahead)
  __host__ __device__ size_t ring_off() const { return 512 + SG_MAX_ASLOTS * SG_DESC_BYTES; }
  __host__ __device__ size_t slot_bytes() const { return (size_t)arows * lda * 2; }
  __host__ __device__ size_t a_off() const { return ring_off() + (size_t)stages * stage_bytes; }
  __host__ __device__ size_t zero_off() const { return a_off() + (size_t)aslots * slot_bytes(); }
  __host__ __device__ size_t total() const { return zero_off() + (size_t)lda * 2; }
};

// shared-memory loads with the constant part of the address as an immediate (no address arithmetic per tile)
template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr), "n"(OFF));
}

// k-tile I of a stage for one output tile. The tensor core computes D^T = W'^T * X^T: the decoded tile is the A operand
// (16 output columns x 16 k; the lane's 8 decoded weights are exactly its A fragment, in the order b0, b2, b1, b3), the
// activations are the B operand (16 k x 8 rows), so 8 activation rows cost one mma.m16n8k16 per tile. MT = number of
// 8-row groups (1, 2, 4, 8); a_row[p] is the ldmatrix address of row-group pair p for k-tile 0 of the stage, tile I
// sits I * 32 bytes further in the A rows. acc[g] = D^T fragment of group g: (column gq, rows 2q, 2q+1), (column gq + 8, ..).
template <int MT>
struct RowPairs { static constexpr int N = MT == 1 ? 1 : MT / 2; };

template <int OFF>
__device__ __forceinline__ void ldsm2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2+%3];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr), "n"(OFF));
}

template <int K, int MT, int I>
__device__ __forceinline__ void tile_mma(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t la,
                                         const uint32_t (&a_row)[RowPairs<MT>::N], float (&acc)[MT][4]) {
  uint32_t b[4];
#if SG_DBG == 2  // timing only: no decode, the raw words go to the tensor core
  b[0] = w0; b[1] = w1; b[2] = w2; b[3] = w0 ^ la;
#else
  dec8<K>(w0, w1, w2, la, b);
#endif
#if SG_DBG == 1  // timing only: decode without the MMA
  acc[0][0] = __uint_as_float(__float_as_uint(acc[0][0]) ^ b[0] ^ b[1]);
  acc[0][1] = __uint_as_float(__float_as_uint(acc[0][1]) ^ b[2] ^ b[3]);
  (void)a_row;
#else
  const uint32_t wa[4] = {b[0], b[2], b[1], b[3]};
  if constexpr (MT == 1) {
    uint32_t x[2];
    ldsm2<I * 32>(x, a_row[0]);
    mma_16816(acc[0], wa, x[0], x[1]);
  } else {
#pragma unroll
    for (int p = 0; p < MT / 2; p++) {
      uint32_t x[4];
      ldsm4<I * 32>(x, a_row[p]);
      mma_16816(acc[2 * p], wa, x[0], x[1]);
      mma_16816(acc[2 * p + 1], wa, x[2], x[3]);
    }
  }
#endif
}
// A stage's SG_KS k-tiles: all window words are loaded first (3 * SG_KS independent shared loads in flight), then
// decoded and multiplied tile by tile.
template <int K, int MT, int I, int N>
struct TileLoop {
  static constexpr int KSTEP = SG_WARPS * Codec<K>::TILE_BYTES;
  static constexpr int NP = RowPairs<MT>::N;
  static __device__ __forceinline__ void load(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t (&w)[SG_KS][3]) {
    w[I][0] = lds32<I * KSTEP>(p0);
    w[I][1] = lds32<I * KSTEP>(p1);
    w[I][2] = lds32<I * KSTEP>(p2);
    TileLoop<K, MT, I + 1, N>::load(p0, p1, p2, w);
  }
  static __device__ __forceinline__ void run(const uint32_t (&w)[SG_KS][3], uint32_t la, const uint32_t (&a_row)[NP],
                                             float (&acc)[MT][4], int n) {
    if (I < n) tile_mma<K, MT, I>(w[I][0], w[I][1], w[I][2], la, a_row, acc);
    TileLoop<K, MT, I + 1, N>::run(w, la, a_row, acc, n);
  }
  static __device__ __forceinline__ void run_all(const uint32_t (&w)[SG_KS][3], uint32_t la, const uint32_t (&a_row)[NP],
                                                 float (&acc)[MT][4]) {  // straight-line: the tiles interleave freely
    tile_mma<K, MT, I>(w[I][0], w[I][1], w[I][2], la, a_row, acc);
    TileLoop<K, MT, I + 1, N>::run_all(w, la, a_row, acc);
  }
};
template <int K, int MT, int N>
struct TileLoop<K, MT, N, N> {
  static constexpr int NP = RowPairs<MT>::N;
  static __device__ __forceinline__ void load(uint32_t, uint32_t, uint32_t, uint32_t (&)[SG_KS][3]) {}
  static __device__ __forceinline__ void run(const uint32_t (&)[SG_KS][3], uint32_t, const uint32_t (&)[NP], float (&)[MT][4], int) {}
  static __device__ __forceinline__ void run_all(const uint32_t (&)[SG_KS][3], uint32_t, const uint32_t (&)[NP], float (&)[MT][4]) {}
};

// All k-steps of one unit for one warp. Returns false if a bounded wait gave up.
template <int K, int MT>
__device__ __forceinline__ bool consume_unit(int kc, uint32_t ring_addr, int stage_bytes, int nstages, uint64_t *full,
                                             uint64_t *empty, int &stage, uint32_t &phase, bool live, int warp, int lane,
                                             uint32_t a_addr, const uint32_t (&a_rowoff)[RowPairs<MT>::N], float (&acc)[MT][4],
                                             int *status) {
  const typename Codec<K>::Lane L = Codec<K>::lane(lane);
  const uint32_t tb = ring_addr + (uint32_t)warp * Codec<K>::TILE_BYTES;
  for (int k = 0; k < kc; k += SG_KS) {
    if (!mbar_wait(&full[stage], phase, status, 2)) return false;
    if (live) {
      const uint32_t sb = tb + (uint32_t)stage * (uint32_t)stage_bytes;
      const uint32_t p0 = sb + L.o0, p1 = sb + L.o1, p2 = sb + L.o2;
      uint32_t a_row[RowPairs<MT>::N];
#pragma unroll
      for (int m = 0; m < RowPairs<MT>::N; m++) a_row[m] = a_addr + a_rowoff[m] + (uint32_t)k * 32u;
      uint32_t w[SG_KS][3];
      TileLoop<K, MT, 0, SG_KS>::load(p0, p1, p2, w);  // a short last stage loads stale ring bytes it never uses
      if (kc - k >= SG_KS) TileLoop<K, MT, 0, SG_KS>::run_all(w, L.a, a_row, acc);
      else TileLoop<K, MT, 0, SG_KS>::run(w, L.a, a_row, acc, kc - k);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);
    if (++stage == nstages) { stage = 0; phase ^= 1u; }
  }
  return true;
}

// per-unit dispatch on the bits per weight and on the unit's live rows: a launch compiled for up to 8 * MT rows runs a unit
// with fewer rows through the narrowest path that holds them (one MMA per 8 rows), since most units of a wide launch are
// experts that only one or two rows selected
template <int K, int MT, int SUB>
__device__ __forceinline__ bool consume_rows(int nrows, int kc, uint32_t ring_addr, int stage_bytes, int nstages, uint64_t *full,
                                             uint64_t *empty, int &stage, uint32_t &phase, bool live, int warp, int lane, uint32_t a_addr,
                                             const uint32_t (&a_rowoff)[RowPairs<MT>::N], float (&acc)[MT][4], int *status) {
  if constexpr (SUB < MT) {
    if (nrows <= 8 * SUB)
      return consume_unit<K, SUB>(kc, ring_addr, stage_bytes, nstages, full, empty, stage, phase, live, warp, lane, a_addr,
                                  reinterpret_cast<const uint32_t(&)[RowPairs<SUB>::N]>(a_rowoff), reinterpret_cast<float(&)[SUB][4]>(acc),
                                  status);
    return consume_rows<K, MT, SUB * 2>(nrows, kc, ring_addr, stage_bytes, nstages, full, empty, stage, phase, live, warp, lane, a_addr,
                                        a_rowoff, acc, status);
  } else {
    return consume_unit<K, MT>(kc, ring_addr, stage_bytes, nstages, full, empty, stage, phase, live, warp, lane, a_addr, a_rowoff, acc, status);
  }
}

template <int MT>
__device__ __forceinline__ bool consume_any(int K, int nrows, int kc, uint32_t ring_addr, int stage_bytes, int nstages,
                                            uint64_t *full, uint64_t *empty, int &stage, uint32_t &phase, bool live, int warp,
                                            int lane, uint32_t a_addr, const uint32_t (&a_rowoff)[RowPairs<MT>::N],
                                            float (&acc)[MT][4], int *status) {
#define SG_CASE(KK)                                                                                                                 \
  case KK:                                                                                                                          \
    return consume_rows<KK, MT, 1>(nrows, kc, ring_addr, stage_bytes, nstages, full, empty, stage, phase, live, warp, lane, a_addr, \
                                   a_rowoff, acc, status);
  switch (K) {
    SG_CASE(4)
    SG_CASE(5)
    SG_CASE(6)
    SG_CASE(7)
    default:
      SG_CASE(8)
  }
#undef SG_CASE
}

template <class P, int MT>
__global__ void __launch_bounds__(SG_THREADS, 2) stream_gemm_kernel(const P prob, const StreamLayout lay, int *status) {
  static_assert(sizeof(typename P::Unit) <= SG_DESC_UNIT_BYTES, "unit descriptor too large for its shared-memory slot");
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + SG_MAX_STAGES;
  uint64_t *a_full = empty + SG_MAX_STAGES;
  uint64_t *a_empty = a_full + SG_MAX_ASLOTS;
  unsigned char *desc = smem + 512;  // per A slot: the unit descriptor, then the row indices of its rows
  unsigned char *ring = smem + lay.ring_off();
  unsigned char *aslot = smem + lay.a_off();
  unsigned char *zrow = smem + lay.zero_off();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < lay.stages; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], SG_WARPS);
    }
    for (int s = 0; s < lay.aslots; s++) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], SG_WARPS);
    }
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < lay.lda / 2; i += blockDim.x) reinterpret_cast<uint32_t *>(zrow)[i] = 0u;
  __syncthreads();

  if (warp == SG_WARPS) {
    // ---------------------------------------------------------------- producer (one warp, lanes work in parallel)
    // Only this warp reads the unit list from global memory; the consumers get each unit's descriptor and row indices
    // through shared memory together with the A rows, so no consumer ever waits on a global load. The next unit's
    // descriptor is fetched while the current unit's copies are issued, and lane i issues copy i, so the metadata
    // latency and the issue cost of the copies stay off the critical path.
    //
    // Start-up under programmatic dependent launch: the A rows (and for some problems the unit list itself) are written
    // by the preceding kernel, the compressed weights are not. A problem whose unit list is final when the kernel is
    // launched (P::kUnitsFinalAtLaunch) streams the first unit's weight stages into the fresh ring before it waits for
    // the predecessor, so the ring is full when the A rows arrive.
    int stage = 0, slot = 0;
    uint32_t phase = 0, aphase = 0;
    int u = blockIdx.x;
    typename P::Unit un;
    int nunits = 0, k_pre = 0;
    const uint64_t wpol = l2_evict_first_policy();
    if constexpr (P::kUnitsFinalAtLaunch) {
      nunits = prob.num_units();
      if (u < nunits) {
        un = prob.unit(u);
        const uint32_t kb = (uint32_t)un.ntiles * 32u * (uint32_t)un.K, ks = (uint32_t)SG_WARPS * 32u * (uint32_t)un.K;
        for (; k_pre < un.kc && stage < lay.stages; k_pre += SG_KS) {  // fresh ring: no empty-wait needed
          const int n = min(SG_KS, un.kc - k_pre);
          if (lane == 0) mbar_arrive_expect_tx(&full[stage], (uint32_t)n * kb);
          __syncwarp();
          if (lane < n)
            bulk_g2s_hint(ring + (size_t)stage * lay.stage_bytes + lane * ks, un.w + (size_t)(k_pre + lane) * un.kstride, kb, &full[stage], wpol);
          ++stage;
        }
        if (stage == lay.stages) { stage = 0; phase ^= 1u; }
      }
      pdl_wait();
    } else {
      pdl_wait();
      nunits = prob.num_units();
      if (u < nunits) un = prob.unit(u);
    }
    pdl_launch();
    while (u < nunits) {
      const int u_next = u + gridDim.x;
      typename P::Unit nx;
      if (u_next < nunits) nx = prob.unit(u_next);
      const int i0 = lane < un.nrows ? prob.row_index(un, lane) : 0;
      const int i1 = lane + 32 < un.nrows ? prob.row_index(un, lane + 32) : 0;
      if (!mbar_wait(&a_empty[slot], aphase ^ 1u, status, 3)) return;
      typename P::Unit *du = reinterpret_cast<typename P::Unit *>(desc + (size_t)slot * SG_DESC_BYTES);
      int *didx = reinterpret_cast<int *>(desc + (size_t)slot * SG_DESC_BYTES + SG_DESC_UNIT_BYTES);
      didx[lane] = i0;
      didx[lane + 32] = i1;
      const uint32_t rowb = (uint32_t)un.kc * 32u;
      __syncwarp();
      if (lane == 0) {
        *du = un;
        mbar_arrive_expect_tx(&a_full[slot], (uint32_t)un.nrows * rowb);  // release: descriptor and indices are visible
      }
      __syncwarp();
      unsigned char *adst = aslot + (size_t)slot * lay.slot_bytes();
      if (lane < un.nrows) bulk_g2s(adst + (size_t)lane * lay.lda * 2, prob.a_row(un, i0), rowb, &a_full[slot]);
      if (lane + 32 < un.nrows) bulk_g2s(adst + (size_t)(lane + 32) * lay.lda * 2, prob.a_row(un, i1), rowb, &a_full[slot]);
      if (++slot == lay.aslots) { slot = 0; aphase ^= 1u; }
      // compressed tiles, SG_KS k-steps per stage, lane i copies k-step i
      const uint32_t kb = (uint32_t)un.ntiles * 32u * (uint32_t)un.K, ks = (uint32_t)SG_WARPS * 32u * (uint32_t)un.K;
      for (int k = k_pre; k < un.kc; k += SG_KS) {
        const int n = min(SG_KS, un.kc - k);
        if (!mbar_wait(&empty[stage], phase ^ 1u, status, 1)) return;
        if (lane == 0) mbar_arrive_expect_tx(&full[stage], (uint32_t)n * kb);
        __syncwarp();
        if (lane < n)
          bulk_g2s_hint(ring + (size_t)stage * lay.stage_bytes + lane * ks, un.w + (size_t)(k + lane) * un.kstride, kb, &full[stage], wpol);
        if (++stage == lay.stages) { stage = 0; phase ^= 1u; }
      }
      k_pre = 0;
      un = nx;
      u = u_next;
    }
    return;
  }

  // ------------------------------------------------------------------ consumers (8 warps)
  const int g = lane >> 2, q = lane & 3;
  int stage = 0, slot = 0;
  uint32_t phase = 0, aphase = 0;
  // ldmatrix row addresses: lanes 0-7 rows 0-7 (k 0-7), 8-15 rows 0-7 (k 8-15), 16-23 rows 8-15 (k 0-7), 24-31 rows 8-15
  // (k 8-15); the .x2 form used for <= 8 rows takes the first 16 lanes' addresses
  const int lrow = (lane & 7) + (lane >> 4) * 8;
  const uint32_t lkof = (uint32_t)((lane >> 3) & 1) * 16u;
  const uint32_t ring_addr = smem_u32(ring), a0_addr = smem_u32(aslot), z_addr = smem_u32(zrow);

  if constexpr (!P::kUnitsFinalAtLaunch) pdl_wait();  // the unit count is the predecessor's output
  const int nunits = prob.num_units();
  for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
    if (!mbar_wait(&a_full[slot], aphase, status, 4)) return;
    const typename P::Unit un = *reinterpret_cast<const typename P::Unit *>(desc + (size_t)slot * SG_DESC_BYTES);
    const int *didx = reinterpret_cast<const int *>(desc + (size_t)slot * SG_DESC_BYTES + SG_DESC_UNIT_BYTES);
    int idx[MT][2];  // row indices of the accumulator entries this lane holds: rows 8 m + 2q and 8 m + 2q + 1
#pragma unroll
    for (int m = 0; m < MT; m++) {
      idx[m][0] = m * 8 + 2 * q < un.nrows ? didx[m * 8 + 2 * q] : -1;
      idx[m][1] = m * 8 + 2 * q + 1 < un.nrows ? didx[m * 8 + 2 * q + 1] : -1;
    }
    const uint32_t a_addr = a0_addr + (uint32_t)slot * (uint32_t)lay.slot_bytes();
    uint32_t a_rowoff[RowPairs<MT>::N];
#pragma unroll
    for (int m = 0; m < RowPairs<MT>::N; m++) {
      const int r = m * 16 + lrow;  // dead rows read the zero row
      a_rowoff[m] = (r < un.nrows ? (uint32_t)r * (uint32_t)lay.lda * 2u : (z_addr - a_addr)) + lkof;
    }
    float acc[MT][4];
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
      for (int j = 0; j < 4; j++) acc[m][j] = 0.0f;

    const bool live = warp < un.ntiles;
    if (!consume_any<MT>(un.K, un.nrows, un.kc, ring_addr, lay.stage_bytes, lay.stages, full, empty, stage, phase, live, warp, lane,
                         a_addr, a_rowoff, acc, status))
      return;
    __syncwarp();
    if (lane == 0) mbar_arrive(&a_empty[slot]);  // descriptor and A rows are in registers / consumed: slot may be refilled
    if (++slot == lay.aslots) { slot = 0; aphase ^= 1u; }
    if (live) {
      const int col = warp * 16 + g;
#pragma unroll
      for (int m = 0; m < MT; m++) {
        if (idx[m][0] >= 0) { prob.store(un, idx[m][0], col, acc[m][0]); prob.store(un, idx[m][0], col + 8, acc[m][2]); }
        if (idx[m][1] >= 0) { prob.store(un, idx[m][1], col, acc[m][1]); prob.store(un, idx[m][1], col + 8, acc[m][3]); }
      }
    }
  }
}

}  // namespace ijah
