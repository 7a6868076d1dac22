// Streaming trellis GEMM for decode widths (1..64 activation rows) on sm_100a.
//
//   raw[rows][cols] = A[rows][k] (fp16, prepared beforehand in global memory)  x  W'[k][cols] (EXL3 tiles, decoded in
//   registers)
//
// One CTA = 8 consumer warps + 1 producer warp and is persistent over a list of work units. A unit is a block of
// <= 8 output tiles (128 columns) x a run of k-tiles of one matrix. The producer moves the compressed tiles with ONE tiled
// TMA copy per ring stage (a 3-D tensor map over the trellis: x = bytes along the tile row, y = k-tile, z = expert; box =
// 8 tiles x SG_KS k-tiles) and the unit's A rows with 1-D bulk copies into one of a few A slots, always one unit ahead
// of the tiles; completion is signalled on mbarriers by transaction count. It runs ahead across unit boundaries, so HBM
// stays busy and the consumers never wait for an operand that could have been fetched earlier. The producer warp shares
// its scheduler with consumer warps that are always ready to issue, so every instruction it needs per stage delays the
// stream: one copy instruction per stage (instead of one per k-tile) is what keeps the ring full. Each consumer warp owns one output tile:
// per k-tile it reads its lane window (3 words) from the ring, decodes 8 weights per lane and issues two
// mma.m16n8k16 per 16 activation rows; accumulators are fp32 registers. Only compressed bytes cross HBM.
//
// The "problem" type P supplies the unit list and the operand / result addresses:
//   bool P::units_final() const                        // the unit list does not depend on the preceding kernel's output
//   int  P::num_units() const
//   Unit P::unit(int u) const                         // where the tiles are, how many k-steps, K, rows, ...
//   const CUtensorMap *P::tmap(int i) const            // tensor map i over a trellis (see make_trellis_map)
//   int  P::row_index(const Unit&, int i) const       // which operand / result row the unit's i-th row is
//   const __half *P::a_row(const Unit&, int idx) const  // global address of that row's first element of the unit's k range
//   float *P::out_base(const Unit&) const               // raw output of the unit: element (row idx, unit column c) is
//   int P::out_row_off(const Unit&, int idx) const      //   out_base(un)[out_row_off(un, idx) + c]
#pragma once
#include <cuda.h>

#include "exl3_decode.cuh"
#include "pipeline.cuh"

// SG_DBG: timing-only builds that answer "is it the decode, the MMA or the bytes" (results are wrong on purpose):
// 1 = decode but no MMA, 2 = MMA on the undecoded words. 0 = the product.
#ifndef SG_DBG
#define SG_DBG 0
#endif

namespace ijah {

#ifndef SG_KS_STEPS
#define SG_KS_STEPS 16
#endif
#ifndef SG_CTAS_PER_SM
#define SG_CTAS_PER_SM 2
#endif
constexpr int SG_WARPS = 8;               // consumer warps = output tiles per unit
constexpr int SG_THREADS = 32 * (SG_WARPS + 1);
constexpr int SG_KS = SG_KS_STEPS;        // k-steps per ring stage
constexpr int SG_CTAS = SG_CTAS_PER_SM;   // persistent CTAs per SM
constexpr int SG_MAX_STAGES = 16;
constexpr int SG_MAX_ASLOTS = 4;
constexpr int SG_DESC_UNIT_BYTES = 128;   // shared-memory room for one unit descriptor
constexpr int SG_DESC_BYTES = SG_DESC_UNIT_BYTES + 64 * 4;  // + the row indices of up to 64 rows

struct UnitBase {
  int map;             // which of the problem's tensor maps (P::tmap) holds the unit's tiles
  int x, y, z;         // box coordinates of the unit's first stage: x in 8-byte elements (= n0 * 4K), y = first k-tile, z = expert
  int kc;              // k-tiles in this unit
  int ntiles;          // output tiles (1..8)
  int K;               // bits per weight
  int nrows;           // live activation rows (<= 8 * MT)
};

// What the consumer warps need of a unit; the producer writes it into the unit's A slot together with one output row
// offset per activation row, so the consumers never touch the unit list nor do any address arithmetic beyond one add.
struct UnitDesc {
  float *out;
  int kc, ntiles, K, nrows;
};

struct StreamLayout {  // dynamic shared memory carve-up (host computes, kernel mirrors)
  int stages;          // ring stages
  int stage_bytes;     // SG_KS * 8 * 32 * Kmax
  int lda;             // A row stride in halfs (32 per k-tile + 8 pad: keeps ldmatrix rows on distinct banks)
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
// (16 output columns x 16 k), the activations are the B operand (16 k x 8 rows). Each decoded weight arrives as the pair of
// fp16 summands (lo, hi) the codebook function yields (dec8_raw) and takes the place of TWO k elements of the A fragment,
// against activation rows that hold two halfs per input (store_a), so the 16 inputs of the k-tile take two mma.m16n8k16
// per 8 activation rows: the even inputs (slots 0, 4, 2, 6 of the lane) and the odd ones (slots 1, 5, 3, 7).
//   EX (default): one half add turns (lo, hi) into (w, w), w = fp16(lo + hi), the weight as the format defines it; the
//                 rows hold (v, 0) and the accumulator receives w * v.
//   !EX (opt-in): (lo, hi) goes in as it is against (v, v): lo * v + hi * v, the sum of the summands unrounded.
// MT = number of 8-row groups (1, 2, 4, 8); a_row[g] is the ldmatrix address of row group g for k-tile 0 of the stage,
// tile I sits I * 64 bytes further in the A rows. acc[g] = D^T fragment of group g: (column gq, rows 2q, 2q+1), (column gq + 8, ..).
constexpr uint32_t SG_A_TILE_BYTES = 16 * A_HALFS_PER_INPUT * 2;  // one k-tile of one prepared activation row

template <int K, bool EX, int MT, int I>
__device__ __forceinline__ void tile_mma(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t la, const McgConst &mc,
                                         const uint32_t (&a_row)[MT], float (&acc)[MT][4]) {
  uint32_t r[8];
#if SG_DBG == 2  // timing only: no decode, the raw words go to the tensor core
  r[0] = w0; r[1] = w1; r[2] = w2; r[3] = w0 ^ la; r[4] = w1 ^ la; r[5] = w2 ^ la; r[6] = w0 + la; r[7] = w1 + la;
#else
  dec8_raw<K>(w0, w1, w2, la, mc, r);
#endif
  if constexpr (EX) {  // both halves = fp16(lo + hi), the format's weight; the activation rows then hold (v, 0) pairs
#pragma unroll
    for (int t = 0; t < 8; t++) {
      const __half2 h = *reinterpret_cast<const __half2 *>(&r[t]);
      const __half2 w = __hadd2(__low2half2(h), __high2half2(h));
      r[t] = *reinterpret_cast<const uint32_t *>(&w);
    }
  }
#if SG_DBG == 1  // timing only: decode without the MMA
  acc[0][0] = __uint_as_float(__float_as_uint(acc[0][0]) ^ r[0] ^ r[1] ^ r[2] ^ r[3]);
  acc[0][1] = __uint_as_float(__float_as_uint(acc[0][1]) ^ r[4] ^ r[5] ^ r[6] ^ r[7]);
  (void)a_row;
#else
  const uint32_t we[4] = {r[0], r[4], r[2], r[6]}, wo[4] = {r[1], r[5], r[3], r[7]};
#pragma unroll
  for (int g = 0; g < MT; g++) {
    uint32_t x[4];
    ldsm4<I * (int)SG_A_TILE_BYTES>(x, a_row[g]);
    mma_16816(acc[g], we, x[0], x[1]);
    mma_16816(acc[g], wo, x[2], x[3]);
  }
#endif
}
// Half a stage (SG_HALF k-tiles starting at tile B): all window words are loaded first (3 * SG_HALF independent shared
// loads in flight), then decoded and multiplied tile by tile. Half stages keep the window words at 12 registers; the other
// warps of the SM cover the shared-memory latency at the start of each half.
constexpr int SG_HALF = 4;
constexpr int SG_GROUPS = SG_KS / SG_HALF;
template <int K, bool EX, int MT, int B, int I, int N>
struct TileLoop {
  static constexpr int KSTEP = SG_WARPS * Codec<K>::TILE_BYTES;
  static constexpr int NP = MT;
  static __device__ __forceinline__ void load(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t (&w)[SG_HALF][3]) {
    w[I][0] = lds32<(B + I) * KSTEP>(p0);
    w[I][1] = lds32<(B + I) * KSTEP>(p1);
    w[I][2] = lds32<(B + I) * KSTEP>(p2);
    TileLoop<K, EX, MT, B, I + 1, N>::load(p0, p1, p2, w);
  }
  static __device__ __forceinline__ void run(const uint32_t (&w)[SG_HALF][3], uint32_t la, const McgConst &mc, const uint32_t (&a_row)[NP],
                                             float (&acc)[MT][4], int n) {
    if (B + I < n) tile_mma<K, EX, MT, B + I>(w[I][0], w[I][1], w[I][2], la, mc, a_row, acc);
    TileLoop<K, EX, MT, B, I + 1, N>::run(w, la, mc, a_row, acc, n);
  }
  static __device__ __forceinline__ void run_all(const uint32_t (&w)[SG_HALF][3], uint32_t la, const McgConst &mc, const uint32_t (&a_row)[NP],
                                                 float (&acc)[MT][4]) {  // straight-line: the tiles interleave freely
    tile_mma<K, EX, MT, B + I>(w[I][0], w[I][1], w[I][2], la, mc, a_row, acc);
    TileLoop<K, EX, MT, B, I + 1, N>::run_all(w, la, mc, a_row, acc);
  }
};
template <int K, bool EX, int MT, int B, int N>
struct TileLoop<K, EX, MT, B, N, N> {
  static constexpr int NP = MT;
  static __device__ __forceinline__ void load(uint32_t, uint32_t, uint32_t, uint32_t (&)[SG_HALF][3]) {}
  static __device__ __forceinline__ void run(const uint32_t (&)[SG_HALF][3], uint32_t, const McgConst &, const uint32_t (&)[NP], float (&)[MT][4], int) {}
  static __device__ __forceinline__ void run_all(const uint32_t (&)[SG_HALF][3], uint32_t, const McgConst &, const uint32_t (&)[NP], float (&)[MT][4]) {}
};

// the SG_GROUPS groups of a stage, one after the other
template <int K, bool EX, int MT, int G, int NG>
struct StageLoop {
  static constexpr int NP = MT;
  static __device__ __forceinline__ void run_all(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t (&w)[SG_HALF][3], uint32_t la, const McgConst &mc,
                                                 const uint32_t (&a_row)[NP], float (&acc)[MT][4]) {
    TileLoop<K, EX, MT, G * SG_HALF, 0, SG_HALF>::load(p0, p1, p2, w);
    TileLoop<K, EX, MT, G * SG_HALF, 0, SG_HALF>::run_all(w, la, mc, a_row, acc);
    StageLoop<K, EX, MT, G + 1, NG>::run_all(p0, p1, p2, w, la, mc, a_row, acc);
  }
  static __device__ __forceinline__ void run(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t (&w)[SG_HALF][3], uint32_t la, const McgConst &mc,
                                             const uint32_t (&a_row)[NP], float (&acc)[MT][4], int n) {
    if (G * SG_HALF < n) {
      TileLoop<K, EX, MT, G * SG_HALF, 0, SG_HALF>::load(p0, p1, p2, w);
      TileLoop<K, EX, MT, G * SG_HALF, 0, SG_HALF>::run(w, la, mc, a_row, acc, n);
    }
    StageLoop<K, EX, MT, G + 1, NG>::run(p0, p1, p2, w, la, mc, a_row, acc, n);
  }
};
template <int K, bool EX, int MT, int NG>
struct StageLoop<K, EX, MT, NG, NG> {
  static constexpr int NP = MT;
  static __device__ __forceinline__ void run_all(uint32_t, uint32_t, uint32_t, uint32_t (&)[SG_HALF][3], uint32_t, const McgConst &,
                                                 const uint32_t (&)[NP], float (&)[MT][4]) {}
  static __device__ __forceinline__ void run(uint32_t, uint32_t, uint32_t, uint32_t (&)[SG_HALF][3], uint32_t, const McgConst &,
                                             const uint32_t (&)[NP], float (&)[MT][4], int) {}
};

// The consumer side of the ring, all in registers: stage index and parity, the shared-memory addresses of the barriers
// (empty[s] sits SG_MAX_STAGES * 8 bytes after full[s]) and of the warp's tile inside stage 0.
struct RingCursor {
  uint32_t full;          // address of full[0]
  uint32_t tile0;         // address of this warp's tile of k-step 0 in stage 0
  uint32_t stage_bytes;
  uint32_t nstages, stage, phase;
  __device__ __forceinline__ void advance() {
    const uint32_t nx = stage + 1u, wrap = nx == nstages ? 1u : 0u;
    stage = wrap ? 0u : nx;
    phase ^= wrap;
  }
};
constexpr uint32_t SG_EMPTY_OFF = SG_MAX_STAGES * 8;

// All k-steps of one unit for one warp: 8 * MT activation rows, accumulators zeroed here, results stored to
// out[rowoff[row] + col]. Returns false if a bounded wait gave up. The steady-state loop (full stages of a live warp) is
// straight-line code between one wait and one arrive; a short last stage and the warps without a tile (units narrower
// than 8 tiles) take their own loops.
template <int K, bool EX, int MT>
__device__ __forceinline__ bool consume_unit(const UnitDesc &d, RingCursor &rc, bool live, int lane, const McgConst &mc, uint32_t a_addr,
                                             uint32_t lda_bytes, uint32_t z_addr, const int *rowoff, int col, int *status) {
  const uint32_t lane0 = lane == 0 ? 1u : 0u;
  const int nfull = d.kc / SG_KS, rem = d.kc - nfull * SG_KS;
  if (!live) {
    for (int s = 0; s < nfull + (rem ? 1 : 0); s++) {
      const uint32_t bar = rc.full + rc.stage * 8u;
      if (!mbar_wait_poll(bar, rc.phase)) { atomicExch(status, 2); return false; }
      mbar_arrive_if(bar + SG_EMPTY_OFF, lane0);
      rc.advance();
    }
    return true;
  }
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; m++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[m][j] = 0.0f;
  // ldmatrix.x4 row addresses of an 8-row group: lanes 8j .. 8j+7 give rows 0-7 at byte 16 j of the k-tile (the even
  // inputs' low and high halves of the tile, then the odd inputs'). A dead row (its results are never stored) reads the
  // unit's row 0 again: the same address as a live lane, i.e. a broadcast. (A separate zero row sat at the same offset
  // modulo 128 bytes as row 0 and cost every ldmatrix a two-way bank conflict: 4 of 14 load wavefronts per tile.)
  uint32_t a_row[MT];
  {
    const uint32_t lkof = (uint32_t)(lane >> 3) * 16u;
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const int r = m * 8 + (lane & 7);
      a_row[m] = a_addr + (uint32_t)(r < d.nrows ? r : 0) * lda_bytes + lkof;
    }
  }
  (void)z_addr;
  const typename Codec<K>::Lane L = Codec<K>::lane(lane);
  const uint32_t d1 = L.o1 - L.o0, d2 = L.o2 - L.o0, t0 = rc.tile0 + L.o0;
  uint32_t w[SG_HALF][3];
  for (int s = 0; s < nfull; s++) {
    const uint32_t bar = rc.full + rc.stage * 8u;
    if (!mbar_wait_poll(bar, rc.phase)) { atomicExch(status, 2); return false; }
    const uint32_t p0 = t0 + rc.stage * rc.stage_bytes, p1 = p0 + d1, p2 = p0 + d2;
    StageLoop<K, EX, MT, 0, SG_GROUPS>::run_all(p0, p1, p2, w, L.a, mc, a_row, acc);
#pragma unroll
    for (int m = 0; m < MT; m++) a_row[m] += SG_KS * SG_A_TILE_BYTES;  // the zero row is a full row too
    __syncwarp();
    mbar_arrive_if(bar + SG_EMPTY_OFF, lane0);
    rc.advance();
  }
  if (rem) {  // a short last stage: the loads beyond it read stale ring bytes that are never used
    const uint32_t bar = rc.full + rc.stage * 8u;
    if (!mbar_wait_poll(bar, rc.phase)) { atomicExch(status, 2); return false; }
    const uint32_t p0 = t0 + rc.stage * rc.stage_bytes, p1 = p0 + d1, p2 = p0 + d2;
    StageLoop<K, EX, MT, 0, SG_GROUPS>::run(p0, p1, p2, w, L.a, mc, a_row, acc, rem);
    __syncwarp();
    mbar_arrive_if(bar + SG_EMPTY_OFF, lane0);
    rc.advance();
  }
  const int q = lane & 3;
#pragma unroll
  for (int m = 0; m < MT; m++) {
    const int r0 = m * 8 + 2 * q;
    if (r0 < d.nrows) {
      float *o = d.out + rowoff[r0] + col;
      o[0] = acc[m][0];
      o[8] = acc[m][2];
    }
    if (r0 + 1 < d.nrows) {
      float *o = d.out + rowoff[r0 + 1] + col;
      o[0] = acc[m][1];
      o[8] = acc[m][3];
    }
  }
  return true;
}

// per-unit dispatch on the unit's live rows: a launch compiled for up to 8 * MT rows runs a unit with fewer rows through the
// narrowest path that holds them (one MMA per 8 rows), since most units of a wide launch are experts that only one or two
// rows selected
template <int K, bool EX, int MT, int SUB>
__device__ __forceinline__ bool consume_rows(const UnitDesc &d, RingCursor &rc, bool live, int lane, const McgConst &mc, uint32_t a_addr,
                                             uint32_t lda_bytes, uint32_t z_addr, const int *rowoff, int col, int *status) {
  if constexpr (SUB < MT) {
    if (d.nrows <= 8 * SUB) return consume_unit<K, EX, SUB>(d, rc, live, lane, mc, a_addr, lda_bytes, z_addr, rowoff, col, status);
    return consume_rows<K, EX, MT, SUB * 2>(d, rc, live, lane, mc, a_addr, lda_bytes, z_addr, rowoff, col, status);
  } else {
    return consume_unit<K, EX, MT>(d, rc, live, lane, mc, a_addr, lda_bytes, z_addr, rowoff, col, status);
  }
}

template <bool EX, int MT>
__device__ __forceinline__ bool consume_any(const UnitDesc &d, RingCursor &rc, bool live, int warp, int lane, const McgConst &mc, uint32_t a_addr,
                                            uint32_t lda_bytes, uint32_t z_addr, const int *rowoff, int col, int *status) {
  const uint32_t ring0 = rc.tile0;  // address of stage 0; the warp's tile offset depends on the unit's K
#define SG_CASE(KK)                                                                                              \
  case KK: {                                                                                                     \
    rc.tile0 = ring0 + (uint32_t)warp * Codec<KK>::TILE_BYTES;                                                   \
    const bool ok = consume_rows<KK, EX, MT, 1>(d, rc, live, lane, mc, a_addr, lda_bytes, z_addr, rowoff, col, status); \
    rc.tile0 = ring0;                                                                                            \
    return ok;                                                                                                   \
  }
  switch (d.K) {
    SG_CASE(4)
    SG_CASE(5)
    SG_CASE(6)
    SG_CASE(7)
    default:
      SG_CASE(8)
  }
#undef SG_CASE
}

template <class P, int MT, bool EX>
__global__ void __launch_bounds__(SG_THREADS, SG_CTAS) stream_gemm_kernel(const __grid_constant__ P prob, const StreamLayout lay, int *status) {
  static_assert(sizeof(UnitDesc) <= SG_DESC_UNIT_BYTES, "unit descriptor too large for its shared-memory slot");
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + SG_MAX_STAGES;
  uint64_t *a_full = empty + SG_MAX_STAGES;
  uint64_t *a_empty = a_full + SG_MAX_ASLOTS;
  unsigned char *desc = smem + 512;  // per A slot: the unit descriptor, then the output row offsets of its rows
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
    // ---------------------------------------------------------------- producer (one warp)
    // Only this warp reads the unit list from global memory; the consumers get each unit's descriptor and output row
    // offsets through shared memory together with the A rows, so no consumer ever waits on a global load. Per ring stage
    // the producer executes one wait, one expect_tx and ONE tensor copy (lane 0); per unit, one unit AHEAD of the tiles it
    // is streaming, the descriptor and one bulk copy per activation row (lane i copies row i).
    //
    // Start-up under programmatic dependent launch: the A rows (and for some problems the unit list itself) are written
    // by the preceding kernel, the compressed weights are not. A problem whose unit list is final when the kernel is
    // launched (P::units_final()) streams the first unit's weight stages into the fresh ring before it waits for
    // the predecessor, so the ring is full when the A rows arrive.
    pdl_launch();  // the successor's CTAs only take resources this grid has released; they wait for its completion themselves
    uint32_t stage = 0, phase = 0;
    int slot = 0;
    uint32_t aphase = 0;
    int u = blockIdx.x;
    typename P::Unit un;
    int nunits = 0, k_pre = 0;
    const uint64_t wpol = l2_evict_first_policy();
    const uint32_t full_a = smem_u32(full), ring_a = smem_u32(ring), nstages = (uint32_t)lay.stages;
    // one stage of unit `t`, k-tiles [k, k + SG_KS): the box is always full size (what lies beyond the unit, the matrix or
    // its last column tile is zero-filled or simply not used), so the byte count depends on K only
    auto issue_stage = [&](const typename P::Unit &t, int k) {
      if (lane == 0) {
        const uint32_t bar = full_a + stage * 8u;
        mbar_arrive_expect_tx_a(bar, (uint32_t)(SG_KS * SG_WARPS * 32) * (uint32_t)t.K);
        tma_load_3d(ring_a + stage * (uint32_t)lay.stage_bytes, prob.tmap(t.map), t.x, t.y + k, t.z, bar, wpol);
      }
      if (++stage == nstages) { stage = 0; phase ^= 1u; }
    };
    // descriptor, output row offsets and A rows of unit `t` into the next A slot
    auto issue_rows = [&](const typename P::Unit &t) -> bool {
      const int i0 = lane < t.nrows ? prob.row_index(t, lane) : 0;
      const int i1 = lane + 32 < t.nrows ? prob.row_index(t, lane + 32) : 0;
      if (!mbar_wait(&a_empty[slot], aphase ^ 1u, status, 3)) return false;
      UnitDesc *du = reinterpret_cast<UnitDesc *>(desc + (size_t)slot * SG_DESC_BYTES);
      int *doff = reinterpret_cast<int *>(desc + (size_t)slot * SG_DESC_BYTES + SG_DESC_UNIT_BYTES);
      doff[lane] = lane < t.nrows ? prob.out_row_off(t, i0) : 0;
      doff[lane + 32] = lane + 32 < t.nrows ? prob.out_row_off(t, i1) : 0;
      const uint32_t rowb = (uint32_t)t.kc * SG_A_TILE_BYTES;
      __syncwarp();
      if (lane == 0) {
        *du = UnitDesc{prob.out_base(t), t.kc, t.ntiles, t.K, t.nrows};
        mbar_arrive_expect_tx(&a_full[slot], (uint32_t)t.nrows * rowb);  // release: descriptor and offsets are visible
      }
      __syncwarp();
      unsigned char *adst = aslot + (size_t)slot * lay.slot_bytes();
      if (lane < t.nrows) bulk_g2s(adst + (size_t)lane * lay.lda * 2, prob.a_row(t, i0), rowb, &a_full[slot]);
      if (lane + 32 < t.nrows) bulk_g2s(adst + (size_t)(lane + 32) * lay.lda * 2, prob.a_row(t, i1), rowb, &a_full[slot]);
      if (++slot == lay.aslots) { slot = 0; aphase ^= 1u; }
      return true;
    };
    if (prob.units_final()) {
      nunits = prob.num_units();
      if (u < nunits) {
        un = prob.unit(u);
        for (; k_pre < un.kc && k_pre < SG_KS * lay.stages; k_pre += SG_KS) issue_stage(un, k_pre);  // fresh ring: no empty-wait needed
      }
      pdl_wait();
    } else {
      pdl_wait();
      nunits = prob.num_units();
      if (u < nunits) un = prob.unit(u);
    }
    if (u < nunits && !issue_rows(un)) return;
    while (u < nunits) {
      const int u_next = u + gridDim.x;
      typename P::Unit nx;
      if (u_next < nunits) {  // the next unit's rows go out before this unit's remaining tiles: they arrive stages early
        nx = prob.unit(u_next);
        if (!issue_rows(nx)) return;
      }
      for (int k = k_pre; k < un.kc; k += SG_KS) {
#ifdef SG_PRODUCER_SLEEP_NS
        if (!mbar_wait_sleep(&empty[stage], phase ^ 1u, status, 1, SG_PRODUCER_SLEEP_NS)) return;
#else
        if (!mbar_wait(&empty[stage], phase ^ 1u, status, 1)) return;
#endif
        issue_stage(un, k);
      }
      k_pre = 0;
      un = nx;
      u = u_next;
    }
    return;
  }

  // ------------------------------------------------------------------ consumers (8 warps)
  RingCursor rc;
  rc.full = smem_u32(full); rc.tile0 = smem_u32(ring);
  rc.stage_bytes = (uint32_t)lay.stage_bytes; rc.nstages = (uint32_t)lay.stages; rc.stage = 0u; rc.phase = 0u;
  int slot = 0;
  uint32_t aphase = 0;
  const uint32_t a0_addr = smem_u32(aslot), z_addr = smem_u32(zrow), slot_bytes = (uint32_t)lay.slot_bytes(), lda_bytes = (uint32_t)lay.lda * 2u;
  const uint32_t afull_a = smem_u32(a_full), aempty_a = smem_u32(a_empty);
  const McgConst mc = McgConst::load();
  const int col = warp * 16 + (lane >> 2);

  if (!prob.units_final()) pdl_wait();  // the unit count is the predecessor's output
  const int nunits = prob.num_units();
  for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
    if (!mbar_wait_a(afull_a + (uint32_t)slot * 8u, aphase, status, 4)) return;
    const UnitDesc d = *reinterpret_cast<const UnitDesc *>(desc + (size_t)slot * SG_DESC_BYTES);
    const int *rowoff = reinterpret_cast<const int *>(desc + (size_t)slot * SG_DESC_BYTES + SG_DESC_UNIT_BYTES);
    if (!consume_any<EX, MT>(d, rc, warp < d.ntiles, warp, lane, mc, a0_addr + (uint32_t)slot * slot_bytes, lda_bytes, z_addr, rowoff, col, status))
      return;
    // the stores above read the slot's row offsets: only now may it be refilled
    __syncwarp();
    if (lane == 0) mbar_arrive_a(aempty_a + (uint32_t)slot * 8u);
    if (++slot == lay.aslots) { slot = 0; aphase ^= 1u; }
  }
}

}  // namespace ijah
