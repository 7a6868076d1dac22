// Prefill MoE kernels. See pf_moe.cuh.
#include <algorithm>

#include "common.hpp"
#include "exl3_decode.cuh"
#include "pf_moe.cuh"
#include "umma.cuh"

namespace ijah {

// =============================================================================================== grouped trellis GEMM
// out[pos][col] = sum_k act[pos][k] * W'_e[k][col] for one work item = (expert, <= 128 sorted rows, 256 output columns).
//
// The contraction runs on the 5th-generation tensor core as D^T = W'^T * act^T: M = 128 output columns per accumulator
// (two accumulators per item), N = the item's rows (16..128), K = 16 per instruction, accumulators in TMEM
// (2 buffers x 2 x 128 columns = all 512, so the epilogue of one item overlaps the MMAs of the next).
// One CTA per SM, warp-specialised:
//   warp 0        producer: bulk-copies compressed tiles (4 k-tiles x 16 column tiles per stage) and the activations
//                 (blocked layout, 1 KB per 8-row group per stage) into shared memory
//   warp 1        issues tcgen05.mma (one thread) when a stage's decoded weights and activations are both present
//   warps 2-5     epilogue: tcgen05.ld the accumulators, store the live rows
//   warps 6-21    decoders: each owns one of the 16 column tiles, decodes its tile of every k-tile with the same
//                 register decode as the decode-width kernels and writes fp16 into the MMA's shared-memory layout
// so every expert tile is decoded once per 128 rows instead of once per 16/32-row window.
constexpr int PG_KS = 4;                      // k-tiles per stage
constexpr int PG_RING = 4;                    // compressed-tile stages
constexpr int PG_AB = 3;                      // decoded-weight / activation stages
constexpr int PG_THREADS = 32 * 22;
constexpr int PG_A_STAGE = PG_KS * 2 * 4096;  // [ks][ng][khalf][16 groups][128 B]
constexpr int PG_B_STAGE = 16 * 1024;         // [row group][8 k-chunks][128 B]

struct PgGemm {
  const PfItem *items;
  const int *nitems;
  const char *w_routed[2], *w_shared[2];  // trellis bases per projection
  const __half *act[2];                   // blocked activations per projection
  float *out[2];                          // output base per projection; element (pos, col) at out + pos * ldo + col
  int ldo, in, IT, OT, Kx, Ks;
};

struct PgSmem {
  uint64_t ring_full[PG_RING], ring_empty[PG_RING];
  uint64_t a_full[PG_AB], b_full[PG_AB], ab_empty[PG_AB];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};

template <int K>
__device__ __forceinline__ void pg_decode_stage(const unsigned char *ring_stage, unsigned char *a_stage, int dw, int lane) {
  const typename Codec<K>::Lane L = Codec<K>::lane(lane);
  const McgConst mc = McgConst::load();
  const int ng = dw >> 3, t = dw & 7, q = lane & 3, c = lane >> 2;
#pragma unroll
  for (int ks = 0; ks < PG_KS; ks++) {
    const unsigned char *tile = ring_stage + (size_t)(ks * 16 + dw) * Codec<K>::TILE_BYTES;
    uint32_t b[4];
    dec8<K>(*reinterpret_cast<const uint32_t *>(tile + L.o0), *reinterpret_cast<const uint32_t *>(tile + L.o1),
            *reinterpret_cast<const uint32_t *>(tile + L.o2), L.a, mc, b);
    // lane (q, c): b[0] = k (2q, 2q+1) of column c, b[1] = k (2q+8, 2q+9) of column c, b[2], b[3] the same of column c + 8
    unsigned char *dst = a_stage + (size_t)(ks * 2 + ng) * 4096 + (2 * t) * 128 + c * 16 + q * 4;
    *reinterpret_cast<uint32_t *>(dst) = b[0];
    *reinterpret_cast<uint32_t *>(dst + 2048) = b[1];
    *reinterpret_cast<uint32_t *>(dst + 128) = b[2];
    *reinterpret_cast<uint32_t *>(dst + 128 + 2048) = b[3];
  }
}

__global__ void __launch_bounds__(PG_THREADS, 1) pf_gemm_kernel(const PgGemm g, int *status) {
  extern __shared__ __align__(1024) unsigned char pf_smem[];
  unsigned char *smem = pf_smem;
  PgSmem *sm = reinterpret_cast<PgSmem *>(smem);
  const int kmax = max(g.Kx, g.Ks);
  const int ring_stage_bytes = PG_KS * 16 * 32 * kmax;
  unsigned char *ring = smem + 1024;
  unsigned char *abuf = ring + (size_t)PG_RING * ring_stage_bytes;  // ring_stage_bytes is a multiple of 2048
  unsigned char *bbuf = abuf + (size_t)PG_AB * PG_A_STAGE;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PG_RING; s++) { mbar_init(&sm->ring_full[s], 1); mbar_init(&sm->ring_empty[s], 16); }
    for (int s = 0; s < PG_AB; s++) { mbar_init(&sm->a_full[s], 16); mbar_init(&sm->b_full[s], 1); mbar_init(&sm->ab_empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&sm->acc_full[b], 1); mbar_init(&sm->acc_empty[b], 4); }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&sm->tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm->tmem_base;
  const int nitems = *g.nitems;
  const int nst = g.IT / PG_KS;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------ producer
    int rs = 0, as = 0;
    uint32_t rph = 0, aph = 0;
    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
      const PfItem im = g.items[it];
      const int K = im.expert < 0 ? g.Ks : g.Kx;
      const char *w = (im.expert < 0 ? g.w_shared[im.proj] : g.w_routed[im.proj] + (size_t)im.expert * g.IT * g.OT * 32 * K) +
                      (size_t)im.ngpair * 16 * 32 * K;
      const uint32_t kb = 16u * 32u * (uint32_t)K, kstride = (uint32_t)g.OT * 32u * (uint32_t)K;
      const int ngroups = (im.nrows + 7) >> 3;
      const __half *act = g.act[im.proj] + (size_t)(im.row0 >> 3) * (g.in >> 3) * 64;
      for (int st = 0; st < nst; st++) {
        if (!mbar_wait(&sm->ring_empty[rs], rph ^ 1u, status, 11)) return;
        if (lane == 0) mbar_arrive_expect_tx(&sm->ring_full[rs], PG_KS * kb);
        __syncwarp();
        if (lane < PG_KS)
          bulk_g2s(ring + (size_t)rs * ring_stage_bytes + lane * kb, w + (size_t)(st * PG_KS + lane) * kstride, kb, &sm->ring_full[rs]);
        if (++rs == PG_RING) { rs = 0; rph ^= 1u; }
        if (!mbar_wait(&sm->ab_empty[as], aph ^ 1u, status, 12)) return;
        if (lane == 0) mbar_arrive_expect_tx(&sm->b_full[as], (uint32_t)ngroups * 1024u);
        __syncwarp();
        if (lane < ngroups)
          bulk_g2s(bbuf + (size_t)as * PG_B_STAGE + lane * 1024, act + ((size_t)lane * (g.in >> 3) + st * 8) * 64, 1024, &sm->b_full[as]);
        if (++as == PG_AB) { as = 0; aph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    int as = 0, buf = 0;
    uint32_t aph = 0, cph[2] = {0, 0};
    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
      const PfItem im = g.items[it];
      const uint32_t idesc = umma_idesc_f16(128, (im.nrows + 15) & ~15);
      if (!mbar_wait(&sm->acc_empty[buf], cph[buf] ^ 1u, status, 13)) break;
      tc_fence_after_sync();
      for (int st = 0; st < nst; st++) {
        if (!mbar_wait(&sm->a_full[as], aph, status, 14)) goto done;
        if (!mbar_wait(&sm->b_full[as], aph, status, 15)) goto done;
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a0 = smem_u32(abuf + (size_t)as * PG_A_STAGE), b0 = smem_u32(bbuf + (size_t)as * PG_B_STAGE);
#pragma unroll
          for (int ks = 0; ks < PG_KS; ks++) {
            const uint64_t bd = umma_smem_desc(b0 + ks * 256, 128, 1024);
#pragma unroll
            for (int ng = 0; ng < 2; ng++)
              umma_f16_ss(tmem + (uint32_t)(buf * 2 + ng) * 128u, umma_smem_desc(a0 + (ks * 2 + ng) * 4096, 2048, 128), bd, idesc,
                          (st > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(&sm->ab_empty[as]);  // the stage may be overwritten once these MMAs have read it
          if (st == nst - 1) umma_commit(&sm->acc_full[buf]);
        }
        __syncwarp();
        if (++as == PG_AB) { as = 0; aph ^= 1u; }
      }
      cph[buf] ^= 1u;
      buf ^= 1;
    }
  done:;
  } else if (warp < 6) {
    // ------------------------------------------------------------------------------------------ epilogue
    const int qd = warp & 3;  // TMEM lanes 32 qd .. 32 qd + 31 are this warp's
    int buf = 0;
    uint32_t cph[2] = {0, 0};
    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
      const PfItem im = g.items[it];
      if (!mbar_wait(&sm->acc_full[buf], cph[buf], status, 16)) break;
      tc_fence_after_sync();
      float *out = g.out[im.proj] + (size_t)im.row0 * g.ldo + im.ngpair * PF_NCOL + qd * 32 + lane;
      for (int ng = 0; ng < 2; ng++)
        for (int c0 = 0; c0 < im.nrows; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)(buf * 2 + ng) * 128u + (uint32_t)c0, r);
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (c0 + j < im.nrows) out[(size_t)(c0 + j) * g.ldo + ng * 128] = __uint_as_float(r[j]);
        }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->acc_empty[buf]);
      cph[buf] ^= 1u;
      buf ^= 1;
    }
  } else {
    // ------------------------------------------------------------------------------------------ decoders
    const int dw = warp - 6;
    int rs = 0, as = 0;
    uint32_t rph = 0, aph = 0;
    for (int it = blockIdx.x; it < nitems; it += gridDim.x) {
      const PfItem im = g.items[it];
      const int K = im.expert < 0 ? g.Ks : g.Kx;
      for (int st = 0; st < nst; st++) {
        if (!mbar_wait(&sm->ring_full[rs], rph, status, 17)) goto out;
        if (!mbar_wait(&sm->ab_empty[as], aph ^ 1u, status, 18)) goto out;
        const unsigned char *rsrc = ring + (size_t)rs * ring_stage_bytes;
        unsigned char *adst = abuf + (size_t)as * PG_A_STAGE;
        switch (K) {
          case 4: pg_decode_stage<4>(rsrc, adst, dw, lane); break;
          case 5: pg_decode_stage<5>(rsrc, adst, dw, lane); break;
          case 6: pg_decode_stage<6>(rsrc, adst, dw, lane); break;
          case 7: pg_decode_stage<7>(rsrc, adst, dw, lane); break;
          default: pg_decode_stage<8>(rsrc, adst, dw, lane); break;
        }
        fence_proxy_async_smem();  // the tensor core reads what these ordinary stores wrote
        __syncwarp();
        if (lane == 0) { mbar_arrive(&sm->a_full[as]); mbar_arrive(&sm->ring_empty[rs]); }
        if (++rs == PG_RING) { rs = 0; rph ^= 1u; }
        if (++as == PG_AB) { as = 0; aph ^= 1u; }
      }
    }
  out:;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

static size_t pg_smem_bytes(int kmax) { return 1024 + (size_t)PG_RING * PG_KS * 16 * 32 * kmax + (size_t)PG_AB * (PG_A_STAGE + PG_B_STAGE); }

static void launch_pf_gemm(const PgGemm &g, int *status, cudaStream_t st) {
  IJ_CHECK(g.IT % PG_KS == 0 && g.OT % 16 == 0 && g.in % 64 == 0, "prefill GEMM needs in %% 64 == 0 and out %% 256 == 0 (in %d, out %d)", g.in, g.OT * 16);
  const size_t smem = pg_smem_bytes(std::max(g.Kx, g.Ks));
  IJ_CUDA(cudaFuncSetAttribute(pf_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));  // per device: every launch
  pf_gemm_kernel<<<sm_count(), PG_THREADS, smem, st>>>(g, status);
  IJ_CUDA(cudaGetLastError());
}

// (the routing, sorting, operand and finishing kernels follow)

// =============================================================================================== router
// logits[n][0 .. E) = x . W^T (bf16 W, f32 x) on tensor cores without giving up f32 accuracy: x is split into three bf16
// terms (x = hi + mid + lo to 2^-24), each multiplied with the bf16 weights by mma.sync.m16n8k16 (products exact, f32
// accumulate). 128 tokens x 128 experts per CTA, 8 warps of 32 x 64, k in steps of 32 through double-buffered shared
// memory (rows padded to 80 bytes: conflict-free ldmatrix). Reference: the router GEMM of the chunked prefill
// (kernels/prefill/pf_gemm.metal:159-186). The shared expert's gate logit (column E) is a plain dot product in
// pf_route_kernel.
constexpr int LG_T = 128, LG_K = 32, LG_LD = LG_K + 8;              // halfs per staged row
constexpr int LG_PLANE = LG_T * LG_LD, LG_BUF = 4 * LG_PLANE;       // x hi, mid, lo, W
constexpr int LG_SMEM = 2 * LG_BUF * 2;                             // bytes

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t bf16_rn_bits(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
}
// (a, b) -> packed bf16 pairs of the three terms
__device__ __forceinline__ void split3(float a, float b, uint32_t &hi, uint32_t &mid, uint32_t &lo) {
  const uint32_t ah = bf16_rn_bits(a), bh = bf16_rn_bits(b);
  const float a1 = a - __uint_as_float(ah << 16), b1 = b - __uint_as_float(bh << 16);
  const uint32_t am = bf16_rn_bits(a1), bm = bf16_rn_bits(b1);
  const float a2 = a1 - __uint_as_float(am << 16), b2 = b1 - __uint_as_float(bm << 16);
  hi = ah | (bh << 16);
  mid = am | (bm << 16);
  lo = bf16_rn_bits(a2) | (bf16_rn_bits(b2) << 16);
}

__global__ void __launch_bounds__(256) pf_logits_kernel(const PfParams p) {
  extern __shared__ __align__(16) unsigned char lg_smem[];
  uint16_t *sm = reinterpret_cast<uint16_t *>(lg_smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, t0 = blockIdx.x * LG_T, c0 = blockIdx.y * LG_T, H = p.H;
  const int wm = warp >> 1, wn = warp & 1;  // warp tile: tokens 32 wm .. +31, experts 64 wn .. +63
  // loads. x: thread -> rows (tid >> 3) + 32 j, floats 4 (tid & 7) .. +3; W: rows (tid >> 2) + 64 j, 16-byte chunk tid & 3
  const int xr = tid >> 3, xc = (tid & 7) * 4, wr = tid >> 2, wc = (tid & 3) * 8;
  const float *xsrc[4];
  const uint16_t *wsrc[2];
#pragma unroll
  for (int j = 0; j < 4; j++) xsrc[j] = p.x + (size_t)min(t0 + xr + 32 * j, p.n - 1) * H + xc;
#pragma unroll
  for (int j = 0; j < 2; j++) wsrc[j] = p.router + (size_t)min(c0 + wr + 64 * j, p.E - 1) * H + wc;
  float4 xv[4];
  auto load_x = [&](int ks) {
#pragma unroll
    for (int j = 0; j < 4; j++) xv[j] = *reinterpret_cast<const float4 *>(xsrc[j] + ks * LG_K);
  };
  auto load_w = [&](int ks, int buf) {
    const uint32_t dst = smem_u32(sm + buf * LG_BUF + 3 * LG_PLANE);
#pragma unroll
    for (int j = 0; j < 2; j++)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)(((wr + 64 * j) * LG_LD + wc) * 2)), "l"(wsrc[j] + ks * LG_K) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto stash_x = [&](int buf) {
    uint16_t *b = sm + buf * LG_BUF;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      uint32_t h0, m0, l0, h1, m1, l1;
      split3(xv[j].x, xv[j].y, h0, m0, l0);
      split3(xv[j].z, xv[j].w, h1, m1, l1);
      const int o = (xr + 32 * j) * LG_LD + xc;
      *reinterpret_cast<uint2 *>(b + o) = make_uint2(h0, h1);
      *reinterpret_cast<uint2 *>(b + LG_PLANE + o) = make_uint2(m0, m1);
      *reinterpret_cast<uint2 *>(b + 2 * LG_PLANE + o) = make_uint2(l0, l1);
    }
  };
  float acc[2][8][4];
#pragma unroll
  for (int i = 0; i < 2; i++)
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
      for (int q = 0; q < 4; q++) acc[i][j][q] = 0.0f;
  load_x(0);
  load_w(0, 0);
  stash_x(0);
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  // ldmatrix lane offsets (in halfs): A rows (lane & 15), k half (lane >> 4); B rows (lane & 7) + 8 ((lane >> 4) & 1), k half (lane >> 3) & 1
  const int a_off = (32 * wm + (lane & 15)) * LG_LD + (lane >> 4) * 8;
  const int b_off = (64 * wn + (lane & 7) + ((lane >> 4) & 1) * 8) * LG_LD + ((lane >> 3) & 1) * 8;
  const int nk = H / LG_K;
  for (int ks = 0; ks < nk; ks++) {
    const int buf = ks & 1;
    if (ks + 1 < nk) {
      load_x(ks + 1);
      load_w(ks + 1, buf ^ 1);  // that buffer was last read one step ago, before the barrier below
    }
    const uint32_t base = smem_u32(sm + buf * LG_BUF);
#pragma unroll
    for (int kk = 0; kk < LG_K; kk += 16) {
      uint32_t bfr[4][4];  // per pair of expert tiles: b0, b1 of tile 2 j, b0, b1 of tile 2 j + 1
#pragma unroll
      for (int j = 0; j < 4; j++) ldmatrix_x4(bfr[j], base + (uint32_t)((3 * LG_PLANE + b_off + j * 16 * LG_LD + kk) * 2));
#pragma unroll
      for (int t = 0; t < 3; t++) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
          uint32_t afr[4];
          ldmatrix_x4(afr, base + (uint32_t)((t * LG_PLANE + a_off + i * 16 * LG_LD + kk) * 2));
#pragma unroll
          for (int j = 0; j < 4; j++) {
            mma_bf16_16816(acc[i][2 * j], afr, bfr[j][0], bfr[j][1]);
            mma_bf16_16816(acc[i][2 * j + 1], afr, bfr[j][2], bfr[j][3]);
          }
        }
      }
    }
    if (ks + 1 < nk) {
      stash_x(buf ^ 1);
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
  }
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int i = 0; i < 2; i++)
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
      const int t = t0 + 32 * wm + 16 * i + g + 8 * hh;
      if (t >= p.n) continue;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int c = c0 + 64 * wn + 8 * j + 2 * q;
        float *dst = p.logits + (size_t)t * (p.E + 1) + c;
        if (c < p.E) dst[0] = acc[i][j][2 * hh];
        if (c + 1 < p.E) dst[1] = acc[i][j][2 * hh + 1];
      }
    }
}

// top-k on the logits (ties -> lowest index), weights = softmax over the k selected; one warp per token
__global__ void __launch_bounds__(256) pf_route_kernel(const PfParams p) {
  __shared__ float sl[8][1024];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x * 8 + warp;
  if (t >= p.n) return;
  float *s = sl[warp];
  const int E = p.E, k = p.topk;
  for (int i = lane; i < E; i += 32) s[i] = p.logits[(size_t)t * (E + 1) + i];
  if (p.has_shared) {  // the shared expert's gate logit: x[t] . w_sg
    float g = 0.0f;
    for (int i = lane * 8; i < p.H; i += 256) {
      const float4 a = *reinterpret_cast<const float4 *>(p.x + (size_t)t * p.H + i), b = *reinterpret_cast<const float4 *>(p.x + (size_t)t * p.H + i + 4);
      const uint4 u = *reinterpret_cast<const uint4 *>(p.sgate + i);
      g += a.x * __uint_as_float(u.x << 16) + a.y * __uint_as_float(u.x & 0xFFFF0000u) + a.z * __uint_as_float(u.y << 16) +
           a.w * __uint_as_float(u.y & 0xFFFF0000u) + b.x * __uint_as_float(u.z << 16) + b.y * __uint_as_float(u.z & 0xFFFF0000u) +
           b.z * __uint_as_float(u.w << 16) + b.w * __uint_as_float(u.w & 0xFFFF0000u);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) g += __shfl_xor_sync(0xFFFFFFFFu, g, o);
    if (lane == 0) p.logits[(size_t)t * (E + 1) + E] = g;
  }
  __syncwarp();
  float myv = 0.0f, top = 0.0f;
  int myi = 0;
  for (int r = 0; r < k; r++) {
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
    if (r == 0) top = best;
    if (lane == r) { myv = best; myi = bi; }
    if ((bi & 31) == lane) s[bi] = -INFINITY;
    __syncwarp();
  }
  float pr = lane < k ? expf(myv - top) : 0.0f, sum = pr;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  if (lane < k) {
    p.route[(size_t)t * 2 * k + lane] = (uint32_t)myi;
    p.route[(size_t)t * 2 * k + k + lane] = __float_as_uint(pr / sum);
  }
}

// =============================================================================================== sort by expert
// Deterministic counting sort of the n * topk slots by expert (reference kernels/prefill/pf_moe.metal:29-83), three passes:
//   pf_hist_kernel   one warp per block of PS_BLOCK consecutive slots: per-expert counts of the block
//   pf_scan_kernel   per expert, exclusive scan of the counts over the blocks (a warp per expert); then one CTA lays out
//                    the experts' position ranges (padded to 8 rows, the granule of the blocked operand layout) and
//                    writes the work items
//   pf_place_kernel  the same warps walk their block in slot order: rank of a slot among its expert's slots = the block's
//                    base + earlier equals in the block (warp match), position = expert offset + rank
constexpr int PS_BLOCK = 256;
__global__ void __launch_bounds__(32) pf_hist_kernel(const PfParams p, int *hist) {
  __shared__ int cnt[1024];
  const int b = blockIdx.x, lane = threadIdx.x, k = p.topk;
  for (int e = lane; e < p.E; e += 32) cnt[e] = 0;
  __syncwarp();
  for (int i = lane; i < PS_BLOCK; i += 32) {
    const int s = b * PS_BLOCK + i;
    if (s < p.S) {
      const int e = (int)p.route[(size_t)(s / k) * 2 * k + s % k];
      if (e >= p.e0 && e < p.e0 + p.ecount) atomicAdd(&cnt[e], 1);  // slots of experts held elsewhere are not placed
    }
  }
  __syncwarp();
  for (int e = lane; e < p.E; e += 32) hist[(size_t)b * p.E + e] = cnt[e];
}

// hist[b][e] -> exclusive scan over b (in place), cnt[e] = total; one warp per expert
__global__ void __launch_bounds__(256) pf_blockscan_kernel(const PfParams p, int *hist, int nb) {
  const int e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= p.E) return;
  int run = 0;
  for (int b0 = 0; b0 < nb; b0 += 32) {
    const int b = b0 + lane, v = b < nb ? hist[(size_t)b * p.E + e] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += a;
    }
    if (b < nb) hist[(size_t)b * p.E + e] = run + inc - v;
    run += __shfl_sync(0xFFFFFFFFu, inc, 31);
  }
  if (lane == 0) p.cnt[e] = run;
}

__device__ __forceinline__ int block_excl_scan(int v, int *warp_tot, int *total) {  // blockDim = 1024, all threads call
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int s = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xFFFFFFFFu, s, o);
    if (lane >= o) s += a;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = s;
  __syncthreads();
  if (warp == 0) {
    int t = warp_tot[lane], ts = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xFFFFFFFFu, ts, o);
      if (lane >= o) ts += a;
    }
    warp_tot[lane] = ts - t;
    if (lane == 31) *total = ts;
  }
  __syncthreads();
  return warp_tot[warp] + s - v;
}

__global__ void __launch_bounds__(1024) pf_scan_kernel(const PfParams p) {
  __shared__ int wt[32], tot8, totp;
  __shared__ int s_pb[1024], s_off[1024], s_cnt[1024];
  const int e = threadIdx.x, E = p.E;
  const int c = e < E ? p.cnt[e] : 0, c8 = (c + 7) & ~7, np = (c + PF_NTOK - 1) / PF_NTOK;
  const int o = block_excl_scan(c8, wt, &tot8);
  const int pb = block_excl_scan(np, wt, &totp);
  if (e < E) p.off[e] = o;
  s_pb[e] = e < E ? pb : 0x7FFFFFFF;
  s_off[e] = o;
  s_cnt[e] = c;
  const int nsh = p.has_shared ? p.sh_rows : 0, shp = (nsh + PF_NTOK - 1) / PF_NTOK;
  if (e == 0) {
    p.off[E] = tot8;
    p.off[E + 1] = tot8 + ((nsh + 7) & ~7);
    p.nitems[0] = (totp + shp) * 2 * (p.I / PF_NCOL);
    p.nitems[1] = (totp + shp) * (p.H / PF_NCOL);
  }
  __syncthreads();
  const int GU = p.I / PF_NCOL, DN = p.H / PF_NCOL;
  auto emit = [&](int pass, int expert, int row0, int nrows) {
    for (int j = 0; j < 2 * GU; j++) p.items_gu[pass * 2 * GU + j] = PfItem{expert, j / GU, j % GU, row0, nrows, {0, 0, 0}};
    for (int j = 0; j < DN; j++) p.items_d[pass * DN + j] = PfItem{expert, 0, j, row0, nrows, {0, 0, 0}};
  };
  // one thread per pass: the expert of pass q is the last one whose first pass is <= q (experts without rows share the
  // first-pass index of the next expert that has some)
  for (int q = threadIdx.x; q < totp; q += blockDim.x) {
    int lo = 0, hi = 1024;  // first index with s_pb > q
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s_pb[mid] <= q) lo = mid + 1; else hi = mid;
    }
    const int ex = lo - 1, j = q - s_pb[ex];
    emit(q, ex - p.e0, s_off[ex] + j * PF_NTOK, min(PF_NTOK, s_cnt[ex] - j * PF_NTOK));  // expert index into the local stacks
  }
  for (int j = threadIdx.x; j < shp; j += blockDim.x) emit(totp + j, -1, tot8 + j * PF_NTOK, min(PF_NTOK, nsh - j * PF_NTOK));
}

// order[pos] = slot (S + t for the shared expert's row of token t, -1 = padding), inv[slot] = pos, seid[pos] = expert
// (E = shared). order / seid are pre-set to -1 by the launcher. Blocks 0 .. nb-1 place the routed slots, the rest the shared rows.
__global__ void __launch_bounds__(32) pf_place_kernel(const PfParams p, int *order, const int *hist, int nb) {
  __shared__ int base[1024];
  const int b = blockIdx.x, lane = threadIdx.x, k = p.topk;
  if (b >= nb) {
    if (!p.has_shared) return;
    for (int j = (b - nb) * PS_BLOCK + lane; j < min(p.sh_rows, (b - nb + 1) * PS_BLOCK); j += 32) {
      const int pos = p.off[p.E] + j;
      order[pos] = p.S + p.sh_row0 + j;
      p.seid[pos] = p.E;
    }
    return;
  }
  for (int e = lane; e < p.E; e += 32) base[e] = hist[(size_t)b * p.E + e] + p.off[e];
  __syncwarp();
  const uint32_t lt = (1u << lane) - 1u;
  for (int i = lane; i < PS_BLOCK; i += 32) {  // 32 consecutive slots per round, rounds in slot order
    const int s = b * PS_BLOCK + i;
    const int er = s < p.S ? (int)p.route[(size_t)(s / k) * 2 * k + s % k] : -1;
    const bool on = er >= p.e0 && er < p.e0 + p.ecount;
    if (s < p.S && !on) p.inv[s] = -1;
    const int e = on ? er : -1 - lane;
    const uint32_t same = __match_any_sync(0xFFFFFFFFu, e);
    if (on) {
      const int pos = base[e] + __popc(same & lt);
      order[pos] = s;
      p.inv[s] = pos;
      p.seid[pos] = e;
    }
    __syncwarp();
    if (on && (same & lt) == 0) base[e] += __popc(same);  // the first lane of each expert advances its base
    __syncwarp();
  }
}

// The three elementwise kernels below give one warp a whole operand row (one position, or one slot of one token): the
// row's metadata is fetched once, the loads of several 128-element chunks are in flight together, and a lane owns 4
// consecutive elements of a chunk, i.e. 8 bytes of fp16 output: half a row of a core matrix of the blocked layout.
// All three are bound by instruction issue (the fp32 Hadamard butterflies and their shuffles), not by memory.
constexpr float PF_HS = 0.08838834764831845f;  // 1 / sqrt(128)

__device__ __forceinline__ float4 mul4(float4 a, uint2 h) {  // a * (4 halfs)
  const __half2 h0 = *reinterpret_cast<const __half2 *>(&h.x), h1 = *reinterpret_cast<const __half2 *>(&h.y);
  const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
  return make_float4(a.x * f0.x, a.y * f0.y, a.z * f1.x, a.w * f1.y);
}
__device__ __forceinline__ uint2 pack4(const float (&v)[4]) {
  const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  return make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
}
// lane's 4 elements (k = chunk * 128 + 4 lane ..) of position pos in a blocked operand with `in` columns
__device__ __forceinline__ __half *blocked_lane_ptr(__half *base, int pos, int chunk, int lane, int in) {
  return base + (((size_t)(pos >> 3) * (in >> 3) + chunk * 16 + (lane >> 1)) << 6) + ((pos & 7) << 3) + ((lane & 1) << 2);
}

// gate / up operands: xh[pos] = fp16(H128(x[token(pos)] * suh[expert(pos)])), one warp per position, eight positions (one
// row group of the blocked layout) per CTA (reference kernels/prefill/pf_moe.metal:88-104); padding positions are written
// as zeros. In the blocked layout the eight rows of a group and one 128-input chunk form 2 KB of contiguous memory (16
// core matrices of 8 rows x 16 bytes), of which a warp (one row) owns every eighth 16 bytes: the CTA therefore collects
// four chunks of both operands in shared memory (16-byte slots XOR-swizzled by core matrix: conflict-free both ways)
// and writes them out as whole 512-byte runs per warp instead of 16-byte pieces.
__global__ void __launch_bounds__(256) pf_prep_kernel(const PfParams p, const int *order) {
  __shared__ __align__(16) unsigned char tile[2][4][2048];  // [gate | up][chunk of the pass][core matrix 16][row 8][16 bytes]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = blockIdx.x * 8 + warp, H = p.H;  // pos_cap is a multiple of 8
  const int slot = pos < p.off[p.E + 1] ? order[pos] : -1;
  const bool shared = slot >= p.S;
  const int t = slot < 0 ? 0 : shared ? slot - p.S : slot / p.topk;
  const int e = (slot < 0 || shared) ? 0 : p.seid[pos] - p.e0;
  const __half *sg = shared ? p.sgt.suh : p.gate.suh + (size_t)e * H, *su = shared ? p.sup.suh : p.up.suh + (size_t)e * H;
  const float *xr = p.x + (size_t)t * H;
  const int j = lane >> 1, hsel = lane & 1;
  const uint32_t woff = (uint32_t)(j * 128 + ((warp ^ (j & 7)) * 16) + hsel * 8);  // this lane's 8 bytes of its row's share of a chunk
  for (int c0 = 0; c0 < H / 128; c0 += 4) {
    float4 xv[4];
    uint2 gs[4], us[4];
    if (slot >= 0) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int o = (min(c0 + i, H / 128 - 1)) * 128 + 4 * lane;
        xv[i] = *reinterpret_cast<const float4 *>(xr + o);
        gs[i] = *reinterpret_cast<const uint2 *>(sg + o);
        us[i] = *reinterpret_cast<const uint2 *>(su + o);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint2 go = make_uint2(0u, 0u), uo = make_uint2(0u, 0u);
      if (slot >= 0 && c0 + i < H / 128) {  // uniform over the warp
        const float4 g4 = mul4(xv[i], gs[i]), u4 = mul4(xv[i], us[i]);
        float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
        fwht128_contig(g, lane, PF_HS);
        fwht128_contig(u, lane, PF_HS);
        go = pack4(g);
        uo = pack4(u);
      }
      *reinterpret_cast<uint2 *>(&tile[0][i][woff]) = go;
      *reinterpret_cast<uint2 *>(&tile[1][i][woff]) = uo;
    }
    __syncthreads();
    // 8 blocks of 2 KB (operand, chunk) = 1024 pieces of 16 bytes, four per thread; consecutive threads, consecutive bytes
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int idx = threadIdx.x + 256 * k, blk = idx >> 7, jj = (idx >> 3) & 15, r = idx & 7, op = blk >> 2, ci = blk & 3;
      if (c0 + ci < H / 128) {
        const uint4 v = *reinterpret_cast<const uint4 *>(&tile[op][ci][jj * 128 + ((r ^ (jj & 7)) * 16)]);
        __half *dst = (op ? p.xh_u : p.xh_g) + (((size_t)blockIdx.x * (H >> 3) + (c0 + ci) * 16 + jj) << 6) + (r << 3);
        *reinterpret_cast<uint4 *>(dst) = v;
      }
    }
    __syncthreads();
  }
}

// down operand: SwiGLU of the finished gate / up, times suh_down, H128, fp16 (reference pf_moe.metal:107-125)
__global__ void __launch_bounds__(256) pf_mid_kernel(const PfParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = blockIdx.x * 8 + warp, I = p.I;
  if (pos >= p.pos_cap) return;
  const int e = pos < p.off[p.E + 1] ? p.seid[pos] : -1;
  if (e < 0) {
    for (int c = 0; c < I / 128; c++) *reinterpret_cast<uint2 *>(blocked_lane_ptr(p.xh_d, pos, c, lane, I)) = make_uint2(0u, 0u);
    return;
  }
  const bool shared = e == p.E;
  const int el = shared ? 0 : e - p.e0;
  const __half *svg = shared ? p.sgt.svh : p.gate.svh + (size_t)el * I, *svu = shared ? p.sup.svh : p.up.svh + (size_t)el * I;
  const __half *sud = shared ? p.sdn.suh : p.down.suh + (size_t)el * I;
  const float *raw = p.raw_gu + (size_t)pos * 2 * I;
  for (int c0 = 0; c0 < I / 128; c0 += 2) {
    float4 gr[2], ur[2];
    uint2 s_g[2], s_u[2], s_d[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int o = (min(c0 + i, I / 128 - 1)) * 128 + 4 * lane;
      gr[i] = *reinterpret_cast<const float4 *>(raw + o);
      ur[i] = *reinterpret_cast<const float4 *>(raw + I + o);
      s_g[i] = *reinterpret_cast<const uint2 *>(svg + o);
      s_u[i] = *reinterpret_cast<const uint2 *>(svu + o);
      s_d[i] = *reinterpret_cast<const uint2 *>(sud + o);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
      if (c0 + i < I / 128) {
        float gv[4] = {gr[i].x, gr[i].y, gr[i].z, gr[i].w}, uv[4] = {ur[i].x, ur[i].y, ur[i].z, ur[i].w}, hh[4];
        fwht128_contig(gv, lane, PF_HS);
        fwht128_contig(uv, lane, PF_HS);
        const float4 g4 = mul4(make_float4(gv[0], gv[1], gv[2], gv[3]), s_g[i]), u4 = mul4(make_float4(uv[0], uv[1], uv[2], uv[3]), s_u[i]);
        const float4 d4 = mul4(make_float4(1.0f, 1.0f, 1.0f, 1.0f), s_d[i]);
        hh[0] = g4.x / (1.0f + expf(-g4.x)) * u4.x * d4.x;
        hh[1] = g4.y / (1.0f + expf(-g4.y)) * u4.y * d4.y;
        hh[2] = g4.z / (1.0f + expf(-g4.z)) * u4.z * d4.z;
        hh[3] = g4.w / (1.0f + expf(-g4.w)) * u4.w * d4.w;
        fwht128_contig(hh, lane, PF_HS);
        *reinterpret_cast<uint2 *>(blocked_lane_ptr(p.xh_d, pos, c0 + i, lane, I)) = pack4(hh);
      }
    }
  }
}

// finish: one CTA per (token, 512-column quarter), one warp per slot + one for the shared expert: every warp finishes its
// slot's 4 chunks (H128, svh, routing weight) into shared memory, then the CTA sums the slots in slot order
// (reference pf_moe.metal:129-161)
constexpr int PF_FQ = 512;
__global__ void __launch_bounds__(32 * 17) pf_finish_kernel(const PfParams p) {
  extern __shared__ __align__(16) float vals_dyn[];  // [slots][PF_FQ]; the block has one warp per slot, at least 4 warps
  float(*vals)[PF_FQ] = reinterpret_cast<float(*)[PF_FQ]>(vals_dyn);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, q0 = blockIdx.x * PF_FQ, t = blockIdx.y, H = p.H, k = p.topk;
  const int nslots = k + (p.has_shared ? 1 : 0);
  const int nch = min(PF_FQ, H - q0) / 128;
  bool have = false;
  if (warp < nslots) {
    const bool shared = warp == k;
    const int pos = shared ? (t >= p.sh_row0 && t < p.sh_row0 + p.sh_rows ? p.off[p.E] + t - p.sh_row0 : -1) : p.inv[t * k + warp];
    have = pos >= 0;
  }
  if (have) {
    const bool shared = warp == k;
    const int pos = shared ? p.off[p.E] + t - p.sh_row0 : p.inv[t * k + warp];
    const int e = shared ? 0 : (int)p.route[(size_t)t * 2 * k + warp] - p.e0;
    const float w = shared ? 1.0f / (1.0f + expf(-p.logits[(size_t)t * (p.E + 1) + p.E])) : __uint_as_float(p.route[(size_t)t * 2 * k + k + warp]);
    const __half *sv = (shared ? p.sdn.svh : p.down.svh + (size_t)e * H) + q0;
    const float *raw = p.raw_d + (size_t)pos * H + q0;
    float4 rv[4];
    uint2 sc[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int o = min(i, nch - 1) * 128 + 4 * lane;
      rv[i] = *reinterpret_cast<const float4 *>(raw + o);
      sc[i] = *reinterpret_cast<const uint2 *>(sv + o);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      if (i < nch) {
        float v[4] = {rv[i].x, rv[i].y, rv[i].z, rv[i].w};
        fwht128_contig(v, lane, PF_HS);
        const float4 f = mul4(make_float4(v[0], v[1], v[2], v[3]), sc[i]);
        if (shared) *reinterpret_cast<float4 *>(p.sho + (size_t)t * H + q0 + i * 128 + 4 * lane) = f;
        *reinterpret_cast<float4 *>(&vals[warp][i * 128 + 4 * lane]) = make_float4(f.x * w, f.y * w, f.z * w, f.w * w);
      }
    }
  } else if (warp < nslots) {  // a slot computed on another rank, or a row whose shared expert runs elsewhere
#pragma unroll
    for (int i = 0; i < 4; i++) *reinterpret_cast<float4 *>(&vals[warp][i * 128 + 4 * lane]) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
  __syncthreads();
  const int c = threadIdx.x * 4;  // 128 threads cover the quarter
  if (c >= nch * 128) return;
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int s = 0; s < nslots; s++) {
    const float4 v = *reinterpret_cast<const float4 *>(&vals[s][c]);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  *reinterpret_cast<float4 *>(p.y + (size_t)t * H + q0 + c) = acc;
}

// =============================================================================================== one Linear, many rows
// y[n][out] = x[n][in] @ W for n > 64 rows (reference: t6::record_prefill, kernels/trunk6/trunk6.mm:385-492, which
// decodes W' densely once per chunk and runs an fp16 GEMM): the same grouped GEMM with a single group that holds all
// rows, i.e. every tile is decoded once per 128 rows straight into the tensor core's operand layout.
__global__ void __launch_bounds__(256) pfl_prep_kernel(const float *__restrict__ x, const __half *__restrict__ suh, __half *xh, int n, int n8, int in) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = blockIdx.x * 8 + warp;
  if (r >= n8) return;
  for (int c0 = 0; c0 < in / 128; c0 += 4) {
    float4 xv[4];
    uint2 sc[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int o = min(c0 + i, in / 128 - 1) * 128 + 4 * lane;
      xv[i] = r < n ? *reinterpret_cast<const float4 *>(x + (size_t)r * in + o) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      sc[i] = *reinterpret_cast<const uint2 *>(suh + o);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      if (c0 + i < in / 128) {
        const float4 m = mul4(xv[i], sc[i]);
        float v[4] = {m.x, m.y, m.z, m.w};
        fwht128_contig(v, lane, PF_HS);
        *reinterpret_cast<uint2 *>(blocked_lane_ptr(xh, r, c0 + i, lane, in)) = pack4(v);
      }
    }
  }
}

__global__ void pfl_items_kernel(PfItem *items, int *nitems, int n, int ncb) {
  const int passes = (n + PF_NTOK - 1) / PF_NTOK, total = passes * ncb;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int pass = i / ncb, cb = i - pass * ncb;
    items[i] = PfItem{-1, 0, cb, pass * PF_NTOK, min(PF_NTOK, n - pass * PF_NTOK), {0, 0, 0}};
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *nitems = total;
}

__global__ void __launch_bounds__(256) pfl_finish_kernel(const float *__restrict__ raw, const __half *__restrict__ svh, float *y, int n, int out) {
  const int lane = threadIdx.x & 31, nc = out / 128, job = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (job >= n * nc) return;
  const int r = job / nc, o = (job - r * nc) * 128 + 4 * lane;
  const float4 rv = *reinterpret_cast<const float4 *>(raw + (size_t)r * out + o);
  const uint2 sc = *reinterpret_cast<const uint2 *>(svh + o);
  float v[4] = {rv.x, rv.y, rv.z, rv.w};
  fwht128_contig(v, lane, PF_HS);
  *reinterpret_cast<float4 *>(y + (size_t)r * out + o) = mul4(make_float4(v[0], v[1], v[2], v[3]), sc);
}

size_t pf_linear_scratch_bytes(int in, int out, int n) {
  const size_t n8 = ((size_t)n + 7) & ~(size_t)7, passes = ((size_t)n + PF_NTOK - 1) / PF_NTOK;
  return n8 * in * 2 + n8 * out * 4 + passes * (out / PF_NCOL) * sizeof(PfItem) + 1024;
}

void launch_pf_linear(const void *trellis, const void *suh, const void *svh, int in, int out, int K, const float *x, int n, float *y,
                      void *scratch, int *status, cudaStream_t st) {
  IJ_CHECK(in % 128 == 0 && out % 256 == 0, "prefill Linear needs in %% 128 == 0 and out %% 256 == 0 (%d -> %d)", in, out);
  IJ_CHECK(K >= 4 && K <= 8, "EXL3 bits per weight %d outside 4..8", K);
  IJ_CHECK(n >= 1 && n <= 65535 * 8, "prefill Linear: %d rows", n);
  const size_t n8 = ((size_t)n + 7) & ~(size_t)7, passes = ((size_t)n + PF_NTOK - 1) / PF_NTOK;
  char *base = (char *)scratch;
  __half *xh = (__half *)base;
  float *raw = (float *)(base + n8 * in * 2);
  PfItem *items = (PfItem *)(base + n8 * in * 2 + n8 * out * 4);
  int *nitems = (int *)((char *)items + passes * (out / PF_NCOL) * sizeof(PfItem));
  nitems = (int *)(((uintptr_t)nitems + 15) & ~(uintptr_t)15);
  pfl_prep_kernel<<<(int)(n8 / 8), 256, 0, st>>>(x, (const __half *)suh, xh, n, (int)n8, in);
  pfl_items_kernel<<<8, 256, 0, st>>>(items, nitems, n, out / PF_NCOL);
  IJ_CUDA(cudaGetLastError());
  PgGemm g{};
  g.items = items; g.nitems = nitems;
  g.w_shared[0] = (const char *)trellis;
  g.act[0] = xh;
  g.out[0] = raw;
  g.ldo = out; g.in = in; g.IT = in / 16; g.OT = out / 16; g.Kx = K; g.Ks = K;
  launch_pf_gemm(g, status, st);
  pfl_finish_kernel<<<(n * (out / 128) + 7) / 8, 256, 0, st>>>(raw, (const __half *)svh, y, n, out);
  IJ_CUDA(cudaGetLastError());
}

// =============================================================================================== host side
size_t pf_pos_cap(int n, int topk, int E, bool has_shared) {
  return (((size_t)n * topk + 8 * (size_t)E + (has_shared ? n : 0) + 15) / 8) * 8;
}

void launch_pf_moe(const PfParams &p, int *status, cudaStream_t st) {
  IJ_CHECK(p.E <= 1024 && p.topk <= 16 && p.H % 256 == 0 && p.I % 256 == 0, "prefill: unsupported dims E %d top_k %d H %d I %d", p.E, p.topk, p.H, p.I);
  IJ_CHECK(p.n >= 1 && p.n <= 65535, "prefill: %d tokens outside 1..65535", p.n);
  const int groups = p.pos_cap / 8;
  IJ_CUDA(cudaMemsetAsync(p.order, 0xFF, (size_t)p.pos_cap * 4, st));
  IJ_CUDA(cudaMemsetAsync(p.seid, 0xFF, (size_t)p.pos_cap * 4, st));
  IJ_CHECK(p.H % LG_K == 0, "prefill: hidden %d must be a multiple of %d", p.H, LG_K);
  if (!p.external_route) {
    IJ_CUDA(cudaFuncSetAttribute(pf_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LG_SMEM));
    pf_logits_kernel<<<dim3((p.n + LG_T - 1) / LG_T, (p.E + LG_T - 1) / LG_T), 256, LG_SMEM, st>>>(p);
    pf_route_kernel<<<(p.n + 7) / 8, 256, 0, st>>>(p);
  } else {
    IJ_CHECK(!p.has_shared, "prefill: caller-routed pairs carry no shared expert");
  }
  IJ_CHECK(p.e0 >= 0 && p.ecount >= 0 && p.e0 + p.ecount <= p.E, "prefill: bad expert slice");
  IJ_CHECK(p.sh_row0 >= 0 && p.sh_rows >= 0 && p.sh_row0 + p.sh_rows <= p.n, "prefill: shared rows [%d, %d) outside [0, %d)", p.sh_row0, p.sh_row0 + p.sh_rows, p.n);
  const int nb = (p.S + PS_BLOCK - 1) / PS_BLOCK, nbs = p.has_shared ? (p.sh_rows + PS_BLOCK - 1) / PS_BLOCK : 0;
  pf_hist_kernel<<<nb, 32, 0, st>>>(p, p.hist);
  pf_blockscan_kernel<<<(p.E + 7) / 8, 256, 0, st>>>(p, p.hist, nb);
  pf_scan_kernel<<<1, 1024, 0, st>>>(p);
  pf_place_kernel<<<nb + nbs, 32, 0, st>>>(p, p.order, p.hist, nb);
  pf_prep_kernel<<<groups, 256, 0, st>>>(p, p.order);
  IJ_CUDA(cudaGetLastError());
  PgGemm g{};
  g.items = p.items_gu; g.nitems = p.nitems;
  g.w_routed[0] = p.gate.trellis; g.w_routed[1] = p.up.trellis; g.w_shared[0] = p.sgt.trellis; g.w_shared[1] = p.sup.trellis;
  g.act[0] = p.xh_g; g.act[1] = p.xh_u;
  g.out[0] = p.raw_gu; g.out[1] = p.raw_gu + p.I;
  g.ldo = 2 * p.I; g.in = p.H; g.IT = p.H / 16; g.OT = p.I / 16; g.Kx = p.Kx; g.Ks = p.has_shared ? p.Ks : p.Kx;
  launch_pf_gemm(g, status, st);
  pf_mid_kernel<<<groups, 256, 0, st>>>(p);
  IJ_CUDA(cudaGetLastError());
  PgGemm d{};
  d.items = p.items_d; d.nitems = p.nitems + 1;
  d.w_routed[0] = p.down.trellis; d.w_shared[0] = p.sdn.trellis;
  d.act[0] = p.xh_d;
  d.out[0] = p.raw_d;
  d.ldo = p.H; d.in = p.I; d.IT = p.I / 16; d.OT = p.H / 16; d.Kx = p.Kx; d.Ks = g.Ks;
  launch_pf_gemm(d, status, st);
  const int fslots = p.topk + (p.has_shared ? 1 : 0);  // one warp per slot; caller-routed pairs bring a single slot per row
  pf_finish_kernel<<<dim3((p.H + PF_FQ - 1) / PF_FQ, p.n), 32 * std::max(fslots, 4), (size_t)fslots * PF_FQ * 4, st>>>(p);
  IJ_CUDA(cudaGetLastError());
}

// =============================================================================================== all-to-all helpers
// Stable counting sort of the n * k (token, slot) pairs of a route array by owner rank (= expert id / per): packed row `at`
// of the dispatch buffer takes pair p, send_token[at] = its token, send_route[at] = (id, weight bits), pos[p] = at,
// counts[d] = pairs going to rank d. One CTA; every thread owns a contiguous run of pairs, the ranks are placed one
// after the other with a block-wide exclusive scan each (at most 16 ranks).
__global__ void __launch_bounds__(1024) pairs_by_owner_kernel(const uint32_t *__restrict__ route, int n, int k, int per, int world,
                                                              int *__restrict__ send_token, uint32_t *__restrict__ send_route,
                                                              int *__restrict__ pos, long long *__restrict__ counts) {
  __shared__ int wsum[32];
  const int P = n * k, tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = (P + T - 1) / T, lo = min(P, tid * chunk), hi = min(P, lo + chunk);
  int start = 0;
  for (int d = 0; d < world; d++) {
    int mine = 0;
    for (int pr = lo; pr < hi; pr++) mine += (int)(route[(size_t)(pr / k) * 2 * k + pr % k] / (uint32_t)per) == d ? 1 : 0;
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += a;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    int before = 0, total = 0;
    for (int w = 0; w < T / 32; w++) {
      before += w < warp ? wsum[w] : 0;
      total += wsum[w];
    }
    int at = start + before + inc - mine;
    for (int pr = lo; pr < hi; pr++) {
      const size_t r = (size_t)(pr / k) * 2 * k + pr % k;
      const uint32_t id = route[r];
      if ((int)(id / (uint32_t)per) == d) {
        send_token[at] = pr / k;
        send_route[2 * at] = id;
        send_route[2 * at + 1] = route[r + k];
        pos[pr] = at;
        at++;
      }
    }
    if (tid == 0) counts[d] = total;
    start += total;
    __syncthreads();
  }
}
void launch_pairs_by_owner(const uint32_t *route, int n, int k, int per, int world, int *send_token, uint32_t *send_route, int *pos,
                           long long *counts, cudaStream_t st) {
  IJ_CHECK(n >= 1 && k >= 1 && per >= 1 && world >= 1 && world <= 16, "pairs_by_owner: n %d k %d experts per rank %d ranks %d", n, k, per, world);
  pairs_by_owner_kernel<<<1, 1024, 0, st>>>(route, n, k, per, world, send_token, send_route, pos, counts);
  IJ_CUDA(cudaGetLastError());
}

// dst[i] = src[idx[i]] (rows of H floats, H a multiple of 4): packs the (token, slot) pairs of one destination rank after
// the other for the dispatch all-to-all. One CTA per output row.
__global__ void __launch_bounds__(256) rows_gather_kernel(const float4 *__restrict__ src, const int *__restrict__ idx, float4 *__restrict__ dst, int q) {
  const size_t i = blockIdx.x, r = (size_t)idx[i];
  for (int c = threadIdx.x; c < q; c += blockDim.x) dst[i * q + c] = __ldg(src + r * q + c);
}
void launch_rows_gather(const float *src, const int *idx, int n_out, int H, float *dst, cudaStream_t st) {
  IJ_CHECK(H % 4 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0, "rows_gather: rows of a multiple of 4 floats, 16-byte aligned");
  if (n_out <= 0) return;
  rows_gather_kernel<<<n_out, 256, 0, st>>>(reinterpret_cast<const float4 *>(src), idx, reinterpret_cast<float4 *>(dst), H / 4);
  IJ_CUDA(cudaGetLastError());
}

// y[t] = ((slot[pos[t][0]] + slot[pos[t][1]]) + .. + slot[pos[t][k-1]]) + base[t]: the combine of the all-to-all prefill on a
// token's home rank. The slots are added in slot order and the shared expert's term last, as pf_finish_kernel does on one
// GPU, so the result is bit-identical to it. pos < 0 skips a slot.
__global__ void __launch_bounds__(256) slots_combine_kernel(const float4 *__restrict__ slot, const int *__restrict__ pos, const float4 *__restrict__ base,
                                                            float4 *__restrict__ y, int k, int q) {
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < q; c += blockDim.x) {
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < k; s++) {
      const int ps = pos[t * k + s];
      if (ps >= 0) {
        const float4 v = __ldg(slot + (size_t)ps * q + c);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    if (base != nullptr) {
      const float4 b = base[t * q + c];
      acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    }
    y[t * q + c] = acc;
  }
}
void launch_slots_combine(const float *slot, const int *pos, const float *base, float *y, int n, int k, int H, cudaStream_t st) {
  IJ_CHECK(H % 4 == 0 && (((uintptr_t)slot | (uintptr_t)base | (uintptr_t)y) & 15) == 0, "slots_combine: rows of a multiple of 4 floats, 16-byte aligned");
  IJ_CHECK(n >= 1 && k >= 1, "slots_combine: %d tokens, %d slots", n, k);
  slots_combine_kernel<<<n, 256, 0, st>>>(reinterpret_cast<const float4 *>(slot), pos, reinterpret_cast<const float4 *>(base),
                                          reinterpret_cast<float4 *>(y), k, H / 4);
  IJ_CUDA(cudaGetLastError());
}

}  // namespace ijah
