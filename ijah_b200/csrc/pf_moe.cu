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
  const int ng = dw >> 3, t = dw & 7, q = lane & 3, c = lane >> 2;
#pragma unroll
  for (int ks = 0; ks < PG_KS; ks++) {
    const unsigned char *tile = ring_stage + (size_t)(ks * 16 + dw) * Codec<K>::TILE_BYTES;
    uint32_t b[4];
    dec8<K>(*reinterpret_cast<const uint32_t *>(tile + L.o0), *reinterpret_cast<const uint32_t *>(tile + L.o1),
            *reinterpret_cast<const uint32_t *>(tile + L.o2), L.a, b);
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
  static bool ready = false;
  if (!ready) {
    IJ_CUDA(cudaFuncSetAttribute(pf_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    ready = true;
  }
  pf_gemm_kernel<<<sm_count(), PG_THREADS, smem, st>>>(g, status);
  IJ_CUDA(cudaGetLastError());
}

// (the routing, sorting, operand and finishing kernels follow)

// =============================================================================================== router
// logits[n][E + 1] = x . W^T (bf16 W, fp32 accumulate; row E = the shared expert's gate), one 64 x 64 tile per CTA.
// Reference: the router GEMM of the chunked prefill (kernels/prefill/pf_gemm.metal:159-186) + pf_moe_route
// (kernels/prefill/pf_trunk.metal:278-334).
__global__ void __launch_bounds__(256) pf_logits_kernel(const PfParams p) {
  __shared__ float xs[64][33], ws[64][33];
  const int t0 = blockIdx.x * 64, c0 = blockIdx.y * 64, tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.H; k0 += 32) {
    for (int i = threadIdx.x; i < 64 * 32; i += 256) {
      const int r = i >> 5, k = i & 31;
      xs[r][k] = t0 + r < p.n ? p.x[(size_t)(t0 + r) * p.H + k0 + k] : 0.0f;
      const int c = c0 + r;
      const uint16_t *wr = c < p.E ? p.router + (size_t)c * p.H : (c == p.E ? p.sgate : nullptr);
      ws[r][k] = wr ? __uint_as_float((uint32_t)wr[k0 + k] << 16) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < 32; k++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { a[i] = xs[ty * 4 + i][k]; b[i] = ws[tx * 4 + i][k]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int t = t0 + ty * 4 + i, c = c0 + tx * 4 + j;
      if (t < p.n && c <= p.E) p.logits[(size_t)t * (p.E + 1) + c] = acc[i][j];
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
// Deterministic counting sort of the n * topk slots (reference kernels/prefill/pf_moe.metal:29-83): one CTA per
// expert counts its slots and ranks them in slot order; one CTA lays out the experts' position ranges (padded to 8 rows,
// the granule of the blocked operand layout) and writes the work items; one thread per slot places it.
__global__ void __launch_bounds__(256) pf_count_kernel(const PfParams p) {
  __shared__ int part[256];
  const int e = blockIdx.x, tid = threadIdx.x, k = p.topk;
  const int per = (p.S + 255) / 256, s0 = min(tid * per, p.S), s1 = min(s0 + per, p.S);
  int c = 0;
  for (int s = s0; s < s1; s++) c += (int)p.route[(size_t)(s / k) * 2 * k + s % k] == e ? 1 : 0;
  part[tid] = c;
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int j = 0; j < 256; j++) { const int v = part[j]; part[j] = acc; acc += v; }
    p.cnt[blockIdx.x] = acc;
  }
  __syncthreads();
  int r = part[tid];
  for (int s = s0; s < s1; s++)
    if ((int)p.route[(size_t)(s / k) * 2 * k + s % k] == e) p.rank[s] = r++;
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
  const int e = threadIdx.x, E = p.E;
  const int c = e < E ? p.cnt[e] : 0, c8 = (c + 7) & ~7, np = (c + PF_NTOK - 1) / PF_NTOK;
  const int o = block_excl_scan(c8, wt, &tot8);
  const int pb = block_excl_scan(np, wt, &totp);
  if (e < E) p.off[e] = o;
  const int nsh = p.has_shared ? p.n : 0, shp = (nsh + PF_NTOK - 1) / PF_NTOK;
  if (e == 0) {
    p.off[E] = tot8;
    p.off[E + 1] = tot8 + ((nsh + 7) & ~7);
    p.nitems[0] = (totp + shp) * 2 * (p.I / PF_NCOL);
    p.nitems[1] = (totp + shp) * (p.H / PF_NCOL);
  }
  const int GU = p.I / PF_NCOL, DN = p.H / PF_NCOL;
  auto emit = [&](int pass, int expert, int row0, int nrows) {
    for (int j = 0; j < 2 * GU; j++) p.items_gu[pass * 2 * GU + j] = PfItem{expert, j / GU, j % GU, row0, nrows, {0, 0, 0}};
    for (int j = 0; j < DN; j++) p.items_d[pass * DN + j] = PfItem{expert, 0, j, row0, nrows, {0, 0, 0}};
  };
  for (int j = 0; j < np; j++) emit(pb + j, e, o + j * PF_NTOK, min(PF_NTOK, c - j * PF_NTOK));
  for (int j = e; j < shp; j += blockDim.x) emit(totp + j, -1, tot8 + j * PF_NTOK, min(PF_NTOK, nsh - j * PF_NTOK));
}

// order[pos] = slot (S + t for the shared expert's row of token t, -1 = padding), inv[slot] = pos, seid[pos] = expert
// (E = shared). order / seid are pre-set to -1 by the launcher.
__global__ void __launch_bounds__(256) pf_place_kernel(const PfParams p, int *order) {
  const int i = blockIdx.x * 256 + threadIdx.x, k = p.topk;
  if (i < p.S) {
    const int e = (int)p.route[(size_t)(i / k) * 2 * k + i % k], pos = p.off[e] + p.rank[i];
    order[pos] = i;
    p.inv[i] = pos;
    p.seid[pos] = e;
  } else if (i < p.S + p.n && p.has_shared) {
    const int t = i - p.S, pos = p.off[p.E] + t;
    order[pos] = p.S + t;
    p.seid[pos] = p.E;
  }
}

// 8 positions x 128 k of fp16 in shared memory -> the blocked global layout: 16 core matrices = 2 KB contiguous
__device__ __forceinline__ void store_blocked_chunk(const __half (*tile)[128], __half *dst_group_chunk) {
  const int c = threadIdx.x >> 4, r = (threadIdx.x >> 1) & 7, h = threadIdx.x & 1;  // 256 threads x 8 bytes
  *reinterpret_cast<uint2 *>(dst_group_chunk + c * 64 + r * 8 + h * 4) = *reinterpret_cast<const uint2 *>(&tile[r][c * 8 + h * 4]);
}

// gate / up operands: xh[pos] = fp16(H128(x[token(pos)] * suh[expert(pos)])), one CTA per (8-position group, 128-chunk),
// one warp per position (reference kernels/prefill/pf_moe.metal:88-104)
__global__ void __launch_bounds__(256) pf_prep_kernel(const PfParams p, const int *order) {
  __shared__ __align__(16) __half tg[8][128], tu[8][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x, grp = blockIdx.y, pos = grp * 8 + warp, H = p.H;
  const int slot = pos < p.off[p.E + 1] ? order[pos] : -1;
  float g[4] = {0, 0, 0, 0}, u[4] = {0, 0, 0, 0};
  if (slot >= 0) {
    const bool shared = slot >= p.S;
    const int t = shared ? slot - p.S : slot / p.topk;
    const int e = shared ? 0 : p.seid[pos];
    const __half *sg = shared ? p.sgt.suh : p.gate.suh + (size_t)e * H, *su = shared ? p.sup.suh : p.up.suh + (size_t)e * H;
    const int o = chunk * 128 + lane;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float xv = p.x[(size_t)t * H + o + 32 * j];
      g[j] = xv * __half2float(sg[o + 32 * j]);
      u[j] = xv * __half2float(su[o + 32 * j]);
    }
    fwht_chunk(g, lane, 128, 0.08838834764831845f);
    fwht_chunk(u, lane, 128, 0.08838834764831845f);
  }
#pragma unroll
  for (int j = 0; j < 4; j++) {
    tg[warp][lane + 32 * j] = __float2half_rn(g[j]);
    tu[warp][lane + 32 * j] = __float2half_rn(u[j]);
  }
  __syncthreads();
  const size_t base = ((size_t)grp * (H >> 3) + chunk * 16) * 64;
  store_blocked_chunk(tg, p.xh_g + base);
  store_blocked_chunk(tu, p.xh_u + base);
}

// down operand: SwiGLU of the finished gate / up, times suh_down, H128, fp16 (reference pf_moe.metal:107-125)
__global__ void __launch_bounds__(256) pf_mid_kernel(const PfParams p) {
  __shared__ __align__(16) __half td[8][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x, grp = blockIdx.y, pos = grp * 8 + warp, I = p.I;
  const int e = pos < p.off[p.E + 1] ? p.seid[pos] : -1;
  float hh[4] = {0, 0, 0, 0};
  if (e >= 0) {
    const bool shared = e == p.E;
    const __half *svg = shared ? p.sgt.svh : p.gate.svh + (size_t)e * I, *svu = shared ? p.sup.svh : p.up.svh + (size_t)e * I;
    const __half *sud = shared ? p.sdn.suh : p.down.suh + (size_t)e * I;
    const float *raw = p.raw_gu + (size_t)pos * 2 * I;
    const int o = chunk * 128 + lane;
    float gv[4], uv[4];
#pragma unroll
    for (int j = 0; j < 4; j++) { gv[j] = raw[o + 32 * j]; uv[j] = raw[I + o + 32 * j]; }
    fwht_chunk(gv, lane, 128, 0.08838834764831845f);
    fwht_chunk(uv, lane, 128, 0.08838834764831845f);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      gv[j] *= __half2float(svg[o + 32 * j]);
      uv[j] *= __half2float(svu[o + 32 * j]);
      hh[j] = gv[j] / (1.0f + expf(-gv[j])) * uv[j] * __half2float(sud[o + 32 * j]);
    }
    fwht_chunk(hh, lane, 128, 0.08838834764831845f);
  }
#pragma unroll
  for (int j = 0; j < 4; j++) td[warp][lane + 32 * j] = __float2half_rn(hh[j]);
  __syncthreads();
  store_blocked_chunk(td, p.xh_d + ((size_t)grp * (I >> 3) + chunk * 16) * 64);
}

// finish: per (token, 128-column block) one warp per slot + one for the shared expert; slot-ordered sum
// (reference pf_moe.metal:129-161)
__global__ void __launch_bounds__(32 * 17) pf_finish_kernel(const PfParams p) {
  __shared__ float vals[17][128];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, blk = blockIdx.x, t = blockIdx.y, H = p.H, k = p.topk;
  const float hs = 0.08838834764831845f;
  if (warp <= k) {
    const bool shared = warp == k;
    if (!shared || p.has_shared) {
      const int pos = shared ? p.off[p.E] + t : p.inv[t * k + warp];
      const int e = shared ? 0 : (int)p.route[(size_t)t * 2 * k + warp];
      const float w = shared ? 1.0f / (1.0f + expf(-p.logits[(size_t)t * (p.E + 1) + p.E])) : __uint_as_float(p.route[(size_t)t * 2 * k + k + warp]);
      const __half *sv = (shared ? p.sdn.svh : p.down.svh + (size_t)e * H) + blk * 128;
      const float *raw = p.raw_d + (size_t)pos * H + blk * 128;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; j++) v[j] = raw[lane + 32 * j];
      fwht_chunk(v, lane, 128, hs);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float f = v[j] * __half2float(sv[lane + 32 * j]);
        if (shared) p.sho[(size_t)t * H + blk * 128 + lane + 32 * j] = f;
        vals[warp][lane + 32 * j] = f * w;
      }
    }
  }
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    float acc = 0.0f;
    for (int s = 0; s < k + (p.has_shared ? 1 : 0); s++) acc += vals[s][lane + 32 * j];
    p.y[(size_t)t * H + blk * 128 + lane + 32 * j] = acc;
  }
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
  pf_logits_kernel<<<dim3((p.n + 63) / 64, (p.E + 1 + 63) / 64), 256, 0, st>>>(p);
  pf_route_kernel<<<(p.n + 7) / 8, 256, 0, st>>>(p);
  pf_count_kernel<<<p.E, 256, 0, st>>>(p);
  pf_scan_kernel<<<1, 1024, 0, st>>>(p);
  pf_place_kernel<<<(p.S + p.n + 255) / 256, 256, 0, st>>>(p, p.order);
  pf_prep_kernel<<<dim3(p.H / 128, groups), 256, 0, st>>>(p, p.order);
  IJ_CUDA(cudaGetLastError());
  PgGemm g{};
  g.items = p.items_gu; g.nitems = p.nitems;
  g.w_routed[0] = p.gate.trellis; g.w_routed[1] = p.up.trellis; g.w_shared[0] = p.sgt.trellis; g.w_shared[1] = p.sup.trellis;
  g.act[0] = p.xh_g; g.act[1] = p.xh_u;
  g.out[0] = p.raw_gu; g.out[1] = p.raw_gu + p.I;
  g.ldo = 2 * p.I; g.in = p.H; g.IT = p.H / 16; g.OT = p.I / 16; g.Kx = p.Kx; g.Ks = p.has_shared ? p.Ks : p.Kx;
  launch_pf_gemm(g, status, st);
  pf_mid_kernel<<<dim3(p.I / 128, groups), 256, 0, st>>>(p);
  IJ_CUDA(cudaGetLastError());
  PgGemm d{};
  d.items = p.items_d; d.nitems = p.nitems + 1;
  d.w_routed[0] = p.down.trellis; d.w_shared[0] = p.sdn.trellis;
  d.act[0] = p.xh_d;
  d.out[0] = p.raw_d;
  d.ldo = p.H; d.in = p.I; d.IT = p.I / 16; d.OT = p.H / 16; d.Kx = p.Kx; d.Ks = g.Ks;
  launch_pf_gemm(d, status, st);
  pf_finish_kernel<<<dim3(p.H / 128, p.n), 32 * 17, 0, st>>>(p);
  IJ_CUDA(cudaGetLastError());
}

}  // namespace ijah
