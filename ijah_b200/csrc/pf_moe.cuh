// Prefill MoE: tokens sorted by expert, grouped trellis GEMM on tcgen05 / TMEM, slot-ordered finish.
// Replaces the reference's kernels/prefill/pf_moe.metal (pf_moe_count / scan / place / prep / gemm / mid / finish,
// recorded by models/flash_next/prefill.mm:235-276) and the router part of kernels/prefill/pf_trunk.metal:278-334.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "fn_moe.cuh"

namespace ijah {

constexpr int PF_NTOK = 128;   // token rows per GEMM pass (the N of the MMA)
constexpr int PF_NCOL = 256;   // output columns per work item (two M = 128 accumulators)

// One pass of the grouped GEMM: rows [row0, row0 + nrows) of the sorted (8-row padded) position space, all of one
// expert, times 256 output columns of one projection.
struct PfItem {
  int expert;   // local expert index, or -1 for the shared expert
  int proj;     // gate/up launch: 0 gate, 1 up; down launch: 0
  int ngpair;   // which block of 256 output columns
  int row0;     // first position (multiple of 8)
  int nrows;    // 1..PF_NTOK
  int pad[3];
};

struct PfParams {
  int H, I, E, topk, Kx, Ks, has_shared;
  int e0, ecount;  // the experts this object holds (expert parallel): slots of other experts are left to their owners
  int sh_row0, sh_rows;  // tokens whose shared expert is computed here
  int n;           // tokens
  int S;           // n * topk slots
  int pos_cap;     // capacity of the padded position space
  int external_route;  // `route` was filled by the caller ([n][2 topk], read only): no router GEMM, no top-k
  // weights
  const uint16_t *router, *sgate;
  Exl3Stack gate, up, down, sgt, sup, sdn;
  // activations / scratch
  const float *x;        // [n][H]
  float *logits;         // [n][E + 1]
  uint32_t *route;       // [n][2 topk]
  int *cnt;              // [E] slots per expert
  int *off;              // [E + 2] first position of each expert (8-row padded); [E] = first shared position, [E + 1] = end
  int *hist;             // [ceil(S / 256)][E] per-block expert counts, then their exclusive scan over the blocks
  int *inv;              // [S] slot -> position
  int *order;            // [pos_cap] position -> slot (S + t = shared row of token t, -1 = padding), rewritten every run
  int *seid;             // [pos_cap] position -> expert (E = shared, -1 = padding), rewritten every run
  __half *xh_g, *xh_u;   // [pos_cap / 8][H / 8][8][8] blocked operands (see blocked_index)
  float *raw_gu;         // [pos_cap][2][I]
  __half *xh_d;          // [pos_cap / 8][I / 8][8][8]
  float *raw_d;          // [pos_cap][H]
  PfItem *items_gu, *items_d;
  int *nitems;           // [2]: gate/up items, down items
  float *y;              // [n][H]
  float *sho;            // [n][H] finished shared down (inspection)
};

// element (pos, k) of a blocked operand with `in` columns: core matrices of 8 positions x 8 k, 128 contiguous bytes each,
// the in/8 core matrices of one 8-position group contiguous. A GEMM stage (8 k-chunks of one group) is 1 KB contiguous.
__host__ __device__ inline size_t blocked_index(int pos, int k, int in) {
  return (((size_t)(pos >> 3) * (in >> 3) + (k >> 3)) << 6) + ((pos & 7) << 3) + (k & 7);
}

size_t pf_pos_cap(int n, int topk, int E, bool has_shared);
void launch_pf_moe(const PfParams &p, int *status, cudaStream_t st);
// one EXL3 Linear over n rows through the grouped tensor-core GEMM; scratch: pf_linear_scratch_bytes(in, out, n)
size_t pf_linear_scratch_bytes(int in, int out, int n);
void launch_pf_linear(const void *trellis, const void *suh, const void *svh, int in, int out, int K, const float *x, int n, float *y,
                      void *scratch, int *status, cudaStream_t st);

// helpers of the all-to-all expert-parallel prefill: pack rows by index; add a token's returned slots in slot order
void launch_pairs_by_owner(const uint32_t *route, int n, int k, int per, int world, int *send_token, uint32_t *send_route, int *pos,
                           long long *counts, cudaStream_t st);
void launch_rows_gather(const float *src, const int *idx, int n_out, int H, float *dst, cudaStream_t st);
void launch_slots_combine(const float *slot, const int *pos, const float *base, float *y, int n, int k, int H, cudaStream_t st);

}  // namespace ijah
