// Decode MoE block on sm_100a: router + top-k, routed gate/up, SwiGLU + down, slot-ordered combine, shared expert.
// Replaces the reference's fn_moe_router / fn_moe_gateup / fn_moe_down (kernels/fn_moe.metal:26-452) and, for rows > 1,
// its grouped-by-expert scheduling (kernels/fn_moe.metal:135-241, 692-884): every distinct expert is streamed once and
// multiplied with all rows that routed to it.
#pragma once
#include "ep_exchange.cuh"
#include "exl3_linear.cuh"

namespace ijah {

struct Exl3Stack {
  const char *trellis;
  const __half *suh;
  const __half *svh;
};

struct MoeParams {
  int H, I, E, topk, Kx, Ks;
  int e0, ecount;     // local expert slice
  int rows;           // live rows of this run
  int P;              // rows * topk
  int has_shared;
  int dup;            // store_a's pair form: the product mode in force when the call was enqueued
  int shared_pre;     // the shared expert's output is already in `sho` (8-bit affine shared expert: computed by other kernels)
  // weights
  const uint16_t *router;  // bf16 [E][H]
  const uint16_t *sgate;   // bf16 [H]
  Exl3Stack gate, up, down;        // [ecount]
  Exl3Stack sgt, sup, sdn;         // shared expert
  // activations / scratch (device)
  const float *x;          // [rows][H]
  float *logits;           // [rows][E + 1]
  uint32_t *route;         // [rows][2 topk]
  int *plan;               // see PlanView
  __half *xh_gu;           // [P][2][2H]  prepared gate | up operands per (row, slot) pair (store_a layout)
  __half *xh_sgu;          // [rows][2][2H]  the shared expert's
  __half *xh_d;            // [P][2I]  prepared down operand per pair
  __half *xh_sd;           // [rows][2I]
  float *raw_gu;           // [S_gu][P][2][I]
  float *raw_sgu;          // [S_gu][rows][2][I]
  float *raw_d;            // [S_d][P][H]
  float *raw_sd;           // [S_d][rows][H]
  float *gush;             // [rows][2 I]   finished shared gate | up
  float *sho;              // [rows][H]     finished shared down
  float *y;                // [rows][H]
  unsigned *counter;
  // k-splits
  int S_gu, kc_gu, S_d, kc_d;
  // optional hyper-connection write (reference kernels/fn_moe.metal:446-450): h_out[r][s][c] = h[r][s][c] + y[r][c] * inj[r][s]
  const float *h_mid;      // [rows][HC][H] or null
  const float *inj;        // [rows][2 HC]
  float *h_out;            // [rows][HC][H]
  int HC;
  // rows [sh_row0, sh_row0 + sh_rows) get the shared-expert term in the combine (expert parallel: a rank adds it only
  // for the rows it owns, so that the sum over ranks contains it once); single GPU: 0, rows
  int sh_row0, sh_rows;
  // expert parallel over peer memory (null = off): the combine writes each finished row into the part buffer of the rank that
  // owns it and, when its last CTA is done, raises this rank's flag on every peer with the block's epoch (*ep->epoch)
  const EpDev *ep;
  int ep_rows;         // rows per rank (the gathered rows are world * ep_rows)
  int ldx, ldr;  // row strides of x (floats) and route (words): H and 2 topk unless rows and routes arrive packed side by side
  int lg_row0;  // logits[] holds rows [lg_row0, ..) (expert parallel with own-row routing: only the own rows were routed here)
};

// plan[] layout (ints): [0] = number of entries nu, [1] = number of distinct local experts; then four arrays of P entries
// each: expert id, row count (<= PLAN_ROWS), offset into pairs[], and pairs[] (pair = row * topk + slot) grouped by
// expert, rows ascending. An expert with more than PLAN_ROWS rows has several consecutive entries.
constexpr int PLAN_ROWS = 8;
struct PlanView {
  int *base;
  int P;
  __host__ __device__ int *nu() const { return base; }
  __host__ __device__ int *distinct() const { return base + 1; }
  __host__ __device__ int *expert() const { return base + 4; }
  __host__ __device__ int *nrows() const { return base + 4 + P; }
  __host__ __device__ int *first() const { return base + 4 + 2 * P; }
  __host__ __device__ int *pairs() const { return base + 4 + 3 * P; }
  static size_t ints(int P) { return 4 + 4 * (size_t)P; }
};

// tensor maps over the six trellis stacks of a block (make_trellis_map), built once per MoE object
struct MoeMaps {
  alignas(64) CUtensorMap gate, up, down, sgt, sup, sdn;
};

struct MoeSplits {
  int S_gu, kc_gu, S_d, kc_d, MT;
  StreamLayout lay_gu, lay_d;
  int grid;
};
MoeSplits plan_moe(int H, int I, int E, int topk, int Kx, int Ks, int rows, bool has_shared);

void launch_moe_router(const MoeParams &p, bool build_plan, cudaStream_t st);
// gate / up operands (after routing); build_plan: also the expert plan from the route buffer (when the router did not)
void launch_moe_prep(const MoeParams &p, bool build_plan, cudaStream_t st);
void launch_moe_mid(const MoeParams &p, cudaStream_t st);    // SwiGLU + down operand (after gate / up)
// plan_final: the plan was written by a kernel that completed before this launch can start (the router, with the prep kernel
// in between), so the first weights are streamed before the wait on the predecessor
void launch_moe_gateup(const MoeParams &p, const MoeMaps &maps, const MoeSplits &s, bool plan_final, int *status, cudaStream_t st);
void launch_moe_down(const MoeParams &p, const MoeMaps &maps, const MoeSplits &s, int *status, cudaStream_t st);
void launch_moe_combine(const MoeParams &p, bool routed_only, cudaStream_t st);
// gush[r] = (g | u), act[r] = silu(g) * u for the 8-bit shared expert's gate / up outputs g, u f32 [rows][I]
void launch_swiglu_rows(const float *g, const float *u, int rows, int I, float *gush, float *act, cudaStream_t st);

}  // namespace ijah
