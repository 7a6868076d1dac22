/* libijah_b200: entry points beyond the reference's engine.h, following its extension rule (reference
 * include/engine.h:11-12: other components declare their NE_API functions in a header of their own).
 *
 * These are the dimension-explicit forms of the hot path: one EXL3 Linear, one MoE block (decode widths), the prefill
 * grouped GEMM, and the expert-parallel variants. All pointers named *_dev are device pointers, `stream` is a
 * cudaStream_t passed as void* (NULL = the default stream). Calls that take a stream only enqueue work; the *_host
 * forms copy host inputs in, run, copy results out and return when everything is done. Errors: 0 / -1 and
 * ne_last_error(), as in ijah_engine.h.
 */
#ifndef IJAH_B200_H
#define IJAH_B200_H

#include "ijah_engine.h"

#ifdef __cplusplus
extern "C" {
#endif

/* One EXL3-coded Linear y = x @ W, W [in, out] = diag(suh) H W' H diag(svh)
 * (replaces the reference's t6::Linear, kernels/trunk6/trunk6.h:24-32: trellis U16 [in/16][out/16][16K], suh F16 [in],
 * svh F16 [out]; K = 4..8 bits per weight). */
typedef struct {
  const void *trellis_dev;
  const void *suh_dev;
  const void *svh_dev;
  int in, out, K;
} ne_exl3_weight;

/* W' (the trellis decoded to its fp16 codebook values, no rotations) as F16 [in][out]: the bit-exact parity surface
 * of the decoder (reference decoder: kernels/ne_common.h:133-157 dec_mcg/dec8, kernels/trunk6/trunk6.metal:102-127). */
NE_API int ne_exl3_dequant(const ne_exl3_weight *w, void *w_f16_dev, void *stream);
/* y[rows][out] = x[rows][in] @ W, f32 in / f32 out, rows 1..64 (replaces t6::record, kernels/trunk6/trunk6.h:60-79,
 * kernels t6_simd / t6_prep + t6_nax, kernels/trunk6/trunk6.metal:366-539). Scratch comes from a per-device arena
 * owned by the library (grown on demand). */
NE_API int ne_exl3_linear(const ne_exl3_weight *w, const float *x_dev, int rows, float *y_dev, void *stream);
NE_API int ne_exl3_linear_host(const ne_exl3_weight *w, const float *x_host, int rows, float *y_host);
/* The launch plan ne_exl3_linear would use (host arithmetic only, no device needed): info8 = k-splits S, k-tiles per unit,
 * ring stages, A slots, grid, 8-row groups, dynamic shared memory bytes, bytes per ring stage; scratch_bytes = the scratch
 * the call needs (what ne_exl3_linear_static compares with its capacity). -1 if the shape is not supported. */
NE_API int ne_exl3_linear_plan(int n_in, int n_out, int K, int rows, int *info8, uint64_t *scratch_bytes);
/* The same for one MoE block: info8 = gate/up splits, gate/up k-tiles per unit, down splits, down k-tiles per unit, ring
 * stages (gate/up, down), grid, dynamic shared memory bytes. */
NE_API int ne_moe_plan(int hidden, int inter, int experts, int top_k, int k_expert, int k_shared, int rows, int *info8);
/* n (1..4) Linears applied to the SAME rows x (the q, k, v projections of a layer; replaces t6::record_multi,
 * kernels/trunk6/trunk6.h:78-79, for the case of one shared input): one chain of three launches whose stream kernel holds the units of all matrices, so small
 * matrices neither pay a launch chain each nor leave most of the GPU idle. All w[i].in must be equal; y_dev[i] receives
 * [rows][w[i].out]. rows 1..64. */
NE_API int ne_exl3_linear_multi(const ne_exl3_weight *w, int n, const float *x_dev, int rows, float *const *y_dev, void *stream);
/* The same Linear for many rows (prefill chunks; replaces t6::record_prefill, kernels/trunk6/trunk6.mm:385-492): every tile is
 * decoded once per 128 rows into shared memory and multiplied on tcgen05 tensor cores with TMEM accumulators. rows >= 1;
 * in must be a multiple of 128, out of 256. Scratch from the library's per-device arena. */
NE_API int ne_exl3_linear_prefill(const ne_exl3_weight *w, const float *x_dev, int rows, float *y_dev, void *stream);
/* One 8-bit affine Linear y = x @ W^T, W [out][in] = scale * q + bias per group (replaces the reference's q8 Linears:
 * loader models/flash_next/layer.mm:60-76, arithmetic kernels/ne_common.h:31-91, the LM head kernels/fn_model.metal:152-168;
 * MLX layout: weight bytes [out][in] (U32 [out][in/4] in the pack), scales / biases BF16 [out][in/group]; ne_q8_linear takes
 * groups of 64, 128 or 256 and a multiple of 64 inputs, ne_q8_embed any group from 32). */
typedef struct {
  const void *weight_dev;
  const void *scales_dev;
  const void *biases_dev;
  int in, out, group;
} ne_q8_weight;
/* rows 1..64; x f32 [rows][in], y f32 [rows][out]; one kernel per 16 rows, no scratch. The activations enter the tensor
 * core as fp16 hi + lo pairs, so the result agrees with f32 arithmetic to rounding for |x| < 65504 (the fp16 range; normed
 * activations are far inside it). */
NE_API int ne_q8_linear(const ne_q8_weight *w, const float *x_dev, int rows, float *y_dev, void *stream);
/* Embedding lookup of an 8-bit affine table (reference kernels/fn_model.metal:14-40): x[r] = dequantised row tokens[r],
 * rounded to bf16 when round_bf16 != 0 (the reference's embedding is bf16-valued). tokens_dev: int32 [rows]. */
NE_API int ne_q8_embed(const ne_q8_weight *w, const int *tokens_dev, int rows, float *x_dev, int round_bf16, void *stream);
/* ne_exl3_linear for callers that must not allocate (no counterpart in the reference, whose unified-memory engine has
 * no such constraint). ne_exl3_linear grows a cudaMalloc'ed arena when a call needs more scratch than any call before
 * it; that is unusable from inside an allocator or memory-pool hook, in a serving loop that was given a fixed memory
 * budget at start-up, or next to another runtime that already owns the rest of the device memory. This variant runs
 * the same kernels on a scratch area compiled into the library (a 256-byte aligned __device__ array of
 * ne_exl3_linear_static_capacity() = 8 MiB bytes, held by every GPU that loads the library until the process exits)
 * and calls no cudaMalloc / cudaFree nor any allocating routine. Same arguments and results as ne_exl3_linear. A
 * call whose scratch need exceeds the capacity is refused with -1 and a message naming both sizes. The need is
 * rows * (4 * S * out + 2 * in) bytes plus padding, S = the number of k-splits the launch plan picks to fill the GPU
 * (1 for matrices with many output columns, up to in / 128 for small ones: 4096 x 4096 at 64 rows takes S = 32 and does
 * not fit, every trunk and expert shape of the benchmark configurations fits at <= 32 rows). The first call on a device
 * resolves the array's device address; make it before any stream capture begins. All calls share the one area: it keeps
 * the last call's contents (nothing needs to start at zero), and calls whose GPU work overlaps race on it. A bounded
 * device-side wait that gives up is reported in the same status word as for every other entry point
 * (ne_device_wait_status, which allocates nothing either). */
NE_API int ne_exl3_linear_static(const ne_exl3_weight *w, const float *x_dev, int rows, float *y_dev, void *stream);
NE_API uint64_t ne_exl3_linear_static_capacity(void);

/* ---- MoE block (router, routed experts, shared expert) at decode widths --------------------------------------
 * Replaces the three dispatches fn_moe_router / fn_moe_gateup / fn_moe_down of the reference
 * (kernels/fn_moe.metal:26-452, recorded by models/flash_next/layer.mm:532-564 and layer_t6.mm:191-243). */
typedef struct {
  const void *trellis_dev; /* U16 [n_local][in/16][out/16][16K] */
  const void *suh_dev;     /* F16 [n_local][in] */
  const void *svh_dev;     /* F16 [n_local][out] */
} ne_exl3_stack;

typedef struct {
  int hidden, inter, experts, top_k;
  int k_expert, k_shared;          /* bits per weight of the routed / shared projections */
  int expert_first, expert_count;  /* the slice of experts whose weights this object holds (expert parallel);
                                      single GPU: 0, experts */
  const void *router_dev;          /* BF16 [experts][hidden], all experts */
  const void *shared_gate_w_dev;   /* BF16 [hidden]: the sigmoid gate of the shared expert; NULL = no shared expert */
  ne_exl3_stack gate, up, down;    /* routed experts, local slice */
  ne_exl3_weight sh_gate, sh_up, sh_down;
  /* the shared expert as three 8-bit affine Linears instead (packs whose trunk was not converted to EXL3; reference loader
   * models/flash_next/layer.mm:60-76): used when sh_gate.trellis_dev is NULL and sh_gate_q8.weight_dev is not. Decode-width
   * single-GPU calls only (ne_moe_forward, ne_moe_stage); the prefill and expert-parallel entry points refuse such an object. */
  ne_q8_weight sh_gate_q8, sh_up_q8, sh_down_q8;
} ne_moe_desc;

/* Product mode of the decode-width kernels (ne_exl3_linear*, ne_moe_*, the layer and model objects; not the prefill
 * kernels, which always multiply the rounded weights). No counterpart in the reference.
 *   0 (default): every weight enters the tensor core as fp16(lo + hi), the value the EXL3 format defines
 *                (reference kernels/ne_common.h:133-157); results differ from the reference's only by summation order.
 *   1: every weight enters as its two fp16 summands lo, hi and the fp32 accumulator forms lo * x + hi * x; the sum is not
 *      rounded to fp16 first (at most half an fp16 ulp per weight, about 2e-4 relative on an output), which saves one
 *      instruction per weight in the decode loop. Opt-in.
 * Returns the previous mode; any other argument only reads it. The mode is read when a call is enqueued: a CUDA graph
 * (the layer and model objects record theirs on first use of a row count) keeps the mode it was recorded in, so set it
 * before creating those objects. Not thread-safe against concurrent launches. */
NE_API int ne_exl3_set_summand_product(int on);

typedef struct ne_moe ne_moe;
NE_API ne_moe *ne_moe_create(const ne_moe_desc *d, int max_rows); /* max_rows 1..64; allocates all scratch */
NE_API void ne_moe_free(ne_moe *m);
/* y[rows][hidden] = sum_k w_k expert_k(x) + sigmoid(x . w_sg) shared(x). Enqueues 6 kernels on `stream`
 * (router + plan, operand prep, gate/up, SwiGLU + operand prep, down, combine). */
NE_API int ne_moe_forward(ne_moe *m, const float *x_dev, int rows, float *y_dev, void *stream);
NE_API int ne_moe_forward_host(ne_moe *m, const float *x_host, int rows, float *y_host);
/* The same in pieces (stage numbers of the reference's ne_fn_layer_run_dispatch: 7 router, 8 gate/up, 9 down), and the
 * single kernels of stages 8 and 9 for per-kernel timing: 80 operand prep, 81 gate/up stream GEMM, 90 SwiGLU + operand
 * prep, 91 down stream GEMM, 92 combine. */
NE_API int ne_moe_stage(ne_moe *m, int stage, const float *x_dev, int rows, float *y_dev, void *stream);
/* Expert parallel: routes come from outside (route_dev: [rows][2*top_k], ids then f32 weights, global expert ids);
 * computes only the slots whose expert lies in this object's slice, summed per row in slot order, no shared expert:
 * y_partial[rows][hidden]. The caller adds the partial sums of all ranks. */
NE_API int ne_moe_forward_routed(ne_moe *m, const float *x_dev, const uint32_t *route_dev, int rows, float *y_partial_dev,
                                 void *stream);
/* Prefill: y[n][hidden] for n tokens at once (1..65535), same result definition as ne_moe_forward. Replaces the
 * reference's chunked-prefill MoE (models/flash_next/prefill.mm:235-276 record_moe; kernels/prefill/pf_moe.metal):
 * router GEMM + top-k, deterministic counting sort of the n*top_k slots by expert, per-expert grouped GEMMs whose
 * trellis tiles are decoded into shared memory once per 128 rows and multiplied on tcgen05 tensor cores with TMEM
 * accumulators, SwiGLU, slot-ordered finish. The object must hold all experts (else: ne_moe_prefill_ep); hidden and inter
 * must be multiples of 256. Scratch (about 300 KB per token) is allocated on the first call and grown when a later call brings more tokens. */
NE_API int ne_moe_prefill(ne_moe *m, const float *x_dev, int n_tokens, float *y_dev, void *stream);
/* Expert parallel, whole block (new with this library; the reference is single-device): x_all holds the rows of ALL
 * ranks, [own_row0, own_row0 + own_rows) being the caller's. Routing runs on every row (same result on every rank),
 * only the slots whose expert lies in this object's slice are computed, and the shared expert is added for the
 * caller's own rows only. y_part[rows_all][hidden] is this rank's summand: the sum over ranks is the block output. */
NE_API int ne_moe_forward_ep(ne_moe *m, const float *x_all_dev, int rows_all, int own_row0, int own_rows, float *y_part_dev,
                             void *stream);
/* Expert parallel with every row routed on its home rank only (the router's cost then does not grow with the number of
 * ranks): ne_moe_route runs the router alone on the caller's rows (routes to route_out_dev, row stride ld_route words, 0 =
 * 2*top_k; or into the object when NULL; the gate logits of the shared expert stay in the object); the ranks exchange rows
 * AND routes, then ne_moe_forward_ep_routed computes this rank's summand from the gathered rows and routes. ld_x (floats)
 * and ld_route (words) are the row strides of x_all and route_all, 0 = dense: with ld_x = ld_route = hidden + 2*top_k and
 * route_all = (uint32_t *)x_all + hidden the rows and routes travel packed side by side in ONE all-gather. */
NE_API int ne_moe_route(ne_moe *m, const float *x_dev, int rows, uint32_t *route_out_dev, int ld_route, void *stream);
NE_API int ne_moe_forward_ep_routed(ne_moe *m, const float *x_all_dev, int ld_x, const uint32_t *route_all_dev, int ld_route, int rows_all,
                                    int own_row0, int own_rows, float *y_part_dev, void *stream);
/* The same block with both exchange steps over NVLink peer memory instead of library collectives (one process per GPU
 * of one node). ne_ep_create allocates this rank's exchange buffer (gather area for world * rows_cap packed rows, part area
 * for the partial output rows peers send, flag words); every rank exports its buffer (ne_ep_handle: 64 bytes, a CUDA IPC
 * handle), the ranks exchange the handles by any means (e.g. an all-gather of bytes) and each calls ne_ep_connect with all
 * of them in rank order. ne_moe_forward_ep_fused then runs one block for `rows` own rows (the same count on every rank, all
 * ranks call in the same order): router on the own rows, packed rows written into every peer's gather area, this rank's
 * experts for all rows with the combine kernel storing each finished row into the owning rank's memory, rank-ordered sum of
 * the partial rows that arrived. All device-side waits are bounded (ne_device_wait_status). One context serves all layers. */
typedef struct ne_ep ne_ep;
NE_API ne_ep *ne_ep_create(int rank, int world, int rows_cap, int hidden, int top_k);
NE_API int ne_ep_handle(ne_ep *e, void *handle64);
NE_API int ne_ep_connect(ne_ep *e, const void *handles64 /* world x 64 bytes, rank order */);
NE_API int ne_ep_disconnect(ne_ep *e); /* closes this rank's mappings of the peers' buffers: call on every rank, barrier, then ne_ep_free */
NE_API void ne_ep_free(ne_ep *e);
NE_API int ne_moe_forward_ep_fused(ne_moe *m, ne_ep *e, const float *x_own_dev, int rows, float *y_own_dev, void *stream);
/* Expert-parallel prefill: x_all holds the tokens of ALL ranks, [own_row0, own_row0 + own_rows) being the caller's. Every
 * token is routed (same result on every rank), only the slots whose expert lies in this object's slice are sorted and
 * computed, the shared expert runs for the caller's own tokens only. y_part[n_all][hidden] is this rank's summand. */
NE_API int ne_moe_prefill_ep(ne_moe *m, const float *x_all_dev, int n_all, int own_row0, int own_rows, float *y_part_dev, void *stream);
/* Expert-parallel prefill as an all-to-all (the dispatch / combine the path's multi-GPU form names): a token is routed on
 * its home rank only, each (token, slot) pair travels to the one rank that owns its expert and its output travels back.
 *   home:   ne_moe_prefill_home    routes n tokens (router GEMM + top-k) and runs their shared expert, no routed expert:
 *                                  y_shared [n][hidden] = sigmoid(x . w_sg) * shared(x), route_out [n][2 * top_k] (ids, f32 weights)
 *           ne_ep_pairs_by_owner   stable counting sort of the n * top_k pairs by owner rank (id / experts_per_rank): packed row
 *                                  -> token (send_token) and (id, weight bits) (send_route), pair -> packed row (pos), pairs per
 *                                  rank (counts, int64: the split sizes of the exchange); experts_per_rank * world must
 *                                  cover every expert id of the route array
 *           ne_rows_gather         dst[i] = src[index[i]]: packs the pairs' activation rows in that order
 *   owner:  ne_moe_prefill_routed  n_pairs received pairs, route_pairs [n_pairs][2] = (global expert id inside this object's
 *                                  slice, f32 weight bits): y_pairs[i] = weight_i * expert_i(x_pairs[i]) through the grouped
 *                                  tensor-core GEMM (counting sort by expert as in ne_moe_prefill, one slot per row)
 *   home:   ne_slots_combine       y[t] = slot[pos[t][0]] + .. + slot[pos[t][top_k-1]] + base[t], slots in slot order, the
 *                                  shared term last: bit-identical to ne_moe_prefill on one GPU holding all experts
 * The two exchanges in between are the caller's (ijah_b200/ep.py: torch.distributed all_to_all_single over NCCL). */
NE_API int ne_moe_prefill_home(ne_moe *m, const float *x_dev, int n_tokens, float *y_shared_dev, uint32_t *route_out_dev, void *stream);
NE_API int ne_moe_prefill_routed(ne_moe *m, const float *x_pairs_dev, const uint32_t *route_pairs_dev, int n_pairs, float *y_pairs_dev, void *stream);
NE_API int ne_ep_pairs_by_owner(const uint32_t *route_dev, int n_tokens, int top_k, int experts_per_rank, int world, int *send_token_dev,
                                uint32_t *send_route_dev, int *pos_dev, long long *counts_dev, void *stream);
NE_API int ne_rows_gather(const float *src_dev, const int *index_dev, int n_out, int width, float *dst_dev, void *stream);
NE_API int ne_slots_combine(const float *slots_dev, const int *pos_dev, const float *base_dev, float *y_dev, int n_tokens, int top_k, int width,
                            void *stream);
/* Device pointer and size of a named intermediate of the last run: "logits" "route" "shared_gu" "shared_down"
 * "experts_gu_raw" (per k-split partial products [S][rows*top_k][2][inter]) "plan"; of the last ne_moe_prefill:
 * "prefill_route" [n][2*top_k] (ids, then f32 weights), "prefill_counts" [experts] slots per expert,
 * "prefill_logits" [n][experts + 1]. */
NE_API int ne_moe_buffer(ne_moe *m, const char *name, void **dev, uint64_t *nbytes);
/* Sum of k-split partials: experts_gu[rows][top_k][2][inter] f32, the raw inner products before the output Hadamard
 * (the reference's "experts_gu" buffer). */
NE_API int ne_moe_experts_gu(ne_moe *m, int rows, float *dst_host);
/* Algorithmic bytes the last forward had to read (compressed weights of the distinct experts touched + router +
 * shared expert + scales + activations), for roofline accounting. */
NE_API int ne_moe_last_bytes(ne_moe *m, int rows, uint64_t *total, uint64_t *gateup, uint64_t *down, int *distinct_experts);

/* ---- decoder stack beyond the reference's one-token step (ijah_engine.h: ne_fn_model_*) ---------------------------
 * Dimension-explicit description of a stack; ne_fn_model_create_synthetic generates every weight on the device from
 * `seed` (uniform trellis words, suh +-1, svh +-|N(0,1)| * 0.02, router / gate / head N(0, 0.02) in bf16, embedding and KV
 * cache N(0, 1)), so a full-size stack (tens of GB) needs no pack on disk. expert_first / expert_count select the experts
 * this rank holds (0, 0 = all); every other weight is replicated and identical for equal seeds. */
typedef struct {
  int layers, hidden, inter, experts, top_k, k_expert, k_shared; /* k_shared 0 = no shared expert */
  int q_out, kv_out;             /* attention projections: q hidden -> q_out, k / v hidden -> kv_out, o q_out -> hidden */
  int heads, kv_heads, head_dim; /* q_out = heads * head_dim, kv_out = kv_heads * head_dim; head_dim 64, 128 or 256 */
  int k_trunk, k_trunk_alt, alt_every; /* trunk bits per weight; every alt_every-th layer uses k_trunk_alt (0 = never) */
  int vocab, kv_positions;       /* kv_positions: cached positions the attention stand-in reads (multiple of 64) */
  int expert_first, expert_count;
  int ep_world;                  /* ranks of an expert-parallel run (0 or 1 = single GPU): the MoE blocks are sized for the rows of all ranks */
} ne_fn_model_desc;
NE_API ne_fn_model *ne_fn_model_create_synthetic(const ne_fn_model_desc *d, uint64_t seed, int max_rows);
NE_API ne_fn_model *ne_fn_model_create_rows(ne_pack *pack, int tmax, int max_rows); /* ne_fn_model_create for up to max_rows rows per step */
/* One decode step for `rows` rows (1..max_rows: concurrent sequences x verify width), one token id per row, from HOST
 * memory; logits_host f32 [rows][vocab] and next_host [rows] (greedy) may be NULL. The step is replayed from the model's
 * CUDA graph for this row count (captured on first use); host -> device copy of the tokens and device -> host copies of the
 * results are part of the call. */
NE_API int ne_fn_model_step_rows(ne_fn_model *m, const int *tokens_host, int rows, int head, float *logits_host, int *next_host, double *gpu_ms);
/* Greedy verify of one speculative round (the R = D + 1 row verify of the reference's MTP / DFlash loops,
 * models/flash_next/mtp_loop.h:5-15): tokens = [t1, d_1 .. d_D] run as ONE step of `rows` rows; drafts are accepted while
 * the model's greedy choice after tokens[j] equals tokens[j + 1]. *accepted = a, out[0 .. a] = the accepted drafts and the
 * correction / bonus token (out holds `rows` ints). Drafting and cache roll-back stay with the caller. */
NE_API int ne_fn_model_verify_greedy(ne_fn_model *m, const int *tokens, int rows, int *accepted, int *out, double *gpu_ms);
/* `steps` replays of the captured step for `rows` rows back to back on the model's stream, inputs and results staying on the
 * device: total device time between two events in *total_ms. */
NE_API int ne_fn_model_replay(ne_fn_model *m, int rows, int head, int steps, double *total_ms);
NE_API int ne_fn_model_desc_of(ne_fn_model *m, ne_fn_model_desc *out);
/* Expert parallel: the MoE blocks of every layer exchange rows over the given peer-memory context (ne_ep_*); NULL = off. */
NE_API int ne_fn_model_set_ep(ne_fn_model *m, ne_ep *e);
/* Host copy of "kv_k" / "kv_v" (f16 [kv_positions][kv_heads][head_dim] of `layer`), "hidden" (f32, final normed rows) or "logits". */
NE_API int ne_fn_model_read(ne_fn_model *m, const char *name, int layer, void *dst_host, uint64_t nbytes);
NE_API uint64_t ne_fn_model_weight_bytes(ne_fn_model *m); /* bytes of weights resident on this device */
/* Algorithmic bytes the last step of `rows` rows had to read (weights of the distinct experts touched + trunk + KV + head). */
NE_API int ne_fn_model_last_bytes(ne_fn_model *m, int rows, uint64_t *total, int *distinct_experts_mean);

/* Copy nbytes from a device pointer of this library (e.g. one returned by ne_moe_buffer) to host memory, after
 * synchronising the device. */
NE_API int ne_copy_to_host(void *dst_host, const void *src_dev, uint64_t nbytes);

/* Status word of bounded device-side waits: 0 = every wait completed. Reading it synchronises the device. */
NE_API int ne_device_wait_status(void);

#ifdef __cplusplus
}
#endif
#endif
