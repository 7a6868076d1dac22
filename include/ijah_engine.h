/* libijah_b200: the engine C ABI of the reference (its include/engine.h), implemented on CUDA for B200.
 *
 * Every function below has the name, argument meaning and error behaviour of the reference declaration cited beside
 * it, so the reference's ctypes client (tools/engine.py, server/backend.py) binds to this library when NE_LIB points at
 * it. Conventions (reference include/engine.h:3-13): int results are 0 / -1, pointer results NULL on error, the message
 * is in ne_last_error() per thread; pack tensor handles belong to the pack.
 *
 * What differs by construction:
 *  - Buffers are CUDA managed allocations: ne_buf_contents() is a CPU pointer to the same bytes the GPU uses, as in the
 *    reference's shared-storage model; the caller synchronises (all entry points of this library that launch work
 *    return after the work is done unless they take a stream).
 *  - A pack tensor's GPU view is a device copy made on first use (the reference maps the file without a copy); the
 *    copy is 256-byte aligned whatever the file offset is, so nothing like the reference's align-pack step is needed.
 *  - ne_run_kernel runs this library's operators by name ("exl3_linear", "exl3_dequant": argument lists at its
 *    declaration below); the reference's Metal kernel names are reported as absent, because their argument lists bind the
 *    reference's Metal scratch layout.
 */
#ifndef IJAH_ENGINE_H
#define IJAH_ENGINE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NE_API __attribute__((visibility("default")))
#define NE_ABI_VERSION 1
#define NE_MAX_DIMS 8

/* dtype codes: reference include/engine.h:27-30 (same numbers) */
enum { NE_F32 = 0, NE_F16, NE_BF16, NE_U8, NE_U16, NE_U32, NE_I32, NE_I64, NE_I8, NE_I16, NE_U64, NE_F64, NE_BOOL };

NE_API int ne_abi_version(void);             /* reference include/engine.h:33 */
NE_API const char *ne_last_error(void);      /* :34 */
NE_API const char *ne_dtype_name(int dtype); /* :35  safetensors spelling, "?" if unknown */
NE_API int ne_dtype_size(int dtype);         /* :36  bytes per element, 0 if unknown */

/* device: reference include/engine.h:39-48. has_nax reports tensor cores (1 on B200), has_metal4 is 0,
 * max_threadgroup_memory is the opt-in shared memory per CTA, backend is "cuda". */
typedef struct {
  char name[64];
  int has_nax;
  int has_metal4;
  uint64_t max_buffer_length;
  uint64_t recommended_working_set;
  uint64_t max_threadgroup_memory;
  char backend[16];
} ne_device_info;
NE_API int ne_device_query(ne_device_info *out);

/* buffers: reference include/engine.h:51-58 */
typedef struct ne_buf ne_buf;
NE_API ne_buf *ne_alloc(uint64_t nbytes);           /* zero-filled, at least 16 bytes */
NE_API void ne_free(ne_buf *b);                     /* no-op on NULL and on pack-owned handles */
NE_API uint64_t ne_buf_size(const ne_buf *b);
NE_API void *ne_buf_contents(const ne_buf *b);      /* CPU pointer (managed memory; pack tensors: the read-only file mapping) */
NE_API uint64_t ne_buf_gpu_address(const ne_buf *b);/* device pointer; makes a pack tensor resident */
NE_API int ne_upload(ne_buf *b, uint64_t offset, const void *src, uint64_t nbytes);       /* refused on pack tensors */
NE_API int ne_download(const ne_buf *b, uint64_t offset, void *dst, uint64_t nbytes);

/* packs: reference include/engine.h:61-82 (a directory of safetensors shards + model.safetensors.index.json +
 * config.json; layout read as the reference's core/pack.mm:52-246 reads it) */
typedef struct ne_pack ne_pack;
typedef struct {
  int dtype;
  int ndim;
  int64_t shape[NE_MAX_DIMS];
  uint64_t nbytes;
  const char *file;
  uint64_t file_offset;
  const void *host;
  ne_buf *buf;
  uint64_t buf_offset;
} ne_tensor_desc;

NE_API ne_pack *ne_pack_open(const char *dir);
NE_API void ne_pack_close(ne_pack *p);
NE_API const char *ne_pack_config_json(const ne_pack *p);
NE_API int64_t ne_pack_num_tensors(const ne_pack *p);
NE_API const char *ne_pack_tensor_name(const ne_pack *p, int64_t i); /* sorted by name */
NE_API int ne_tensor_info(const ne_pack *p, const char *name, ne_tensor_desc *out);
NE_API ne_buf *ne_pack_view_rows(const ne_pack *p, const char *name, int64_t row0, int64_t nrows, uint64_t *offset);

/* kernels: reference include/engine.h:85-98 */
typedef struct { uint32_t index; uint32_t type; uint32_t bits; } ne_fconst;
typedef struct { ne_buf *buf; uint64_t offset; const void *bytes; uint32_t nbytes; } ne_arg;
NE_API int ne_kernel_exists(const char *fn); /* 1 for the operators below and for the names of this library's CUDA kernels */
/* Operators that can be run by name, `reps` times, GPU milliseconds of all repetitions in *gpu_ms (fc, grid, tg, tg_mem and
 * backend are accepted and ignored: the planners size the launches):
 *   "exl3_linear"   args: trellis, suh, svh, x (f32 [rows][in]), y (f32 [rows][out]) as (buf, offset), then inline u32 {in, out, K, rows}
 *   "exl3_dequant"  args: trellis, w (f16 [in][out]) as (buf, offset), then inline u32 {in, out, K} */
NE_API int ne_run_kernel(const char *fn, const ne_fconst *fc, int nfc, const ne_arg *args, int nargs,
                         const uint32_t grid[3], const uint32_t tg[3], uint32_t tg_mem, int reps, const char *backend,
                         double *gpu_ms);

/* ---- MoE block of one decoder layer: reference models/flash_next/layer.h:226-268 ------------------------------
 * The layer object holds the MoE weights of layer `layer` of an open pack (dims come from the tensor shapes, not from
 * constants) and scratch for `rows` activation rows. Only the MoE sub-block is implemented: ne_fn_layer_run_stage
 * accepts block 5, ne_fn_layer_run_dispatch accepts 7 (router), 8 (gate/up), 9 (down + combine); ne_fn_layer_step
 * reports an error. Named buffers (all f32 on the host side): "mlp_in" [R][H] "h_mid" [R][4][H] "mlp_inj" [R][8]
 * "logits" [R][E+1] "route" [R][2k: k u32 ids, k f32 weights] "shared_gu" [R][2I] "experts_gu" [R][k][2][I]
 * "shared_down" [R][H] "mlp_out" [R][H] "h_out" [R][4][H] (names: reference models/flash_next/layer.mm:630-640). */
typedef struct ne_fn_layer ne_fn_layer;
NE_API ne_fn_layer *ne_fn_layer_create(ne_pack *pack, int layer);                 /* layer.h:229 */
NE_API ne_fn_layer *ne_fn_layer_create_rows(ne_pack *pack, int layer, int rows);  /* layer.h:232; rows 1..64 */
NE_API void ne_fn_layer_free(ne_fn_layer *l);                                     /* layer.h:233 */
NE_API int ne_fn_layer_step(ne_fn_layer *l, const float *h_in, float *h_out, double *gpu_ms); /* layer.h:244: -1 here */
NE_API int ne_fn_layer_run_stage(ne_fn_layer *l, int block);                      /* layer.h:249 */
NE_API int ne_fn_layer_run_dispatch(ne_fn_layer *l, int stage);                   /* layer.h:252 */
NE_API int ne_fn_set_ref_rounding(int on);                                        /* layer.h:255: only 0 is supported */
NE_API int ne_fn_layer_write(ne_fn_layer *l, const char *name, const float *src, int n); /* layer.h:257 */
NE_API int ne_fn_layer_read(ne_fn_layer *l, const char *name, float *dst, int n); /* layer.h:264: returns the size */
NE_API int ne_fn_layer_time(ne_fn_layer *l, int reps1, int reps2, int flush_mb, double *us_per_step, double *us_flush); /* layer.h:267 */

/* ---- whole decoder stack: reference models/flash_next/model.h:160-246 ----------------------------------------
 * The model object owns the weights of every layer (EXL3 trunk projections q, k, v, o around an attention stand-in over a
 * fixed KV cache; the MoE block), the bf16 embedding and LM head, and the decode step recorded once per row count into a
 * CUDA graph that every later step replays (the reference records into its Recorder, core/recorder.h:45-99). Attention
 * proper, GDN, hyper-connections, MTP and the sampler's knobs are not part of this library: ne_fn_model_step runs the
 * stand-in stack and samples greedily. Pack tensors read: language_model.model.embed_tokens.weight BF16 [vocab][hidden],
 * language_model.lm_head.weight (optional: tied otherwise), per layer self_attn.{q,k,v,o}_proj.{trellis,suh,svh} and the
 * mlp.* tensors of ne_fn_layer_create; config.json: num_hidden_layers, num_attention_heads, num_key_value_heads, head_dim,
 * num_experts_per_tok. */
typedef struct ne_fn_model ne_fn_model;
NE_API ne_fn_model *ne_fn_model_create(ne_pack *pack, int tmax);  /* model.h:163; tmax = cached positions (rounded up to 64) */
NE_API void ne_fn_model_free(ne_fn_model *m);                     /* model.h:168 */
NE_API int ne_fn_model_reset(ne_fn_model *m);                     /* model.h:169 */
/* model.h:204-207: one step for `token`; logits f32 [vocab], next, logprob, argmax may be NULL; head = 0: layers only */
NE_API int ne_fn_model_step(ne_fn_model *m, int token, int head, float *logits, int *next, float *logprob, int *argmax, double *gpu_ms);
/* model.h:217-218: GPU time of the full decode step: median / min over reps graph replays, wall time per synchronous step */
NE_API int ne_fn_model_time(ne_fn_model *m, int T, int reps, double *gpu_ms_median, double *gpu_ms_min, double *wall_ms_median);
NE_API int ne_fn_model_info(ne_fn_model *m, int *n_dispatch_full, int *n_dispatch_body, int *T); /* model.h:219 */
/* model.h:231: the prompt in chunks (one captured step per chunk length, at most 32 kept, least recently used dropped: as the
 * reference's chunked-prefill recordings, prefill.mm:295-345), the head on the last token: its logits f32 [vocab] / greedy token */
NE_API int ne_fn_model_prefill(ne_fn_model *m, const int *prompt, int n, float *logits, int *next, double *ms);

#ifdef __cplusplus
}
#endif
#endif
