// The glue kernels of the decoder stack around the EXL3 linears and MoE blocks: embedding lookup, RMS norm with the
// residual add, the attention stand-in over a fixed KV cache, the bf16 LM head, greedy sampling, and the generators of
// synthetic weights. None of these is on the trellis path; they exist so that a whole decode step (the reference's
// ne_fn_model_step, models/flash_next/model.h:204-207) runs inside the library and can be captured in one CUDA graph.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ijah {

// x[r][:] = float(embed[tokens[r]][:])  (embed: bf16 [vocab][H]; token ids outside [0, vocab) read row 0)
void launch_embed(const int *tokens, const uint16_t *embed_bf16, int vocab, int H, int rows, float *x, cudaStream_t st);
// x += add (if add != null); xn = x * rsqrt(mean(x^2) + eps) * (w ? float(w) : 1)   (w: bf16 [H] or null)
void launch_rms_add(float *x, const float *add, float *xn, const uint16_t *w_bf16, int rows, int H, float eps, cudaStream_t st);

// Attention stand-in for decode rows: every row attends, per query head, over the same fixed cache of T positions plus
// its own new key / value (grouped-query: heads / kv_heads query heads share one KV head):
//   out[r][h] = softmax_j( q[r][h] . k_j / sqrt(hd) ) . v_j,   j over the T cached positions and the row's own (k, v)
// q f32 [rows][heads*hd], knew / vnew f32 [rows][kv_heads*hd], kc / vc f16 [T][kv_heads][hd], out f32 [rows][heads*hd].
// Two launches: partial softmax per block of 64 positions on tensor cores (mma.sync, fp16 operands, fp32 accumulate),
// then the merge over blocks. scratch: attn_scratch_bytes(). hd must be 64, 128 or 256; T a multiple of 64.
size_t attn_scratch_bytes(int rows, int heads, int hd, int T);
void launch_attn_standin(const float *q, const float *knew, const float *vnew, const __half *kc, const __half *vc, int rows, int heads,
                         int kv_heads, int hd, int T, float *out, void *scratch, cudaStream_t st);

// logits[r][v] = sum_k bf16(xn[r][k]) * head[v][k]  (head: bf16 [vocab][H], fp32 accumulate; rows <= 64, H % 64 == 0)
void launch_lm_head(const float *xn, const uint16_t *head_bf16, int vocab, int H, int rows, float *logits, void *scratch, cudaStream_t st);
size_t lm_head_scratch_bytes(int rows, int H);
// next[r] = argmax_v logits[r][v] (lowest id on ties); scratch: rows * 2 * ARGMAX_BLOCKS * 4 bytes
constexpr int ARGMAX_BLOCKS = 64;
void launch_argmax(const float *logits, int vocab, int rows, int *next, void *scratch, cudaStream_t st);

// Synthetic weights, generated in place from a counter-based hash (the same distributions as ijah_b200/packgen.py writes).
// Element i of the destination is a function of (seed, first + i) only, so a slice of a larger tensor (the experts one
// expert-parallel rank holds) gets the values the whole tensor would have there. `first` must be a multiple of 4 for trellis words.
void fill_trellis(void *dst, size_t n_u16, uint64_t seed, cudaStream_t st, size_t first = 0);                 // uniform 16-bit words
void fill_signs_f16(void *dst, size_t n, uint64_t seed, cudaStream_t st, size_t first = 0);                   // +-1
void fill_scales_f16(void *dst, size_t n, float scale, uint64_t seed, cudaStream_t st, size_t first = 0);     // +-|N(0,1)| * scale
void fill_normal_bf16(void *dst, size_t n, float scale, uint64_t seed, cudaStream_t st, size_t first = 0);    // N(0,1) * scale
void fill_normal_f16(void *dst, size_t n, float scale, uint64_t seed, cudaStream_t st, size_t first = 0);

}  // namespace ijah
