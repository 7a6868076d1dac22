// Hyper-connection read in front of the MoE block (reference models/flash_next/layer.mm:524-531, kernels fn_hc_pre /
// fn_hc_mix in kernels/fn_trunk.metal:29-165): from the HC residual streams h [rows][HC * H]
//   normed_s = h_s * rsqrt(mean(h_s^2) + eps) * norm_w_s                      per stream s of H values
//   mix      = silu(W_down . normed / HC)                                     W_down 8-bit affine [LR][HC*H]
//   inj      = 2 * sigmoid(W_inject . normed / HC)                            W_inject bf16 [HC][HC*H]
//   block_in = mean_s sigmoid(W_up[s*H + c] . mix) * normed_s[c]              W_up 8-bit affine [HC*H][LR]
// 8-bit affine (MLX layout, reference kernels/ne_common.h:31-43): bytes row-major [rows][in], bf16 scales / biases
// [rows][in / group], w = scale * q + bias. All arithmetic is f32 (the reference's default, rr() = identity).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "q8_linear.cuh"

namespace ijah {

constexpr int HC_STREAMS = 4;  // reference models/flash_next/layer.h:17-19

struct HcWeights {
  const uint16_t *norm = nullptr;    // bf16 [HC * H]
  const uint16_t *inject = nullptr;  // bf16 [HC][HC * H]
  Q8Weight down, up;                 // [LR][HC*H], [HC*H][LR]
  int H = 0, LR = 0;
};

// mix f32 [rows][LR]; inj f32 [rows][2 * HC]: the HC inject gates, then the HC per-stream 1/rms values
void launch_hc_pre(const HcWeights &w, const float *h, int rows, float *mix, float *inj, cudaStream_t st);
// out f32 [rows][H]
void launch_hc_mix(const HcWeights &w, const float *h, const float *mix, const float *inj, int rows, float *out, cudaStream_t st);
void check_hc_weights(const HcWeights &w);

}  // namespace ijah
