// 8-bit affine Linears (MLX layout, reference kernels/ne_common.h:31-43, loader models/flash_next/layer.mm:60-76): weight
// bytes row-major [rows][in], bf16 scales / biases [rows][in / group], w = scale * q + bias. In the reference these are the
// LM head and the token embedding (models/flash_next/model.mm:229-232), the hyper-connection mixes and, in packs that were
// not converted to EXL3, the trunk and shared-expert Linears.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ijah {

struct Q8Weight {
  const uint8_t *w = nullptr;        // [rows][in]
  const uint16_t *scales = nullptr;  // bf16 [rows][in / group]
  const uint16_t *biases = nullptr;
  int rows = 0, in = 0, group = 64;
};

void check_q8_weight(const Q8Weight &w);
// y[r][o] = sum_i (scale[o][i / group] * q[o][i] + bias[o][i / group]) * x[r][i]   (x, y f32; rows 1..64; one launch per 16 rows, no scratch;
// groups of 64, 128 or 256)
// `status`: the device word bounded waits report to (device_status_word())
void launch_q8_linear(const Q8Weight &w, const float *x, int rows, float *y, int *status, cudaStream_t st);
int q8_linear_launches(const Q8Weight &w, int rows);  // kernels launch_q8_linear starts for this weight and row count
inline uint64_t q8_weight_bytes(const Q8Weight &w) { return (uint64_t)w.rows * w.in + 4ull * w.rows * (w.in / w.group); }
// x[r][:] = scale * q + bias of row tokens[r] (ids outside [0, rows) read row 0), optionally rounded to bf16 as the
// reference's embedding is (kernels/fn_model.metal:14-40)
void launch_q8_embed(const Q8Weight &w, const int *tokens, int rows, float *x, bool round_bf16, cudaStream_t st);

}  // namespace ijah
