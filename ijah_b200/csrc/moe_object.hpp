// The object behind ne_moe: weights description, scratch, per-row-count launch plans.
#pragma once
#include <map>
#include <vector>

#include "../../include/ijah_b200.h"
#include <cuda_fp16.h>

#include "fn_moe.cuh"
#include "pf_moe.cuh"

namespace ijah {

struct Moe {
  ne_moe_desc desc;
  int max_rows;
  bool has_shared = false;
  bool shared_q8 = false;  // the shared expert is three 8-bit affine Linears (decode-width single-GPU calls only)
  float *q8_g = nullptr, *q8_u = nullptr, *q8_act = nullptr;
  void shared_q8_run(const float *x, int rows, cudaStream_t st);  // sho = down(silu(gate x) * up x); gush = gate | up
  int shared_q8_launches(int rows) const;                         // kernels shared_q8_run starts (0 without such an expert)
  int last_rows = 1;
  std::vector<void *> owned;
  float *logits = nullptr, *raw_gu = nullptr, *raw_sgu = nullptr, *raw_d = nullptr, *raw_sd = nullptr, *gush = nullptr, *sho = nullptr;
  float *x_stage = nullptr, *y_stage = nullptr;
  __half *xh_gu = nullptr, *xh_sgu = nullptr, *xh_d = nullptr, *xh_sd = nullptr;
  int max_S_gu = 1, max_S_d = 1;
  uint32_t *route = nullptr;
  int *plan = nullptr, *status = nullptr;
  unsigned *counter = nullptr;
  // optional hyper-connection write (set by the layer object)
  const float *h_mid = nullptr, *inj = nullptr;
  float *h_out = nullptr;
  int HC = 0;
  std::map<int, MoeSplits> split_cache;
  MoeMaps maps{};  // tensor maps over the trellis stacks
  // prefill scratch, (re)allocated when a call brings more tokens than any before it
  PfParams pf{};
  int pf_tokens = 0, pf_slots = 0, pf_last_n = 0;  // scratch capacity in tokens and in (token, slot) pairs
  std::vector<void *> pf_owned;
  enum { PF_ALL = 0, PF_HOME = 1, PF_ROUTED = 2 };
  void prefill(const float *x, int n, int own_row0, int own_rows, float *y, cudaStream_t st, int mode = PF_ALL, const uint32_t *route_in = nullptr);

  Moe(const ne_moe_desc &d, int max_rows);
  ~Moe();
  Moe(const Moe &) = delete;
  MoeParams params(const float *x, int rows, float *y);
  const MoeSplits &splits(int rows);
  void stage(int stage_no, const float *x, int rows, float *y, cudaStream_t st);
  void forward(const float *x, int rows, float *y, cudaStream_t st);
  void forward_ep(const float *x, int rows, int own_row0, int own_rows, float *y, cudaStream_t st);
  void forward_routed(const float *x, const uint32_t *route_in, int rows, float *y, cudaStream_t st);
  void forward_ep_fused(EpCtx &c, const float *x_own, int rows, float *y_own, cudaStream_t st);
  void route_rows(const float *x, int rows, uint32_t *route_out, int ld_route, cudaStream_t st);
  void forward_ep_routed(const float *x, int ld_x, const uint32_t *route_all, int ld_route, int rows, int own_row0, int own_rows, float *y,
                         cudaStream_t st);
};

}  // namespace ijah
