// C ABI, part 3: the layer object of the reference (models/flash_next/layer.h:226-268) restricted to its MoE block and the
// hyper-connection read in front of it, and the kernel-by-name entry points. Dims come from the pack's tensor shapes (the reference hard-codes 2560 / 640).
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../include/ijah_b200.h"
#include "capi_internal.hpp"
#include "hc_read.cuh"
#include "moe_object.hpp"

using namespace ijah;

namespace ijah {
constexpr int kHC = HC_STREAMS;

struct Layer {
  std::shared_ptr<Pack> pack;  // keeps the mapping alive past ne_pack_close (reference core/capi.mm:105-110)
  std::unique_ptr<Moe> moe;
  int rows = 1, H = 0, I = 0, E = 0, k = 0;
  float *mlp_in = nullptr, *mlp_out = nullptr, *h_mid = nullptr, *h_out = nullptr, *inj = nullptr, *mlp_mix = nullptr;
  bool has_hc = false;  // the pack holds this layer's mlp_hyper_connection tensors
  HcWeights hc;
  std::vector<void *> owned;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  cudaStream_t stream = nullptr;       // all of the layer's launches (a capturable stream of its own)
  cudaGraphExec_t block_graph = nullptr;  // the MoE block's six launches, captured on first use (the reference replays a
                                          // recorded command buffer per step: core/recorder.h:45-99)
  cudaGraphExec_t moe_graph() {
    if (block_graph) return block_graph;
    moe->forward(mlp_in, rows, mlp_out, stream);  // eager once: sets the kernels' attributes, surfaces launch errors
    IJ_CUDA(cudaStreamSynchronize(stream));
    cudaGraph_t g = nullptr;
    IJ_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    try {
      moe->forward(mlp_in, rows, mlp_out, stream);
    } catch (...) {
      cudaStreamEndCapture(stream, &g);
      if (g) cudaGraphDestroy(g);
      throw;
    }
    IJ_CUDA(cudaStreamEndCapture(stream, &g));
    const cudaError_t rc = cudaGraphInstantiate(&block_graph, g, 0);
    cudaGraphDestroy(g);
    IJ_CHECK(rc == cudaSuccess, "cudaGraphInstantiate: %s", cudaGetErrorString(rc));
    return block_graph;
  }
  ~Layer() {
    if (block_graph) cudaGraphExecDestroy(block_graph);
    if (stream) cudaStreamDestroy(stream);
    for (void *p : owned) cudaFree(p);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
  }
};

static ne_exl3_weight single(Pack &p, const std::string &pre, int *K) {
  const TensorInfo *t = nullptr;
  ne_exl3_weight w{};
  w.trellis_dev = p.device(pre + ".trellis", &t);
  IJ_CHECK(t->ndim == 3 && t->dtype == NE_U16 && t->shape[2] % 16 == 0, "%s.trellis: want U16 [in/16][out/16][16K]", pre.c_str());
  w.in = (int)t->shape[0] * 16; w.out = (int)t->shape[1] * 16; w.K = (int)t->shape[2] / 16;
  if (K) *K = w.K;
  const TensorInfo *s = nullptr;
  w.suh_dev = p.device(pre + ".suh", &s);
  IJ_CHECK(s->dtype == NE_F16 && (int64_t)(s->nbytes / 2) == w.in, "%s.suh: want F16 [%d]", pre.c_str(), w.in);
  w.svh_dev = p.device(pre + ".svh", &s);
  IJ_CHECK(s->dtype == NE_F16 && (int64_t)(s->nbytes / 2) == w.out, "%s.svh: want F16 [%d]", pre.c_str(), w.out);
  return w;
}

static ne_exl3_stack stack(Pack &p, const std::string &pre, int E, int in, int out, int *K) {
  const TensorInfo *t = nullptr;
  ne_exl3_stack w{};
  w.trellis_dev = p.device(pre + ".trellis", &t);
  IJ_CHECK(t->ndim == 4 && t->dtype == NE_U16 && t->shape[0] == E && t->shape[1] * 16 == in && t->shape[2] * 16 == out && t->shape[3] % 16 == 0,
           "%s.trellis: want U16 [%d][%d][%d][16K]", pre.c_str(), E, in / 16, out / 16);
  const int k = (int)t->shape[3] / 16;
  IJ_CHECK(*K == 0 || *K == k, "%s: K%d differs from the other projections (K%d)", pre.c_str(), k, *K);
  *K = k;
  const TensorInfo *s = nullptr;
  w.suh_dev = p.device(pre + ".suh", &s);
  IJ_CHECK(s->dtype == NE_F16 && (int64_t)(s->nbytes / 2) == (int64_t)E * in, "%s.suh: want F16 [%d][%d]", pre.c_str(), E, in);
  w.svh_dev = p.device(pre + ".svh", &s);
  IJ_CHECK(s->dtype == NE_F16 && (int64_t)(s->nbytes / 2) == (int64_t)E * out, "%s.svh: want F16 [%d][%d]", pre.c_str(), E, out);
  return w;
}

// 8-bit affine Linear of the pack (reference models/flash_next/layer.mm:60-76): <pre>.weight U32 [rows][in / 4],
// <pre>.scales / .biases BF16 [rows][in / group]
Q8Weight pack_q8(Pack &p, const std::string &pre) {
  const TensorInfo *t = nullptr, *s = nullptr, *b = nullptr;
  Q8Weight q;
  q.w = static_cast<const uint8_t *>(p.device(pre + ".weight", &t));
  IJ_CHECK(t->dtype == NE_U32 && t->ndim == 2, "%s.weight: want U32 [rows][in / 4]", pre.c_str());
  q.rows = (int)t->shape[0];
  q.in = (int)t->shape[1] * 4;
  q.scales = static_cast<const uint16_t *>(p.device(pre + ".scales", &s));
  q.biases = static_cast<const uint16_t *>(p.device(pre + ".biases", &b));
  IJ_CHECK(s->dtype == NE_BF16 && b->dtype == NE_BF16 && s->ndim == 2 && s->shape[0] == q.rows && s->shape[1] > 0 && q.in % s->shape[1] == 0 &&
               b->nbytes == s->nbytes, "%s.scales / .biases: want BF16 [rows][in / group]", pre.c_str());
  q.group = q.in / (int)s->shape[1];
  return q;
}

static bool load_hc(Pack &p, const std::string &pre, int H, HcWeights *out) {
  if (!p.info(pre + ".hc_norm.weight")) return false;
  const TensorInfo *t = nullptr;
  HcWeights w;
  w.H = H;
  w.norm = static_cast<const uint16_t *>(p.device(pre + ".hc_norm.weight", &t));
  IJ_CHECK(t->dtype == NE_BF16 && (int64_t)(t->nbytes / 2) == (int64_t)kHC * H, "%s.hc_norm.weight: want BF16 [%d]", pre.c_str(), kHC * H);
  w.inject = static_cast<const uint16_t *>(p.device(pre + ".block_inject_weight.weight", &t));
  IJ_CHECK(t->dtype == NE_BF16 && (int64_t)(t->nbytes / 2) == (int64_t)kHC * kHC * H, "%s.block_inject_weight.weight: want BF16 [%d][%d]", pre.c_str(), kHC, kHC * H);
  w.down = pack_q8(p, pre + ".input_mix_weight_down");
  w.up = pack_q8(p, pre + ".input_mix_weight_up");
  w.LR = w.down.rows;
  check_hc_weights(w);
  *out = w;
  return true;
}

static int config_top_k(const Pack &p) {
  try {
    const Json j = JsonParser(p.config.data(), p.config.size()).parse();
    if (const Json *v = j.get("num_experts_per_tok")) return (int)v->as_int();
    if (const Json *t = j.get("text_config"))
      if (const Json *v = t->get("num_experts_per_tok")) return (int)v->as_int();
  } catch (...) {
  }
  return 10;  // the reference's constant (kernels/fn_moe.metal:17)
}

static Layer *make_layer(ne_pack *cp, int layer, int rows) {
  auto pk = pack_from_c(cp);
  IJ_CHECK(pk != nullptr, "null pack");
  IJ_CHECK(rows >= 1 && rows <= 64, "rows %d outside 1..64", rows);
  auto L = std::make_unique<Layer>();
  L->pack = pk;
  L->rows = rows;
  const std::string pre = "language_model.model.layers." + std::to_string(layer) + ".mlp.";
  const TensorInfo *rt = pk->info(pre + "gate.weight");
  IJ_CHECK(rt && rt->dtype == NE_BF16 && rt->ndim == 2, "layer %d: %sgate.weight (BF16 [experts][hidden]) missing", layer, pre.c_str());
  ne_moe_desc d{};
  d.experts = (int)rt->shape[0];
  d.hidden = (int)rt->shape[1];
  d.top_k = config_top_k(*pk);
  d.router_dev = pk->device(pre + "gate.weight");
  const TensorInfo *gt = pk->info(pre + "switch_mlp.gate_proj.trellis");
  IJ_CHECK(gt && gt->ndim == 4, "layer %d: routed experts are not EXL3-coded (no %sswitch_mlp.gate_proj.trellis)", layer, pre.c_str());
  d.inter = (int)gt->shape[2] * 16;
  d.expert_first = 0;
  d.expert_count = d.experts;
  int K = 0;
  d.gate = stack(*pk, pre + "switch_mlp.gate_proj", d.experts, d.hidden, d.inter, &K);
  d.up = stack(*pk, pre + "switch_mlp.up_proj", d.experts, d.hidden, d.inter, &K);
  d.down = stack(*pk, pre + "switch_mlp.down_proj", d.experts, d.inter, d.hidden, &K);
  d.k_expert = K;
  if (pk->info(pre + "shared_expert_gate.weight") && pk->info(pre + "shared_expert.gate_proj.trellis")) {
    d.shared_gate_w_dev = pk->device(pre + "shared_expert_gate.weight");
    int ks = 0, k2 = 0;
    d.sh_gate = single(*pk, pre + "shared_expert.gate_proj", &ks);
    d.sh_up = single(*pk, pre + "shared_expert.up_proj", &k2);
    IJ_CHECK(ks == k2, "shared expert gate/up use different K");
    d.sh_down = single(*pk, pre + "shared_expert.down_proj", &k2);
    IJ_CHECK(ks == k2, "shared expert down uses a different K");
    IJ_CHECK(d.sh_gate.in == d.hidden && d.sh_gate.out == d.inter && d.sh_down.in == d.inter && d.sh_down.out == d.hidden, "shared expert shape mismatch");
    d.k_shared = ks;
  } else if (pk->info(pre + "shared_expert_gate.weight") && pk->info(pre + "shared_expert.gate_proj.scales")) {
    // the shared expert as three 8-bit affine Linears (packs whose trunk was not converted to EXL3)
    d.shared_gate_w_dev = pk->device(pre + "shared_expert_gate.weight");
    auto q8c = [&](const std::string &name) {
      const Q8Weight q = pack_q8(*pk, pre + "shared_expert." + name);
      return ne_q8_weight{q.w, q.scales, q.biases, q.in, q.rows, q.group};
    };
    d.sh_gate_q8 = q8c("gate_proj");
    d.sh_up_q8 = q8c("up_proj");
    d.sh_down_q8 = q8c("down_proj");
  }
  L->H = d.hidden; L->I = d.inter; L->E = d.experts; L->k = d.top_k;
  L->moe = std::make_unique<Moe>(d, rows);
  auto al = [&](size_t n) { void *p = nullptr; IJ_CUDA(cudaMalloc(&p, n)); IJ_CUDA(cudaMemset(p, 0, n)); L->owned.push_back(p); return (float *)p; };
  const size_t R = rows, H = d.hidden;
  L->mlp_in = al(R * H * 4);
  L->mlp_out = al(R * H * 4);
  L->h_mid = al(R * kHC * H * 4);
  L->h_out = al(R * kHC * H * 4);
  L->inj = al(R * 2 * kHC * 4);
  L->has_hc = load_hc(*pk, "language_model.model.layers." + std::to_string(layer) + ".mlp_hyper_connection", d.hidden, &L->hc);
  if (L->has_hc) L->mlp_mix = al(R * L->hc.LR * 4);
  L->moe->h_mid = L->h_mid; L->moe->inj = L->inj; L->moe->h_out = L->h_out; L->moe->HC = kHC;
  IJ_CUDA(cudaEventCreate(&L->ev0));
  IJ_CUDA(cudaEventCreate(&L->ev1));
  IJ_CUDA(cudaStreamCreateWithFlags(&L->stream, cudaStreamNonBlocking));
  return L.release();
}

struct Named {
  float *dev;
  size_t n;
  bool route;
};
static Named named(Layer *L, const std::string &name) {
  const size_t R = L->rows, H = L->H, I = L->I, E = L->E, k = L->k;
  Moe &m = *L->moe;
  if (name == "mlp_in") return {L->mlp_in, R * H, false};
  if (name == "mlp_out") return {L->mlp_out, R * H, false};
  if (name == "h_mid") return {L->h_mid, R * kHC * H, false};
  if (name == "h_out") return {L->h_out, R * kHC * H, false};
  if (name == "mlp_inj") return {L->inj, R * 2 * kHC, false};
  if (name == "mlp_mix" && L->has_hc) return {L->mlp_mix, R * (size_t)L->hc.LR, false};
  if (name == "logits") return {m.logits, R * (E + 1), false};
  if (name == "route") return {(float *)m.route, R * 2 * k, true};
  if (name == "shared_gu") return {m.gush, R * 2 * I, false};
  if (name == "shared_down") return {m.sho, R * H, false};
  if (name == "experts_gu") return {nullptr, R * k * 2 * I, false};
  return {nullptr, 0, false};
}
}  // namespace ijah

extern "C" {

NE_API ne_fn_layer *ne_fn_layer_create_rows(ne_pack *pack, int layer, int rows) {
  Layer *l = nullptr;
  const int rc = c_call([&] { l = make_layer(pack, layer, rows); });
  return rc == 0 ? reinterpret_cast<ne_fn_layer *>(l) : nullptr;
}
NE_API ne_fn_layer *ne_fn_layer_create(ne_pack *pack, int layer) { return ne_fn_layer_create_rows(pack, layer, 1); }
NE_API void ne_fn_layer_free(ne_fn_layer *l) { delete reinterpret_cast<Layer *>(l); }

NE_API int ne_fn_layer_step(ne_fn_layer *, const float *, float *, double *) {
  return c_call([&] {
    fail("ne_fn_layer_step: only the MLP half of the layer is implemented (ne_fn_layer_run_stage(l, 4 | 5) or "
         "ne_fn_layer_run_dispatch(l, 5..9)); the attention / GDN stages are not part of this library");
  });
}

NE_API int ne_fn_layer_run_stage(ne_fn_layer *l, int block) {
  return c_call([&] {
    Layer *L = reinterpret_cast<Layer *>(l);
    IJ_CHECK(L != nullptr, "null layer");
    IJ_CHECK(block == 4 || block == 5, "sub-block %d is not implemented (4 = MlpHC: h_mid -> mlp_mix, mlp_inj, mlp_in; 5 = Moe: mlp_in, h_mid, "
             "mlp_inj -> logits ... h_out)", block);
    if (block == 4) {  // dispatches 5 and 6 (reference models/flash_next/layer.h:262-264)
      IJ_CHECK(L->has_hc, "the pack holds no mlp_hyper_connection tensors for this layer");
      launch_hc_pre(L->hc, L->h_mid, L->rows, L->mlp_mix, L->inj, L->stream);
      launch_hc_mix(L->hc, L->h_mid, L->mlp_mix, L->inj, L->rows, L->mlp_in, L->stream);
    } else {
      IJ_CUDA(cudaGraphLaunch(L->moe_graph(), L->stream));
    }
    IJ_CUDA(cudaStreamSynchronize(L->stream));
    check_status_word();
  });
}

NE_API int ne_fn_layer_run_dispatch(ne_fn_layer *l, int stage) {
  return c_call([&] {
    Layer *L = reinterpret_cast<Layer *>(l);
    IJ_CHECK(L != nullptr, "null layer");
    IJ_CHECK(stage >= 5 && stage <= 9, "dispatch %d is not implemented (5 mlp_hc_pre, 6 mlp_hc_mix, 7 moe_router, 8 moe_gateup, 9 moe_down)", stage);
    if (stage <= 6) {
      IJ_CHECK(L->has_hc, "the pack holds no mlp_hyper_connection tensors for this layer");
      if (stage == 5) launch_hc_pre(L->hc, L->h_mid, L->rows, L->mlp_mix, L->inj, L->stream);
      else launch_hc_mix(L->hc, L->h_mid, L->mlp_mix, L->inj, L->rows, L->mlp_in, L->stream);
    } else {
      L->moe->stage(stage, L->mlp_in, L->rows, L->mlp_out, L->stream);
    }
    IJ_CUDA(cudaStreamSynchronize(L->stream));
    check_status_word();
  });
}

NE_API int ne_fn_set_ref_rounding(int on) {
  return c_call([&] { IJ_CHECK(on == 0, "reference rounding (bf16 points of the MLX goldens) is not implemented; the f32 path is"); });
}

NE_API int ne_fn_layer_write(ne_fn_layer *l, const char *name, const float *src, int n) {
  return c_call([&] {
    Layer *L = reinterpret_cast<Layer *>(l);
    IJ_CHECK(L && name && src, "null argument");
    const Named t = named(L, name);
    IJ_CHECK(t.dev != nullptr, "unknown or read-only intermediate '%s'", name);
    IJ_CHECK(n >= 0 && (size_t)n <= t.n, "%s: n %d > size %zu", name, n, t.n);
    IJ_CUDA(cudaMemcpyAsync(t.dev, src, (size_t)n * 4, cudaMemcpyHostToDevice, L->stream));
    IJ_CUDA(cudaStreamSynchronize(L->stream));
  });
}

NE_API int ne_fn_layer_read(ne_fn_layer *l, const char *name, float *dst, int n) {
  int size = -1;
  const int rc = c_call([&] {
    Layer *L = reinterpret_cast<Layer *>(l);
    IJ_CHECK(L && name, "null argument");
    const Named t = named(L, name);
    IJ_CHECK(t.n != 0, "unknown intermediate '%s'", name);
    size = (int)t.n;
    IJ_CHECK(n <= size, "%s: n %d > size %d", name, n, size);
    if (!dst || n <= 0) return;
    if (t.dev == nullptr) {  // experts_gu: k-split partials summed on the host
      std::vector<float> tmp(t.n);
      IJ_CHECK(ne_moe_experts_gu(reinterpret_cast<ne_moe *>(L->moe.get()), L->rows, tmp.data()) == 0, "%s", ne_last_error());
      memcpy(dst, tmp.data(), (size_t)n * 4);
      return;
    }
    IJ_CUDA(cudaMemcpyAsync(dst, t.dev, (size_t)n * 4, cudaMemcpyDeviceToHost, L->stream));
    IJ_CUDA(cudaStreamSynchronize(L->stream));
  });
  return rc == 0 ? size : -1;
}

// Differential timing as the reference does it (models/flash_next/layer.mm:642-681): (T(reps2) - T(reps1)) / (reps2 -
// reps1), best of 5; with flush_mb > 0 a buffer of that size is overwritten between steps (evicts L2) and its own
// differential cost is subtracted.
NE_API int ne_fn_layer_time(ne_fn_layer *l, int reps1, int reps2, int flush_mb, double *us_per_step, double *us_flush) {
  return c_call([&] {
    Layer *L = reinterpret_cast<Layer *>(l);
    IJ_CHECK(L != nullptr, "null layer");
    IJ_CHECK(reps2 > reps1 && reps1 >= 1, "bad reps %d %d", reps1, reps2);
    void *fl = nullptr;
    const size_t fb = (size_t)std::max(flush_mb, 0) << 20;
    if (fb) IJ_CUDA(cudaMalloc(&fl, fb));
    cudaGraphExec_t gx = L->moe_graph();
    auto chain = [&](int reps, bool layer, bool flush) {
      double best = 1e30;
      for (int it = 0; it < 5; it++) {
        IJ_CUDA(cudaEventRecord(L->ev0, L->stream));
        for (int i = 0; i < reps; i++) {
          if (layer) IJ_CUDA(cudaGraphLaunch(gx, L->stream));
          if (flush) IJ_CUDA(cudaMemsetAsync(fl, i & 0xFF, fb, L->stream));
        }
        IJ_CUDA(cudaEventRecord(L->ev1, L->stream));
        IJ_CUDA(cudaEventSynchronize(L->ev1));
        float ms = 0;
        IJ_CUDA(cudaEventElapsedTime(&ms, L->ev0, L->ev1));
        best = std::min(best, (double)ms);
      }
      return best;
    };
    const bool f = fb != 0;
    const double t1 = chain(reps1, true, f), t2 = chain(reps2, true, f);
    double ff = 0;
    if (f) ff = (chain(reps2, false, true) - chain(reps1, false, true)) * 1e3 / (reps2 - reps1);
    if (fl) cudaFree(fl);
    if (us_flush) *us_flush = ff;
    if (us_per_step) *us_per_step = (t2 - t1) * 1e3 / (reps2 - reps1) - ff;
    check_status_word();
  });
}

// Kernel-by-name entry (reference core/capi.mm:157-182, client tools/engine.py:392-420). The reference runs one Metal
// pipeline with caller-chosen grid and positional buffer / inline-bytes arguments. The CUDA kernels of this library are
// launched by planners that size grids, shared memory and scratch themselves, so what can be run by name are the operators:
//   "exl3_linear"   args: trellis, suh, svh, x (f32 [rows][in]), y (f32 [rows][out]) buffers, then inline u32 {in, out, K, rows}
//   "exl3_dequant"  args: trellis, w (f16 [in][out]) buffers, then inline u32 {in, out, K}
//   "q8_linear"     args: weight, scales, biases, x (f32 [rows][in]), y (f32 [rows][out]) buffers, then inline u32 {in, out, group, rows}
//                   (the reference's fn_lm_head: kernels/fn_model.metal:152-168, with the row count as an argument)
// with buffer arguments given as (ne_buf, offset) exactly as in the reference, `reps` repetitions timed on the GPU and the
// total returned in *gpu_ms; grid, threadgroup size, threadgroup memory, function constants and backend are accepted and
// ignored. The reference's Metal kernel names (fn_moe_gateup_k5_r1, t6_simd, ...) are reported absent: their argument lists
// bind the reference's Metal scratch layout (its per-row `uq` tables, split buffers and counters), which does not exist here.
static const char *kOperators[] = {"exl3_linear", "exl3_dequant", "q8_linear"};
static const char *kKernels[] = {"stream_gemm_kernel", "moe_router_kernel", "moe_prep_kernel", "moe_mid_kernel", "moe_combine_kernel",
                                 "prep_rows_kernel", "linear_finish_kernel", "dequant_kernel", "pf_gemm_kernel", "pf_logits_kernel",
                                 "pf_route_kernel", "pf_prep_kernel", "pf_mid_kernel", "pf_finish_kernel", "hc_pre_kernel", "hc_mix_kernel",
                                 "q8_linear_kernel", "q8_embed_kernel"};
NE_API int ne_kernel_exists(const char *fn) {
  if (!fn) return -1;
  for (const char *k : kOperators)
    if (strcmp(k, fn) == 0) return 1;
  for (const char *k : kKernels)
    if (strcmp(k, fn) == 0) return 1;
  return 0;
}

static void *arg_device(const ne_arg &a, const char *what) {
  IJ_CHECK(a.buf != nullptr, "%s must be a buffer argument", what);
  const uint64_t base = ne_buf_gpu_address(a.buf);
  IJ_CHECK(base != 0, "%s: %s", what, ne_last_error());
  IJ_CHECK(a.offset <= ne_buf_size(a.buf), "%s: offset beyond the buffer", what);
  return reinterpret_cast<void *>(base + a.offset);
}
static void arg_u32(const ne_arg &a, uint32_t *dst, int n, const char *what) {
  IJ_CHECK(a.buf == nullptr && a.bytes != nullptr && a.nbytes == (uint32_t)n * 4, "%s must be %d inline u32 values", what, n);
  memcpy(dst, a.bytes, (size_t)n * 4);
}

NE_API int ne_run_kernel(const char *fn, const ne_fconst *, int, const ne_arg *args, int nargs, const uint32_t[3], const uint32_t[3], uint32_t,
                         int reps, const char *, double *gpu_ms) {
  return c_call([&] {
    IJ_CHECK(fn != nullptr, "null kernel name");
    IJ_CHECK(reps >= 1 && reps <= 100000, "reps %d outside 1..100000", reps);
    const std::string name = fn;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    auto timed = [&](auto &&launch) {
      IJ_CUDA(cudaEventCreate(&e0));
      IJ_CUDA(cudaEventCreate(&e1));
      launch();  // untimed first run: first-use set-up (scratch arena, attributes)
      IJ_CUDA(cudaEventRecord(e0, 0));
      for (int i = 0; i < reps; i++) launch();
      IJ_CUDA(cudaEventRecord(e1, 0));
      IJ_CUDA(cudaEventSynchronize(e1));
      float ms = 0;
      IJ_CUDA(cudaEventElapsedTime(&ms, e0, e1));
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
      if (gpu_ms) *gpu_ms = ms;
      check_status_word();
    };
    if (name == "exl3_linear") {
      IJ_CHECK(args != nullptr && nargs == 6, "exl3_linear takes 6 arguments: trellis, suh, svh, x, y, {in, out, K, rows}");
      uint32_t d[4];
      arg_u32(args[5], d, 4, "argument 5");
      ne_exl3_weight w{arg_device(args[0], "trellis"), arg_device(args[1], "suh"), arg_device(args[2], "svh"), (int)d[0], (int)d[1], (int)d[2]};
      const float *x = (const float *)arg_device(args[3], "x");
      float *y = (float *)arg_device(args[4], "y");
      timed([&] { IJ_CHECK(ne_exl3_linear(&w, x, (int)d[3], y, nullptr) == 0, "%s", ne_last_error()); });
    } else if (name == "exl3_dequant") {
      IJ_CHECK(args != nullptr && nargs == 3, "exl3_dequant takes 3 arguments: trellis, w, {in, out, K}");
      uint32_t d[3];
      arg_u32(args[2], d, 3, "argument 2");
      ne_exl3_weight w{arg_device(args[0], "trellis"), nullptr, nullptr, (int)d[0], (int)d[1], (int)d[2]};
      void *out = arg_device(args[1], "w");
      timed([&] { IJ_CHECK(ne_exl3_dequant(&w, out, nullptr) == 0, "%s", ne_last_error()); });
    } else if (name == "q8_linear") {
      IJ_CHECK(args != nullptr && nargs == 6, "q8_linear takes 6 arguments: weight, scales, biases, x, y, {in, out, group, rows}");
      uint32_t d[4];
      arg_u32(args[5], d, 4, "argument 5");
      ne_q8_weight w{arg_device(args[0], "weight"), arg_device(args[1], "scales"), arg_device(args[2], "biases"), (int)d[0], (int)d[1], (int)d[2]};
      const float *x = (const float *)arg_device(args[3], "x");
      float *y = (float *)arg_device(args[4], "y");
      timed([&] { IJ_CHECK(ne_q8_linear(&w, x, (int)d[3], y, nullptr) == 0, "%s", ne_last_error()); });
    } else if (ne_kernel_exists(fn) == 1) {
      fail("ne_run_kernel(%s): this CUDA kernel is launched by its operator's planner (grid, shared memory and scratch are the planner's); "
           "run the operator by name instead: exl3_linear, exl3_dequant, q8_linear", fn);
    } else {
      fail("ne_run_kernel(%s): no such kernel in the CUDA build (the reference's Metal kernels bind its Metal scratch layout; operators "
           "that can be run by name: exl3_linear, exl3_dequant, q8_linear)", fn);
    }
  });
}

}  // extern "C"
