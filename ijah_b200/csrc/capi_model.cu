// C ABI, part 4: the whole decoder stack behind the reference's model entry points (models/flash_next/model.h:160-246):
// embedding, per layer the EXL3 trunk projections around an attention stand-in and the MoE block, final norm, bf16 LM
// head, greedy sampling. The reference records its step once into a Recorder and replays it (core/recorder.h:45-99,
// models/flash_next/model.mm:472); here the step is captured once per row count into a CUDA graph owned by the model
// and replayed. Weights come from a pack (ne_fn_model_create) or are generated on the device (ne_fn_model_create_synthetic).
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/ijah_b200.h"
#include "capi_internal.hpp"
#include "exl3_linear.cuh"
#include "moe_object.hpp"
#include "q8_linear.cuh"
#include "stack.cuh"

using namespace ijah;

namespace ijah {

struct ModelLayer {
  ne_exl3_weight q{}, k{}, v{}, o{};
  Q8Weight q8[4];  // q, k, v, o as 8-bit affine Linears instead (packs whose trunk was not converted to EXL3); used when q8[0].w is set
  ne_moe_desc md{};
  std::unique_ptr<Moe> moe;
  const uint16_t *norm1 = nullptr, *norm2 = nullptr;  // bf16 [H] or null (no learned scale)
  const __half *kc = nullptr, *vc = nullptr;          // KV cache of the attention stand-in: f16 [T][kv_heads][head_dim]
};

struct Model {
  std::shared_ptr<Pack> pack;  // keeps a pack's mapping alive (null for synthetic weights)
  ne_fn_model_desc d{};
  int max_rows = 1;
  std::vector<ModelLayer> layers;
  const uint16_t *embed = nullptr, *head = nullptr, *final_norm = nullptr;
  Q8Weight embed_q8, head_q8;  // 8-bit affine embedding / LM head (the reference's pack format); used when .w is set
  std::vector<void *> owned;
  int *tokens = nullptr, *next = nullptr;
  float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *o = nullptr, *y = nullptr, *logits = nullptr;
  void *attn_scratch = nullptr, *head_scratch = nullptr, *argmax_scratch = nullptr, *lin_scratch = nullptr;
  int *status = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::map<int, cudaGraphExec_t> graphs;  // key: rows * 2 + head
  std::vector<int> graph_lru;             // keys, most recently used last; at most kMaxGraphs graphs are kept
  EpCtx *ep = nullptr;                    // expert-parallel exchange over peer memory (not owned); null = single GPU
  int launches_full = 0, launches_body = 0;
  uint64_t steps = 0;

  void *alloc(size_t n) {
    void *p = nullptr;
    IJ_CUDA(cudaMalloc(&p, std::max<size_t>(n, 256)));
    owned.push_back(p);
    return p;
  }
  ~Model() {
    for (auto &g : graphs) cudaGraphExecDestroy(g.second);
    layers.clear();
    for (void *p : owned) cudaFree(p);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    if (stream) cudaStreamDestroy(stream);
  }
  void finish_setup();
  int record(int rows, bool with_head, cudaStream_t st);
  cudaGraphExec_t graph_for(int rows, bool with_head);
  void step(const int *tokens_host, int rows, int with_head, float *logits_host, int *next_host, double *gpu_ms);
};

static void check_desc(const ne_fn_model_desc &d, int max_rows) {
  IJ_CHECK(d.layers >= 1 && d.hidden > 0 && d.vocab > 0, "bad model dims");
  IJ_CHECK(d.heads >= 1 && d.kv_heads >= 1 && d.heads % d.kv_heads == 0, "bad head counts %d / %d", d.heads, d.kv_heads);
  IJ_CHECK(d.q_out == d.heads * d.head_dim && d.kv_out == d.kv_heads * d.head_dim, "q_out / kv_out must be heads * head_dim");
  IJ_CHECK(d.kv_positions >= 64 && d.kv_positions % 64 == 0, "kv_positions %d must be a positive multiple of 64", d.kv_positions);
  IJ_CHECK(max_rows >= 1 && max_rows * std::max(1, d.ep_world) <= 64, "max_rows %d (x %d ranks) outside 1..64", max_rows, std::max(1, d.ep_world));
  IJ_CHECK(d.hidden % 256 == 0, "hidden %d must be a multiple of 256", d.hidden);
}

// activation buffers, scratch, stream; after the layers are in place
void Model::finish_setup() {
  const size_t R = max_rows, H = d.hidden, V = d.vocab;
  tokens = (int *)alloc(R * 4);
  next = (int *)alloc(R * 4);
  x = (float *)alloc(R * H * 4);
  xn = (float *)alloc(R * H * 4);
  q = (float *)alloc(R * d.q_out * 4);
  k = (float *)alloc(R * d.kv_out * 4);
  v = (float *)alloc(R * d.kv_out * 4);
  att = (float *)alloc(R * d.q_out * 4);
  o = (float *)alloc(R * H * 4);
  y = (float *)alloc(R * H * 4);
  logits = (float *)alloc(R * V * 4);
  attn_scratch = alloc(attn_scratch_bytes((int)R, d.heads, d.head_dim, d.kv_positions));
  head_scratch = alloc(lm_head_scratch_bytes((int)R, (int)H));
  argmax_scratch = alloc(R * 2 * ARGMAX_BLOCKS * 4);
  size_t lin = 0;
  for (int r = 1; r <= max_rows; r++) {  // the largest scratch any row count needs (the launch plans differ by row count)
    for (const ModelLayer &L : layers) {
      if (L.q8[0].w) continue;  // the 8-bit affine kernels need no scratch
      const int outs[3] = {L.q.out, L.k.out, L.v.out}, Ks[3] = {L.q.K, L.k.K, L.v.K};
      lin = std::max(lin, plan_linear_multi(3, L.q.in, outs, Ks, r).scratch_bytes());
      lin = std::max(lin, plan_linear(L.o.in, L.o.out, L.o.K, r).scratch_bytes());
      if (&L - layers.data() >= 4) break;  // layers repeat in shape with a short period
    }
  }
  lin_scratch = alloc(lin);
  status = device_status_word();
  IJ_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  IJ_CUDA(cudaEventCreate(&ev0));
  IJ_CUDA(cudaEventCreate(&ev1));
  IJ_CUDA(cudaMemset(tokens, 0, R * 4));
  IJ_CUDA(cudaDeviceSynchronize());
}

// Enqueue one decode step for `rows` rows on `st`; returns the number of kernel launches.
int Model::record(int rows, bool with_head, cudaStream_t st) {
  const int H = d.hidden;
  int n = 0;
  if (embed_q8.w) launch_q8_embed(embed_q8, tokens, rows, x, true, st);
  else launch_embed(tokens, embed, d.vocab, H, rows, x, st);
  n++;
  for (size_t l = 0; l < layers.size(); l++) {
    ModelLayer &L = layers[l];
    launch_rms_add(x, l == 0 ? nullptr : y, xn, L.norm1, rows, H, 1e-6f, st); n++;
    if (L.q8[0].w) {  // 8-bit affine projections: one stream kernel each
      launch_q8_linear(L.q8[0], xn, rows, q, status, st);
      launch_q8_linear(L.q8[1], xn, rows, k, status, st);
      launch_q8_linear(L.q8[2], xn, rows, v, status, st);
      for (int i = 0; i < 3; i++) n += q8_linear_launches(L.q8[i], rows);
    } else {  // q, k, v in one launch chain
      const int outs[3] = {L.q.out, L.k.out, L.v.out}, Ks[3] = {L.q.K, L.k.K, L.v.K};
      const MultiLinearPlan p = plan_linear_multi(3, L.q.in, outs, Ks, rows);
      MultiLinearArgs a{};
      const ne_exl3_weight *w[3] = {&L.q, &L.k, &L.v};
      float *ys[3] = {q, k, v};
      for (int m = 0; m < 3; m++) { a.trellis[m] = w[m]->trellis_dev; a.suh[m] = w[m]->suh_dev; a.svh[m] = w[m]->svh_dev; a.y[m] = ys[m]; }
      launch_linear_multi(p, a, xn, lin_scratch, status, st); n += 3;
    }
    launch_attn_standin(q, k, v, L.kc, L.vc, rows, d.heads, d.kv_heads, d.head_dim, d.kv_positions, att, attn_scratch, st); n += 2;
    if (L.q8[0].w) { launch_q8_linear(L.q8[3], att, rows, o, status, st); n += q8_linear_launches(L.q8[3], rows); }
    else { launch_linear(plan_linear(L.o.in, L.o.out, L.o.K, rows), L.o.trellis_dev, L.o.suh_dev, L.o.svh_dev, att, o, lin_scratch, status, st); n += 3; }
    launch_rms_add(x, o, xn, L.norm2, rows, H, 1e-6f, st); n++;
    if (ep) { L.moe->forward_ep_fused(*ep, xn, rows, y, st); n += 8; }
    else { L.moe->forward(xn, rows, y, st); n += 6 + L.moe->shared_q8_launches(rows); }
  }
  launch_rms_add(x, y, xn, final_norm, rows, H, 1e-6f, st); n++;
  launches_body = n;
  if (with_head) {
    if (head_q8.w) { launch_q8_linear(head_q8, xn, rows, logits, device_status_word(), st); n += q8_linear_launches(head_q8, rows); }
    else { launch_lm_head(xn, head, d.vocab, H, rows, logits, head_scratch, st); n += 2; }
    launch_argmax(logits, d.vocab, rows, next, argmax_scratch, st); n += 2;
    launches_full = n;
  }
  return n;
}

// One captured step per (row count, head), as the reference keeps one recording per chunk length with the least recently
// used one dropped beyond 32 (models/flash_next/prefill.mm:295-345).
constexpr size_t kMaxGraphs = 32;
cudaGraphExec_t Model::graph_for(int rows, bool with_head) {
  const int key = rows * 2 + (with_head ? 1 : 0);
  auto it = graphs.find(key);
  graph_lru.erase(std::remove(graph_lru.begin(), graph_lru.end(), key), graph_lru.end());
  graph_lru.push_back(key);
  if (it != graphs.end()) return it->second;
  if (graphs.size() >= kMaxGraphs) {
    IJ_CUDA(cudaStreamSynchronize(stream));
    const int old = graph_lru.front();
    graph_lru.erase(graph_lru.begin());
    cudaGraphExecDestroy(graphs[old]);
    graphs.erase(old);
  }
  // a first eager run outside capture: opts the kernels in to their shared-memory sizes and surfaces launch errors early
  record(rows, with_head, stream);
  IJ_CUDA(cudaStreamSynchronize(stream));
  check_status_word();
  cudaGraph_t g = nullptr;
  IJ_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
  try {
    record(rows, with_head, stream);
  } catch (...) {
    cudaStreamEndCapture(stream, &g);
    if (g) cudaGraphDestroy(g);
    throw;
  }
  IJ_CUDA(cudaStreamEndCapture(stream, &g));
  cudaGraphExec_t ex = nullptr;
  const cudaError_t rc = cudaGraphInstantiate(&ex, g, 0);
  cudaGraphDestroy(g);
  IJ_CHECK(rc == cudaSuccess, "cudaGraphInstantiate: %s", cudaGetErrorString(rc));
  graphs[key] = ex;
  return ex;
}

void Model::step(const int *tokens_host, int rows, int with_head, float *logits_host, int *next_host, double *gpu_ms) {
  IJ_CHECK(rows >= 1 && rows <= max_rows, "rows %d outside 1..%d", rows, max_rows);
  IJ_CHECK(tokens_host != nullptr, "null tokens");
  cudaGraphExec_t ex = graph_for(rows, with_head != 0);
  IJ_CUDA(cudaMemcpyAsync(tokens, tokens_host, (size_t)rows * 4, cudaMemcpyHostToDevice, stream));
  IJ_CUDA(cudaEventRecord(ev0, stream));
  IJ_CUDA(cudaGraphLaunch(ex, stream));
  IJ_CUDA(cudaEventRecord(ev1, stream));
  if (with_head && next_host) IJ_CUDA(cudaMemcpyAsync(next_host, next, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
  if (with_head && logits_host) IJ_CUDA(cudaMemcpyAsync(logits_host, logits, (size_t)rows * d.vocab * 4, cudaMemcpyDeviceToHost, stream));
  IJ_CUDA(cudaStreamSynchronize(stream));
  steps++;
  if (gpu_ms) {
    float ms = 0;
    IJ_CUDA(cudaEventElapsedTime(&ms, ev0, ev1));
    *gpu_ms = ms;
  }
}

// ------------------------------------------------------------------ weights from a pack
static int cfg_int(const Json &j, const char *key, int dflt) {
  if (const Json *v = j.get(key)) return (int)v->as_int();
  if (const Json *t = j.get("text_config"))
    if (const Json *v = t->get(key)) return (int)v->as_int();
  return dflt;
}

static ne_exl3_weight pack_linear(Pack &p, const std::string &pre) {
  const TensorInfo *t = nullptr;
  ne_exl3_weight w{};
  w.trellis_dev = p.device(pre + ".trellis", &t);
  IJ_CHECK(t->ndim == 3 && t->dtype == NE_U16 && t->shape[2] % 16 == 0, "%s.trellis: want U16 [in/16][out/16][16K]", pre.c_str());
  w.in = (int)t->shape[0] * 16; w.out = (int)t->shape[1] * 16; w.K = (int)t->shape[2] / 16;
  const TensorInfo *s = nullptr;
  w.suh_dev = p.device(pre + ".suh", &s);
  IJ_CHECK(s->dtype == NE_F16 && (int64_t)(s->nbytes / 2) == w.in, "%s.suh: want F16 [%d]", pre.c_str(), w.in);
  w.svh_dev = p.device(pre + ".svh", &s);
  IJ_CHECK(s->dtype == NE_F16 && (int64_t)(s->nbytes / 2) == w.out, "%s.svh: want F16 [%d]", pre.c_str(), w.out);
  return w;
}

static ne_exl3_stack pack_stack(Pack &p, const std::string &pre, int E, int in, int out, int *K) {
  const TensorInfo *t = nullptr;
  ne_exl3_stack w{};
  w.trellis_dev = p.device(pre + ".trellis", &t);
  IJ_CHECK(t->ndim == 4 && t->dtype == NE_U16 && t->shape[0] == E && t->shape[1] * 16 == in && t->shape[2] * 16 == out && t->shape[3] % 16 == 0,
           "%s.trellis: want U16 [%d][%d][%d][16K]", pre.c_str(), E, in / 16, out / 16);
  const int k = (int)t->shape[3] / 16;
  IJ_CHECK(*K == 0 || *K == k, "%s: K%d differs from the other projections (K%d)", pre.c_str(), k, *K);
  *K = k;
  w.suh_dev = p.device(pre + ".suh");
  w.svh_dev = p.device(pre + ".svh");
  return w;
}

static void fill_kv(Model &m, uint64_t seed) {
  const size_t per = (size_t)m.d.kv_positions * m.d.kv_out;
  for (size_t l = 0; l < m.layers.size(); l++) {
    __half *kc = (__half *)m.alloc(per * 2), *vc = (__half *)m.alloc(per * 2);
    fill_normal_f16(kc, per, 1.0f, seed + 1000 * l + 1, 0);
    fill_normal_f16(vc, per, 1.0f, seed + 1000 * l + 2, 0);
    m.layers[l].kc = kc;
    m.layers[l].vc = vc;
  }
}

static Model *model_from_pack(ne_pack *cp, int tmax, int max_rows) {
  auto pk = pack_from_c(cp);
  IJ_CHECK(pk != nullptr, "null pack");
  auto M = std::make_unique<Model>();
  M->pack = pk;
  M->max_rows = max_rows;
  const Json cfg = JsonParser(pk->config.data(), pk->config.size()).parse();
  ne_fn_model_desc &d = M->d;
  d.layers = cfg_int(cfg, "num_hidden_layers", 0);
  d.heads = cfg_int(cfg, "num_attention_heads", 0);
  d.kv_heads = cfg_int(cfg, "num_key_value_heads", 0);
  d.head_dim = cfg_int(cfg, "head_dim", 0);
  d.top_k = cfg_int(cfg, "num_experts_per_tok", 10);
  d.kv_positions = (std::max(tmax, 64) + 63) / 64 * 64;
  IJ_CHECK(d.layers >= 1 && d.heads >= 1 && d.kv_heads >= 1 && d.head_dim >= 1,
           "config.json needs num_hidden_layers, num_attention_heads, num_key_value_heads and head_dim");
  const std::string mp = "language_model.model.";
  const TensorInfo *et = pk->info(mp + "embed_tokens.weight");
  IJ_CHECK(et && et->ndim == 2, "%sembed_tokens.weight missing", mp.c_str());
  if (pk->info(mp + "embed_tokens.scales")) {  // 8-bit affine table, as the reference's packs hold it (model.mm:229-230)
    M->embed_q8 = pack_q8(*pk, mp + "embed_tokens");
    d.vocab = M->embed_q8.rows;
    d.hidden = M->embed_q8.in;
  } else {
    IJ_CHECK(et->dtype == NE_BF16, "%sembed_tokens.weight: want BF16 [vocab][hidden] or an 8-bit affine table with .scales / .biases", mp.c_str());
    d.vocab = (int)et->shape[0];
    d.hidden = (int)et->shape[1];
    M->embed = (const uint16_t *)pk->device(mp + "embed_tokens.weight");
  }
  const TensorInfo *ht = pk->info("language_model.lm_head.weight");
  if (ht && pk->info("language_model.lm_head.scales")) {  // 8-bit affine head (model.mm:231-232)
    M->head_q8 = pack_q8(*pk, "language_model.lm_head");
    IJ_CHECK(M->head_q8.rows == d.vocab && M->head_q8.in == d.hidden, "lm_head: want [%d][%d]", d.vocab, d.hidden);
  } else if (ht) {
    IJ_CHECK(ht->dtype == NE_BF16 && ht->ndim == 2 && ht->shape[0] == d.vocab && ht->shape[1] == d.hidden, "lm_head.weight: want BF16 [%d][%d]", d.vocab, d.hidden);
    M->head = (const uint16_t *)pk->device("language_model.lm_head.weight");
  } else if (M->embed_q8.w) {
    M->head_q8 = M->embed_q8;  // tied
  } else {
    M->head = M->embed;  // tied
  }
  if (pk->info(mp + "norm.weight")) M->final_norm = (const uint16_t *)pk->device(mp + "norm.weight");
  M->layers.resize(d.layers);
  for (int l = 0; l < d.layers; l++) {
    ModelLayer &L = M->layers[l];
    const std::string pre = mp + "layers." + std::to_string(l) + ".";
    int q_out = 0, kv_out = 0;
    if (pk->info(pre + "self_attn.q_proj.scales")) {  // 8-bit affine projections
      const char *names[4] = {"q_proj", "k_proj", "v_proj", "o_proj"};
      for (int i = 0; i < 4; i++) L.q8[i] = pack_q8(*pk, pre + "self_attn." + names[i]);
      IJ_CHECK(L.q8[0].in == d.hidden && L.q8[1].in == d.hidden && L.q8[2].in == d.hidden && L.q8[3].rows == d.hidden && L.q8[3].in == L.q8[0].rows &&
                   L.q8[1].rows == L.q8[2].rows, "layer %d: attention projection shapes do not fit hidden %d", l, d.hidden);
      q_out = L.q8[0].rows; kv_out = L.q8[1].rows;
      if (l == 0) d.k_trunk = 8;
    } else {
      L.q = pack_linear(*pk, pre + "self_attn.q_proj");
      L.k = pack_linear(*pk, pre + "self_attn.k_proj");
      L.v = pack_linear(*pk, pre + "self_attn.v_proj");
      L.o = pack_linear(*pk, pre + "self_attn.o_proj");
      IJ_CHECK(L.q.in == d.hidden && L.k.in == d.hidden && L.v.in == d.hidden && L.o.out == d.hidden && L.o.in == L.q.out && L.k.out == L.v.out,
               "layer %d: attention projection shapes do not fit hidden %d", l, d.hidden);
      q_out = L.q.out; kv_out = L.k.out;
      if (l == 0) d.k_trunk = L.q.K;
    }
    if (l == 0) { d.q_out = q_out; d.kv_out = kv_out; }
    IJ_CHECK(q_out == d.q_out && kv_out == d.kv_out, "layer %d: attention widths differ from layer 0", l);
    if (pk->info(pre + "input_layernorm.weight")) L.norm1 = (const uint16_t *)pk->device(pre + "input_layernorm.weight");
    if (pk->info(pre + "post_attention_layernorm.weight")) L.norm2 = (const uint16_t *)pk->device(pre + "post_attention_layernorm.weight");
    ne_moe_desc &md = L.md;
    const TensorInfo *rt = pk->info(pre + "mlp.gate.weight");
    IJ_CHECK(rt && rt->dtype == NE_BF16 && rt->ndim == 2 && rt->shape[1] == d.hidden, "layer %d: %smlp.gate.weight (BF16 [experts][hidden]) missing", l, pre.c_str());
    md.experts = (int)rt->shape[0]; md.hidden = d.hidden; md.top_k = d.top_k;
    md.router_dev = pk->device(pre + "mlp.gate.weight");
    const TensorInfo *gt = pk->info(pre + "mlp.switch_mlp.gate_proj.trellis");
    IJ_CHECK(gt && gt->ndim == 4, "layer %d: routed experts are not EXL3-coded", l);
    md.inter = (int)gt->shape[2] * 16;
    md.expert_first = 0; md.expert_count = md.experts;
    int K = 0;
    md.gate = pack_stack(*pk, pre + "mlp.switch_mlp.gate_proj", md.experts, md.hidden, md.inter, &K);
    md.up = pack_stack(*pk, pre + "mlp.switch_mlp.up_proj", md.experts, md.hidden, md.inter, &K);
    md.down = pack_stack(*pk, pre + "mlp.switch_mlp.down_proj", md.experts, md.inter, md.hidden, &K);
    md.k_expert = K;
    if (pk->info(pre + "mlp.shared_expert_gate.weight") && pk->info(pre + "mlp.shared_expert.gate_proj.trellis")) {
      md.shared_gate_w_dev = pk->device(pre + "mlp.shared_expert_gate.weight");
      md.sh_gate = pack_linear(*pk, pre + "mlp.shared_expert.gate_proj");
      md.sh_up = pack_linear(*pk, pre + "mlp.shared_expert.up_proj");
      md.sh_down = pack_linear(*pk, pre + "mlp.shared_expert.down_proj");
      md.k_shared = md.sh_gate.K;
    } else if (pk->info(pre + "mlp.shared_expert_gate.weight") && pk->info(pre + "mlp.shared_expert.gate_proj.scales")) {
      md.shared_gate_w_dev = pk->device(pre + "mlp.shared_expert_gate.weight");
      auto q8c = [&](const char *name) {
        const Q8Weight q = pack_q8(*pk, pre + "mlp.shared_expert." + name);
        return ne_q8_weight{q.w, q.scales, q.biases, q.in, q.rows, q.group};
      };
      md.sh_gate_q8 = q8c("gate_proj");
      md.sh_up_q8 = q8c("up_proj");
      md.sh_down_q8 = q8c("down_proj");
      md.k_shared = 8;
    }
    if (l == 0) { d.inter = md.inter; d.experts = md.experts; d.k_expert = md.k_expert; d.k_shared = md.k_shared; d.expert_count = md.experts; }
    L.moe = std::make_unique<Moe>(md, max_rows);
  }
  check_desc(d, max_rows);
  fill_kv(*M, 0xC0FFEEull);
  M->finish_setup();
  return M.release();
}

// ------------------------------------------------------------------ synthetic weights generated on the device
static ne_exl3_weight synth_linear(Model &m, int in, int out, int K, uint64_t seed) {
  ne_exl3_weight w{};
  const size_t nt = (size_t)in * out * K / 16;  // u16 words
  void *tr = m.alloc(nt * 2), *su = m.alloc((size_t)in * 2), *sv = m.alloc((size_t)out * 2);
  fill_trellis(tr, nt, seed, 0);
  fill_signs_f16(su, in, seed + 1, 0);
  fill_scales_f16(sv, out, 0.02f, seed + 2, 0);
  w.trellis_dev = tr; w.suh_dev = su; w.svh_dev = sv; w.in = in; w.out = out; w.K = K;
  return w;
}
// experts [first, first + count) of a stack: the same values whatever slice a rank holds
static ne_exl3_stack synth_stack(Model &m, int first, int count, int in, int out, int K, uint64_t seed) {
  ne_exl3_stack w{};
  const size_t per = (size_t)in * out * K / 16, nt = (size_t)count * per;
  void *tr = m.alloc(nt * 2), *su = m.alloc((size_t)count * in * 2), *sv = m.alloc((size_t)count * out * 2);
  fill_trellis(tr, nt, seed, 0, (size_t)first * per);
  fill_signs_f16(su, (size_t)count * in, seed + 1, 0, (size_t)first * in);
  fill_scales_f16(sv, (size_t)count * out, 0.02f, seed + 2, 0, (size_t)first * out);
  w.trellis_dev = tr; w.suh_dev = su; w.svh_dev = sv;
  return w;
}

static Model *model_synthetic(const ne_fn_model_desc &din, uint64_t seed, int max_rows) {
  ne_fn_model_desc d = din;
  if (d.expert_count <= 0) { d.expert_first = 0; d.expert_count = d.experts; }
  check_desc(d, max_rows);
  IJ_CHECK(d.experts >= 1 && d.top_k >= 1 && d.inter > 0 && d.expert_first >= 0 && d.expert_first + d.expert_count <= d.experts, "bad MoE dims");
  auto M = std::make_unique<Model>();
  M->d = d;
  M->max_rows = max_rows;
  const size_t H = d.hidden, V = d.vocab;
  uint16_t *emb = (uint16_t *)M->alloc(V * H * 2), *head = (uint16_t *)M->alloc(V * H * 2);
  fill_normal_bf16(emb, V * H, 1.0f, seed + 11, 0);
  fill_normal_bf16(head, V * H, 0.02f, seed + 12, 0);
  M->embed = emb; M->head = head;
  M->layers.resize(d.layers);
  for (int l = 0; l < d.layers; l++) {
    ModelLayer &L = M->layers[l];
    const uint64_t ls = seed + 100003ull * (l + 1);  // replicated weights: the same on every rank
    const int Kt = (d.alt_every > 0 && d.k_trunk_alt > 0 && l % d.alt_every == d.alt_every - 1) ? d.k_trunk_alt : d.k_trunk;
    L.q = synth_linear(*M, d.hidden, d.q_out, Kt, ls + 1);
    L.k = synth_linear(*M, d.hidden, d.kv_out, Kt, ls + 4);
    L.v = synth_linear(*M, d.hidden, d.kv_out, Kt, ls + 7);
    L.o = synth_linear(*M, d.q_out, d.hidden, Kt, ls + 10);
    ne_moe_desc &md = L.md;
    md.hidden = d.hidden; md.inter = d.inter; md.experts = d.experts; md.top_k = d.top_k; md.k_expert = d.k_expert; md.k_shared = d.k_shared;
    md.expert_first = d.expert_first; md.expert_count = d.expert_count;
    uint16_t *router = (uint16_t *)M->alloc((size_t)d.experts * H * 2);
    fill_normal_bf16(router, (size_t)d.experts * H, 0.02f, ls + 20, 0);
    md.router_dev = router;
    md.gate = synth_stack(*M, d.expert_first, d.expert_count, d.hidden, d.inter, d.k_expert, ls + 30);
    md.up = synth_stack(*M, d.expert_first, d.expert_count, d.hidden, d.inter, d.k_expert, ls + 33);
    md.down = synth_stack(*M, d.expert_first, d.expert_count, d.inter, d.hidden, d.k_expert, ls + 36);
    if (d.k_shared > 0) {
      uint16_t *sg = (uint16_t *)M->alloc(H * 2);
      fill_normal_bf16(sg, H, 0.02f, ls + 40, 0);
      md.shared_gate_w_dev = sg;
      md.sh_gate = synth_linear(*M, d.hidden, d.inter, d.k_shared, ls + 41);
      md.sh_up = synth_linear(*M, d.hidden, d.inter, d.k_shared, ls + 44);
      md.sh_down = synth_linear(*M, d.inter, d.hidden, d.k_shared, ls + 47);
    }
    L.moe = std::make_unique<Moe>(md, max_rows * std::max(1, d.ep_world));  // expert parallel: the block sees the rows of all ranks
  }
  fill_kv(*M, seed + 5);
  M->finish_setup();
  return M.release();
}

}  // namespace ijah

extern "C" {

NE_API ne_fn_model *ne_fn_model_create(ne_pack *pack, int tmax) {
  Model *m = nullptr;
  const int rc = c_call([&] { m = model_from_pack(pack, tmax, 8); });
  return rc == 0 ? reinterpret_cast<ne_fn_model *>(m) : nullptr;
}
NE_API ne_fn_model *ne_fn_model_create_rows(ne_pack *pack, int tmax, int max_rows) {
  Model *m = nullptr;
  const int rc = c_call([&] { m = model_from_pack(pack, tmax, max_rows); });
  return rc == 0 ? reinterpret_cast<ne_fn_model *>(m) : nullptr;
}
NE_API ne_fn_model *ne_fn_model_create_synthetic(const ne_fn_model_desc *d, uint64_t seed, int max_rows) {
  Model *m = nullptr;
  const int rc = c_call([&] {
    IJ_CHECK(d != nullptr, "null ne_fn_model_desc");
    m = model_synthetic(*d, seed, max_rows);
  });
  return rc == 0 ? reinterpret_cast<ne_fn_model *>(m) : nullptr;
}
NE_API void ne_fn_model_free(ne_fn_model *m) {
  if (!m) return;
  cudaDeviceSynchronize();
  delete reinterpret_cast<Model *>(m);
}
NE_API int ne_fn_model_reset(ne_fn_model *m) {
  return c_call([&] {
    IJ_CHECK(m != nullptr, "null model");
    reinterpret_cast<Model *>(m)->steps = 0;  // the stand-in cache is fixed: there is no position state to rewind
  });
}
NE_API int ne_fn_model_step(ne_fn_model *m, int token, int head, float *logits, int *next, float *logprob, int *argmax, double *gpu_ms) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr, "null model");
    int nx = 0;
    M->step(&token, 1, head, logits, &nx, gpu_ms);
    check_status_word();
    if (head) {
      if (next) *next = nx;
      if (argmax) *argmax = nx;
      if (logprob) {  // log-probability of the greedy token at temperature 1 over the full vocabulary
        std::vector<float> lg;
        const float *src = logits;
        if (!src) {
          lg.resize(M->d.vocab);
          IJ_CUDA(cudaMemcpy(lg.data(), M->logits, (size_t)M->d.vocab * 4, cudaMemcpyDeviceToHost));
          src = lg.data();
        }
        double mx = src[nx], sum = 0;
        for (int i = 0; i < M->d.vocab; i++) sum += std::exp((double)src[i] - mx);
        *logprob = (float)(-std::log(sum));
      }
    }
  });
}
NE_API int ne_fn_model_step_rows(ne_fn_model *m, const int *tokens_host, int rows, int head, float *logits_host, int *next_host, double *gpu_ms) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr, "null model");
    M->step(tokens_host, rows, head, logits_host, next_host, gpu_ms);
  });
}
// Prompt prefill (reference models/flash_next/model.h:231): the prompt goes through the stack in chunks of up to max_rows
// rows, each chunk replayed from the graph of its length (captured on first use, least recently used dropped beyond 32);
// the head runs on the last chunk only and the last token's logits / greedy token are returned. The attention stand-in
// keeps no per-token state, so unlike the reference nothing is appended to a cache.
NE_API int ne_fn_model_prefill(ne_fn_model *m, const int *prompt, int n, float *logits, int *next, double *ms) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr && prompt != nullptr && n >= 1, "bad arguments");
    const auto t0 = std::chrono::steady_clock::now();
    std::vector<int> nx(M->max_rows);
    std::vector<float> lg;
    for (int i = 0; i < n; i += M->max_rows) {
      const int rows = std::min(M->max_rows, n - i);
      const bool last = i + rows >= n;
      if (last && logits) lg.resize((size_t)rows * M->d.vocab);
      M->step(prompt + i, rows, last ? 1 : 0, last && logits ? lg.data() : nullptr, last ? nx.data() : nullptr, nullptr);
      if (last) {
        if (next) *next = nx[rows - 1];
        if (logits) memcpy(logits, lg.data() + (size_t)(rows - 1) * M->d.vocab, (size_t)M->d.vocab * 4);
      }
    }
    check_status_word();
    if (ms) *ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  });
}
// Greedy verify of one speculative round (reference models/flash_next/mtp_loop.h:5-15): rows = [t1, d_1 .. d_D] (the last
// emitted token and D drafted ones, R = D + 1 <= max_rows) go through ONE R-row step; row j's greedy token is the model's
// choice after tokens[j], so the drafts are accepted while tokens[j + 1] equals it. *accepted = a (0..D), out[0 .. a] =
// the accepted drafts followed by the correction (a < D) or bonus (a = D) token, as the reference emits them. Drafting
// (the MTP head) and the cache roll-back of rejected rows are the caller's; the attention stand-in keeps no per-token state.
NE_API int ne_fn_model_verify_greedy(ne_fn_model *m, const int *tokens, int rows, int *accepted, int *out, double *gpu_ms) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr && tokens != nullptr && accepted != nullptr && out != nullptr, "null argument");
    IJ_CHECK(rows >= 1 && rows <= M->max_rows, "rows %d outside 1..%d", rows, M->max_rows);
    std::vector<int> nx(rows);
    M->step(tokens, rows, 1, nullptr, nx.data(), gpu_ms);
    check_status_word();
    int a = 0;
    while (a < rows - 1 && tokens[a + 1] == nx[a]) a++;
    for (int j = 0; j < a; j++) out[j] = tokens[j + 1];
    out[a] = nx[a];
    *accepted = a;
  });
}
NE_API int ne_fn_model_replay(ne_fn_model *m, int rows, int head, int steps, double *total_ms) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr && steps >= 1, "bad arguments");
    IJ_CHECK(rows >= 1 && rows <= M->max_rows, "rows %d outside 1..%d", rows, M->max_rows);
    cudaGraphExec_t ex = M->graph_for(rows, head != 0);
    IJ_CUDA(cudaStreamSynchronize(M->stream));
    IJ_CUDA(cudaEventRecord(M->ev0, M->stream));
    for (int i = 0; i < steps; i++) IJ_CUDA(cudaGraphLaunch(ex, M->stream));
    IJ_CUDA(cudaEventRecord(M->ev1, M->stream));
    IJ_CUDA(cudaStreamSynchronize(M->stream));
    float ms = 0;
    IJ_CUDA(cudaEventElapsedTime(&ms, M->ev0, M->ev1));
    if (total_ms) *total_ms = ms;
    M->steps += steps;
  });
}
NE_API int ne_fn_model_time(ne_fn_model *m, int T, int reps, double *gpu_ms_median, double *gpu_ms_min, double *wall_ms_median) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr && reps >= 1, "bad arguments");
    (void)T;  // the stand-in attention always reads the whole fixed cache
    std::vector<double> g(reps), w(reps);
    int tok = 1, nx = 0;
    M->step(&tok, 1, 1, nullptr, &nx, nullptr);
    for (int i = 0; i < reps; i++) {
      const auto t0 = std::chrono::steady_clock::now();
      M->step(&tok, 1, 1, nullptr, &nx, &g[i]);
      w[i] = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    }
    std::sort(g.begin(), g.end());
    std::sort(w.begin(), w.end());
    if (gpu_ms_median) *gpu_ms_median = g[reps / 2];
    if (gpu_ms_min) *gpu_ms_min = g[0];
    if (wall_ms_median) *wall_ms_median = w[reps / 2];
    check_status_word();
  });
}
NE_API int ne_fn_model_info(ne_fn_model *m, int *n_dispatch_full, int *n_dispatch_body, int *T) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr, "null model");
    if (M->launches_full == 0) M->graph_for(1, true);
    if (n_dispatch_full) *n_dispatch_full = M->launches_full;
    if (n_dispatch_body) *n_dispatch_body = M->launches_body;
    if (T) *T = M->d.kv_positions;
  });
}
NE_API int ne_fn_model_desc_of(ne_fn_model *m, ne_fn_model_desc *out) {
  return c_call([&] {
    IJ_CHECK(m && out, "null argument");
    *out = reinterpret_cast<Model *>(m)->d;
  });
}
NE_API int ne_fn_model_set_ep(ne_fn_model *m, ne_ep *e) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr, "null model");
    IJ_CHECK(M->graphs.empty(), "set the exchange context before the first step (the captured steps hold the single-GPU blocks)");
    M->ep = reinterpret_cast<EpCtx *>(e);
  });
}
NE_API int ne_fn_model_read(ne_fn_model *m, const char *name, int layer, void *dst_host, uint64_t nbytes) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M && name && dst_host, "null argument");
    const std::string n = name;
    const void *src = nullptr;
    size_t have = 0;
    const size_t kv = (size_t)M->d.kv_positions * M->d.kv_out * 2;
    if (n == "kv_k" || n == "kv_v") {
      IJ_CHECK(layer >= 0 && layer < (int)M->layers.size(), "layer %d outside the model", layer);
      src = n == "kv_k" ? (const void *)M->layers[layer].kc : (const void *)M->layers[layer].vc;
      have = kv;
    } else if (n == "hidden") { src = M->xn; have = (size_t)M->max_rows * M->d.hidden * 4; }
    else if (n == "logits") { src = M->logits; have = (size_t)M->max_rows * M->d.vocab * 4; }
    else fail("unknown model buffer '%s' (kv_k, kv_v, hidden, logits)", name);
    IJ_CHECK(nbytes <= have, "%s: %llu bytes asked, %zu held", name, (unsigned long long)nbytes, have);
    IJ_CUDA(cudaDeviceSynchronize());
    IJ_CUDA(cudaMemcpy(dst_host, src, nbytes, cudaMemcpyDeviceToHost));
  });
}
NE_API uint64_t ne_fn_model_weight_bytes(ne_fn_model *m) {
  Model *M = reinterpret_cast<Model *>(m);
  if (!M) return 0;
  auto lin = [](const ne_exl3_weight &w) { return (uint64_t)w.in * w.out * w.K / 8 + 2ull * w.in + 2ull * w.out; };
  auto q8b = [](const Q8Weight &w) { return q8_weight_bytes(w); };
  auto q8c = [](const ne_q8_weight &w) { return (uint64_t)w.out * w.in + 4ull * w.out * (w.in / w.group); };
  uint64_t b = 0;
  if (M->embed_q8.w) b += q8b(M->embed_q8); else b += 2ull * M->d.vocab * M->d.hidden;
  if (M->head_q8.w) b += M->head_q8.w == M->embed_q8.w ? 0 : q8b(M->head_q8);
  else if (M->head != M->embed) b += 2ull * M->d.vocab * M->d.hidden;
  for (const ModelLayer &L : M->layers) {
    if (L.q8[0].w) for (const Q8Weight &w : L.q8) b += q8b(w);
    else b += lin(L.q) + lin(L.k) + lin(L.v) + lin(L.o);
    b += 2ull * L.md.experts * L.md.hidden;
    b += 3ull * L.md.expert_count * ((uint64_t)L.md.hidden * L.md.inter * L.md.k_expert / 8 + 2ull * L.md.hidden + 2ull * L.md.inter);
    if (L.md.shared_gate_w_dev && L.md.sh_gate_q8.weight_dev) b += q8c(L.md.sh_gate_q8) + q8c(L.md.sh_up_q8) + q8c(L.md.sh_down_q8) + 2ull * L.md.hidden;
    else if (L.md.shared_gate_w_dev) b += lin(L.md.sh_gate) + lin(L.md.sh_up) + lin(L.md.sh_down) + 2ull * L.md.hidden;
  }
  return b;
}
// algorithmic bytes one step of `rows` rows had to read (the last step's distinct experts), for roofline accounting
NE_API int ne_fn_model_last_bytes(ne_fn_model *m, int rows, uint64_t *total, int *distinct_experts_mean) {
  return c_call([&] {
    Model *M = reinterpret_cast<Model *>(m);
    IJ_CHECK(M != nullptr, "null model");
    auto lin = [](const ne_exl3_weight &w) { return (uint64_t)w.in * w.out * w.K / 8 + 2ull * w.in + 2ull * w.out; };
    uint64_t b = (M->head_q8.w ? (uint64_t)M->head_q8.rows * M->head_q8.in + 4ull * M->head_q8.rows * (M->head_q8.in / M->head_q8.group)
                               : 2ull * M->d.vocab * M->d.hidden) + (uint64_t)rows * M->d.hidden * 2;
    long nu = 0;
    for (ModelLayer &L : M->layers) {
      uint64_t t = 0;
      int n = 0;
      IJ_CHECK(ne_moe_last_bytes(reinterpret_cast<ne_moe *>(L.moe.get()), rows * std::max(1, M->d.ep_world), &t, nullptr, nullptr, &n) == 0, "%s", ne_last_error());
      if (L.q8[0].w) for (const Q8Weight &w : L.q8) b += q8_weight_bytes(w);
      else b += lin(L.q) + lin(L.k) + lin(L.v) + lin(L.o);
      b += t + 2ull * (uint64_t)M->d.kv_positions * M->d.kv_out * 2;
      nu += n;
    }
    if (total) *total = b;
    if (distinct_experts_mean) *distinct_experts_mean = (int)(nu / (long)M->layers.size());
  });
}

}  // extern "C"
