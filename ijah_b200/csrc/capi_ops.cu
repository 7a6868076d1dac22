// C ABI, part 2: the dimension-explicit operators (include/ijah_b200.h): EXL3 Linear, dequant, MoE block.
#include <cstring>
#include <memory>
#include <vector>

#include "../../include/ijah_b200.h"
#include "capi_internal.hpp"
#include "fn_moe.cuh"
#include "moe_object.hpp"
#include "q8_linear.cuh"

using namespace ijah;

namespace ijah {

static void check_weight(const ne_exl3_weight *w) {
  IJ_CHECK(w && w->trellis_dev && w->suh_dev && w->svh_dev, "null EXL3 weight pointer");
  IJ_CHECK(((uintptr_t)w->trellis_dev & 15) == 0, "trellis must be 16-byte aligned on the device");
}

// ------------------------------------------------------------------ MoE object
Moe::Moe(const ne_moe_desc &d, int max_rows_) : desc(d), max_rows(max_rows_) {
  IJ_CHECK(d.hidden > 0 && d.inter > 0 && d.experts > 0 && d.top_k > 0 && d.top_k <= d.experts, "bad MoE dims");
  IJ_CHECK(d.expert_first >= 0 && d.expert_count >= 0 && d.expert_first + d.expert_count <= d.experts, "bad expert slice");
  IJ_CHECK(d.router_dev != nullptr, "null router weights");
  IJ_CHECK(d.expert_count == 0 || (d.gate.trellis_dev && d.up.trellis_dev && d.down.trellis_dev), "null expert weights");
  has_shared = d.shared_gate_w_dev != nullptr && d.sh_gate.trellis_dev != nullptr;
  shared_q8 = d.shared_gate_w_dev != nullptr && !has_shared && d.sh_gate_q8.weight_dev != nullptr;
  if (shared_q8) {
    IJ_CHECK(d.sh_up_q8.weight_dev && d.sh_down_q8.weight_dev, "null 8-bit shared-expert weights");
    IJ_CHECK(d.sh_gate_q8.in == d.hidden && d.sh_gate_q8.out == d.inter && d.sh_up_q8.in == d.hidden && d.sh_up_q8.out == d.inter &&
                 d.sh_down_q8.in == d.inter && d.sh_down_q8.out == d.hidden, "8-bit shared expert shape mismatch");
  }
  // the router reads its rows (and the shared gate) with 16-byte loads; the trellis stacks are checked where their tensor
  // maps are made
  IJ_CHECK(((uintptr_t)d.router_dev & 15) == 0 && ((uintptr_t)d.shared_gate_w_dev & 15) == 0, "router / shared-gate weights must be 16-byte aligned");
  for (int r = 1; r <= max_rows; r++) {  // validates dims; scratch is sized for the largest k-split of any row count
    const MoeSplits &sp = splits(r);
    max_S_gu = std::max(max_S_gu, sp.S_gu);
    max_S_d = std::max(max_S_d, sp.S_d);
  }
  const size_t H = d.hidden, I = d.inter, E = d.experts, k = d.top_k, R = max_rows, P = R * k;
  const size_t Sg = max_S_gu, Sd = max_S_d;
  auto al = [&](size_t n) { void *p = nullptr; IJ_CUDA(cudaMalloc(&p, std::max<size_t>(n, 16))); IJ_CUDA(cudaMemset(p, 0, std::max<size_t>(n, 16))); owned.push_back(p); return p; };
  logits = (float *)al(R * (E + 1) * 4);
  route = (uint32_t *)al(R * 2 * k * 4);
  plan = (int *)al(PlanView::ints((int)P) * 4);
  raw_gu = (float *)al(Sg * P * 2 * I * 4);
  raw_sgu = (float *)al(Sg * R * 2 * I * 4);
  raw_d = (float *)al(Sd * P * H * 4);
  raw_sd = (float *)al(Sd * R * H * 4);
  xh_gu = (__half *)al(P * 2 * H * 2 * A_HALFS_PER_INPUT);
  xh_sgu = (__half *)al(R * 2 * H * 2 * A_HALFS_PER_INPUT);
  xh_d = (__half *)al(P * I * 2 * A_HALFS_PER_INPUT);
  xh_sd = (__half *)al(R * I * 2 * A_HALFS_PER_INPUT);
  gush = (float *)al(R * 2 * I * 4);
  if (shared_q8) { q8_g = (float *)al(R * I * 4); q8_u = (float *)al(R * I * 4); q8_act = (float *)al(R * I * 4); }
  sho = (float *)al(R * H * 4);
  counter = (unsigned *)al(16);
  x_stage = (float *)al(R * H * 4);
  y_stage = (float *)al(R * H * 4);
  status = device_status_word();
  const int IT = d.hidden / 16, OT = d.inter / 16;
  if (d.expert_count > 0) {
    make_trellis_map(&maps.gate, d.gate.trellis_dev, d.expert_count, IT, OT, d.k_expert, SG_KS);
    make_trellis_map(&maps.up, d.up.trellis_dev, d.expert_count, IT, OT, d.k_expert, SG_KS);
    make_trellis_map(&maps.down, d.down.trellis_dev, d.expert_count, OT, IT, d.k_expert, SG_KS);
  }
  if (has_shared) {
    IJ_CHECK(d.sh_up.trellis_dev && d.sh_down.trellis_dev, "null shared-expert weights");
    make_trellis_map(&maps.sgt, d.sh_gate.trellis_dev, 1, IT, OT, d.k_shared, SG_KS);
    make_trellis_map(&maps.sup, d.sh_up.trellis_dev, 1, IT, OT, d.k_shared, SG_KS);
    make_trellis_map(&maps.sdn, d.sh_down.trellis_dev, 1, OT, IT, d.k_shared, SG_KS);
  }
}

Moe::~Moe() {
  for (void *p : owned) cudaFree(p);
  for (void *p : pf_owned) cudaFree(p);
}

// Prefill: n tokens at once through the sorted / grouped path (pf_moe.cu). Scratch grows with the largest n seen.
// mode 0: route the n tokens here, run the slots of the experts this object holds and the shared expert of the own rows.
// mode PF_HOME: route here, no routed expert at all (their slots are computed by the owners), shared expert of all n tokens.
// mode PF_ROUTED: n (token, slot) pairs that were routed elsewhere: route_in [n][2] = (global expert id, weight bits), every
//   id inside this object's slice; y[i] = weight_i * expert_i(x[i]), no shared expert.
void Moe::prefill(const float *x, int n, int own_row0, int own_rows, float *y, cudaStream_t st, int mode, const uint32_t *route_in) {
  IJ_CHECK(!shared_q8, "an 8-bit affine shared expert runs in the decode-width single-GPU calls only (ne_moe_forward, ne_moe_stage)");
  IJ_CHECK(n >= 1 && n <= 65535, "prefill: %d tokens outside 1..65535", n);
  IJ_CHECK(own_row0 >= 0 && own_rows >= 0 && own_row0 + own_rows <= n, "own rows [%d, %d) outside [0, %d)", own_row0, own_row0 + own_rows, n);
  IJ_CHECK((mode == PF_ROUTED) == (route_in != nullptr), "prefill: a route array goes with the routed mode only");
  const size_t H = desc.hidden, I = desc.inter, E = desc.experts;
  const size_t k = mode == PF_ROUTED ? 1 : desc.top_k;
  const bool shared = has_shared && mode != PF_ROUTED;
  if (n > pf_tokens || n * (int)k > pf_slots) {
    IJ_CUDA(cudaDeviceSynchronize());
    for (void *p : pf_owned) cudaFree(p);
    pf_owned.clear();
    pf_tokens = std::max(pf_tokens, n);
    pf_slots = std::max(pf_slots, n * (int)k);
    auto al = [&](size_t b) { void *p = nullptr; IJ_CUDA(cudaMalloc(&p, std::max<size_t>(b, 16))); pf_owned.push_back(p); return p; };
    const size_t T = pf_tokens, S = pf_slots, cap = ((S + 8 * E + T + 15) / 8) * 8;  // >= pf_pos_cap of any call that fits
    const size_t passes = S / PF_NTOK + E + T / PF_NTOK + 2;
    pf.logits = (float *)al(T * (E + 1) * 4);
    pf.route = (uint32_t *)al(T * 2 * desc.top_k * 4);
    pf.cnt = (int *)al(E * 4);
    pf.off = (int *)al((E + 2) * 4);
    pf.hist = (int *)al(((S + 255) / 256) * E * 4);
    pf.inv = (int *)al(S * 4);
    pf.order = (int *)al(cap * 4);
    pf.seid = (int *)al(cap * 4);
    pf.xh_g = (__half *)al(cap * H * 2);
    pf.xh_u = (__half *)al(cap * H * 2);
    pf.raw_gu = (float *)al(cap * 2 * I * 4);
    pf.xh_d = (__half *)al(cap * I * 2);
    pf.raw_d = (float *)al(cap * H * 4);
    pf.items_gu = (PfItem *)al(passes * 2 * (I / PF_NCOL) * sizeof(PfItem));
    pf.items_d = (PfItem *)al(passes * (H / PF_NCOL) * sizeof(PfItem));
    pf.nitems = (int *)al(16);
    pf.sho = (float *)al(T * H * 4);
  }
  PfParams p = pf;
  p.H = (int)H; p.I = (int)I; p.E = (int)E; p.topk = (int)k; p.Kx = desc.k_expert; p.Ks = desc.k_shared; p.has_shared = shared ? 1 : 0;
  p.n = n; p.S = n * (int)k;
  p.e0 = desc.expert_first; p.ecount = mode == PF_HOME ? 0 : desc.expert_count;
  p.sh_row0 = own_row0; p.sh_rows = shared ? own_rows : 0;
  p.pos_cap = (int)pf_pos_cap(n, (int)k, (int)E, shared);
  p.external_route = mode == PF_ROUTED ? 1 : 0;
  if (mode == PF_ROUTED) p.route = const_cast<uint32_t *>(route_in);  // read only in this mode
  p.router = (const uint16_t *)desc.router_dev;
  p.sgate = (const uint16_t *)desc.shared_gate_w_dev;
  auto stack = [](const ne_exl3_stack &s) { return Exl3Stack{(const char *)s.trellis_dev, (const __half *)s.suh_dev, (const __half *)s.svh_dev}; };
  auto single = [](const ne_exl3_weight &s) { return Exl3Stack{(const char *)s.trellis_dev, (const __half *)s.suh_dev, (const __half *)s.svh_dev}; };
  p.gate = stack(desc.gate); p.up = stack(desc.up); p.down = stack(desc.down);
  p.sgt = single(desc.sh_gate); p.sup = single(desc.sh_up); p.sdn = single(desc.sh_down);
  p.x = x; p.y = y;
  if (mode != PF_ROUTED) pf_last_n = n;
  launch_pf_moe(p, status, st);
}

MoeParams Moe::params(const float *x, int rows, float *y) {
  IJ_CHECK(rows >= 1 && rows <= max_rows, "rows %d outside 1..%d", rows, max_rows);
  // rows are staged with 16-byte asynchronous copies and exchanged as float4: a misaligned view would fault on the device
  IJ_CHECK(((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0, "activation rows (x, y) must be 16-byte aligned on the device");
  MoeParams p{};
  p.H = desc.hidden; p.I = desc.inter; p.E = desc.experts; p.topk = desc.top_k;
  p.Kx = desc.k_expert; p.Ks = desc.k_shared;
  p.e0 = desc.expert_first; p.ecount = desc.expert_count;
  p.rows = rows; p.P = rows * desc.top_k; p.has_shared = has_shared ? 1 : 0; p.shared_pre = shared_q8 ? 1 : 0; p.dup = g_summand_product;
  p.router = (const uint16_t *)desc.router_dev;
  p.sgate = (const uint16_t *)desc.shared_gate_w_dev;
  auto stack = [](const ne_exl3_stack &s) { return Exl3Stack{(const char *)s.trellis_dev, (const __half *)s.suh_dev, (const __half *)s.svh_dev}; };
  auto single = [](const ne_exl3_weight &s) { return Exl3Stack{(const char *)s.trellis_dev, (const __half *)s.suh_dev, (const __half *)s.svh_dev}; };
  p.gate = stack(desc.gate); p.up = stack(desc.up); p.down = stack(desc.down);
  p.sgt = single(desc.sh_gate); p.sup = single(desc.sh_up); p.sdn = single(desc.sh_down);
  p.x = x; p.logits = logits; p.route = route; p.plan = plan;
  p.xh_gu = xh_gu; p.xh_sgu = xh_sgu; p.xh_d = xh_d; p.xh_sd = xh_sd;
  p.raw_gu = raw_gu; p.raw_sgu = raw_sgu; p.raw_d = raw_d; p.raw_sd = raw_sd;
  p.gush = gush; p.sho = sho; p.y = y; p.counter = counter;
  const MoeSplits &s = splits(rows);
  p.S_gu = s.S_gu; p.kc_gu = s.kc_gu; p.S_d = s.S_d; p.kc_d = s.kc_d;
  p.h_mid = h_mid; p.inj = inj; p.h_out = h_out; p.HC = HC;
  p.sh_row0 = 0; p.sh_rows = rows; p.lg_row0 = 0;
  p.ldx = desc.hidden; p.ldr = 2 * desc.top_k;
  p.ep = nullptr; p.ep_rows = 0;
  return p;
}

const MoeSplits &Moe::splits(int rows) {
  auto it = split_cache.find(rows);
  if (it == split_cache.end())
    it = split_cache.emplace(rows, plan_moe(desc.hidden, desc.inter, desc.experts, desc.top_k, desc.k_expert, desc.k_shared, rows, has_shared)).first;
  return it->second;
}

void Moe::stage(int stage_no, const float *x, int rows, float *y, cudaStream_t st) {
  const MoeParams p = params(x, rows, y);
  const MoeSplits &s = splits(rows);
  switch (stage_no) {
    case 7: launch_moe_router(p, true, st); break;
    case 8: launch_moe_prep(p, false, st); launch_moe_gateup(p, maps, s, true, status, st); break;
    case 9:
      if (shared_q8) shared_q8_run(x, rows, st);
      launch_moe_mid(p, st); launch_moe_down(p, maps, s, status, st); launch_moe_combine(p, false, st); break;
    // single kernels of stages 8 and 9 (for per-kernel timing; each needs the state the kernels before it leave)
    case 80: launch_moe_prep(p, false, st); break;
    case 81: launch_moe_gateup(p, maps, s, true, status, st); break;
    case 90: launch_moe_mid(p, st); break;
    case 91: launch_moe_down(p, maps, s, status, st); break;
    case 92: launch_moe_combine(p, false, st); break;
    default: fail("bad MoE stage %d (7 router, 8 gate/up, 9 down; 80 81 90 91 92 their single kernels)", stage_no);
  }
  last_rows = rows;
}

static Q8Weight q8_of(const ne_q8_weight &w) {
  Q8Weight q;
  q.w = static_cast<const uint8_t *>(w.weight_dev);
  q.scales = static_cast<const uint16_t *>(w.scales_dev);
  q.biases = static_cast<const uint16_t *>(w.biases_dev);
  q.rows = w.out; q.in = w.in; q.group = w.group;
  return q;
}

// the 8-bit affine shared expert: four launches that depend on x only (they precede the router in the chain)
void Moe::shared_q8_run(const float *x, int rows, cudaStream_t st) {
  launch_q8_linear(q8_of(desc.sh_gate_q8), x, rows, q8_g, status, st);
  launch_q8_linear(q8_of(desc.sh_up_q8), x, rows, q8_u, status, st);
  launch_swiglu_rows(q8_g, q8_u, rows, desc.inter, gush, q8_act, st);
  launch_q8_linear(q8_of(desc.sh_down_q8), q8_act, rows, sho, status, st);
}

int Moe::shared_q8_launches(int rows) const {
  if (!shared_q8) return 0;
  return q8_linear_launches(q8_of(desc.sh_gate_q8), rows) + q8_linear_launches(q8_of(desc.sh_up_q8), rows) + 1 +
         q8_linear_launches(q8_of(desc.sh_down_q8), rows);
}

void Moe::forward(const float *x, int rows, float *y, cudaStream_t st) {
  const MoeParams p = params(x, rows, y);
  const MoeSplits &s = splits(rows);
  if (shared_q8) shared_q8_run(x, rows, st);
  launch_moe_router(p, true, st);  // the finisher also builds the plan: final before the gate/up kernel can start
  launch_moe_prep(p, false, st);
  launch_moe_gateup(p, maps, s, true, status, st);
  launch_moe_mid(p, st);
  launch_moe_down(p, maps, s, status, st);
  launch_moe_combine(p, false, st);
  last_rows = rows;
}

// Expert parallel: all ranks' rows come in; routing runs on all of them (replicated), the plan keeps only this object's
// experts, and the shared expert is added for the caller's own rows only. y is this rank's summand of the block output.
void Moe::forward_ep(const float *x, int rows, int own_row0, int own_rows, float *y, cudaStream_t st) {
  IJ_CHECK(!shared_q8, "an 8-bit affine shared expert runs in the decode-width single-GPU calls only (ne_moe_forward, ne_moe_stage)");
  MoeParams p = params(x, rows, y);
  IJ_CHECK(own_row0 >= 0 && own_rows >= 0 && own_row0 + own_rows <= rows, "own rows [%d, %d) outside [0, %d)", own_row0, own_row0 + own_rows, rows);
  p.sh_row0 = own_row0;
  p.sh_rows = own_rows;
  const MoeSplits &s = splits(rows);
  launch_moe_router(p, true, st);  // the finisher also builds the plan: final before the gate/up kernel can start
  launch_moe_prep(p, false, st);
  launch_moe_gateup(p, maps, s, true, status, st);
  launch_moe_mid(p, st);
  launch_moe_down(p, maps, s, status, st);
  launch_moe_combine(p, false, st);
  last_rows = rows;
}

// The router alone on `rows` rows: routes to route_out ([rows][2 top_k], or the object's own buffer), logits (with the shared
// expert's gate logit) stay in the object for a following forward_ep_routed.
void Moe::route_rows(const float *x, int rows, uint32_t *route_out, int ld_route, cudaStream_t st) {
  MoeParams p = params(x, rows, nullptr);
  if (route_out) { p.route = route_out; p.ldr = ld_route > 0 ? ld_route : p.ldr; }
  IJ_CHECK(p.ldr >= 2 * desc.top_k, "route row stride %d < %d", p.ldr, 2 * desc.top_k);
  launch_moe_router(p, false, st);
}

// Expert parallel with the routing done by each row's home rank: rows and routes of all ranks come in; the shared expert's
// gate logits of the own rows are the ones route_rows left in the object.
void Moe::forward_ep_routed(const float *x, int ld_x, const uint32_t *route_all, int ld_route, int rows, int own_row0, int own_rows, float *y,
                            cudaStream_t st) {
  IJ_CHECK(!shared_q8, "an 8-bit affine shared expert runs in the decode-width single-GPU calls only (ne_moe_forward, ne_moe_stage)");
  MoeParams p = params(x, rows, y);
  if (ld_x > 0) p.ldx = ld_x;
  if (ld_route > 0) p.ldr = ld_route;
  IJ_CHECK(p.ldx >= desc.hidden && p.ldr >= 2 * desc.top_k, "row strides %d / %d too small", p.ldx, p.ldr);
  IJ_CHECK(p.ldx % 4 == 0, "the row stride of x (%d floats) must keep every row 16-byte aligned", p.ldx);
  IJ_CHECK(own_row0 >= 0 && own_rows >= 0 && own_row0 + own_rows <= rows, "own rows [%d, %d) outside [0, %d)", own_row0, own_row0 + own_rows, rows);
  p.route = const_cast<uint32_t *>(route_all);
  p.sh_row0 = own_row0; p.sh_rows = own_rows; p.lg_row0 = own_row0;
  const MoeSplits &s = splits(rows);
  launch_moe_prep(p, true, st);
  launch_moe_gateup(p, maps, s, false, status, st);
  launch_moe_mid(p, st);
  launch_moe_down(p, maps, s, status, st);
  launch_moe_combine(p, false, st);
  last_rows = rows;
}

// The whole expert-parallel block over peer memory: route the own rows, exchange packed rows, compute this rank's experts
// for all rows with the combine writing into the owners' memory, sum the partial rows that arrived here.
void Moe::forward_ep_fused(EpCtx &c, const float *x_own, int rows, float *y_own, cudaStream_t st) {
  IJ_CHECK(!shared_q8, "an 8-bit affine shared expert runs in the decode-width single-GPU calls only (ne_moe_forward, ne_moe_stage)");
  const int H = desc.hidden, k = desc.top_k, world = c.host.world, all = rows * world;
  IJ_CHECK(c.connected, "expert-parallel context is not connected");
  IJ_CHECK(c.host.H == H && c.top_k == k, "expert-parallel context was made for other dims");
  IJ_CHECK(rows >= 1 && rows <= c.host.rows_cap && all <= max_rows, "rows %d x %d ranks exceed the context (%d) or the object (%d)", rows, world,
           c.host.rows_cap, max_rows);
  const int W = c.host.W;
  route_rows(x_own, rows, c.route_own, 0, st);
  launch_ep_exchange(c, x_own, c.route_own, rows, status, st);
  const float *gathered = c.host.gather[c.host.rank];
  MoeParams p = params(gathered, all, y_own);
  p.ldx = W; p.ldr = W;
  p.route = reinterpret_cast<uint32_t *>(const_cast<float *>(gathered) + H);
  p.sh_row0 = c.host.rank * rows; p.sh_rows = rows; p.lg_row0 = p.sh_row0;
  p.ep = c.dev; p.ep_rows = rows;
  const MoeSplits &s = splits(all);
  launch_moe_prep(p, true, st);
  launch_moe_gateup(p, maps, s, false, status, st);
  launch_moe_mid(p, st);
  launch_moe_down(p, maps, s, status, st);
  launch_moe_combine(p, false, st);
  launch_ep_sum(c, rows, y_own, status, st);
  last_rows = all;
}

void Moe::forward_routed(const float *x, const uint32_t *route_in, int rows, float *y, cudaStream_t st) {
  IJ_CHECK(!shared_q8, "an 8-bit affine shared expert runs in the decode-width single-GPU calls only (ne_moe_forward, ne_moe_stage)");
  MoeParams p = params(x, rows, y);
  IJ_CUDA(cudaMemcpyAsync(route, route_in, (size_t)rows * 2 * desc.top_k * 4, cudaMemcpyDeviceToDevice, st));
  p.has_shared = 0;
  const MoeSplits &s = splits(rows);
  launch_moe_prep(p, true, st);
  launch_moe_gateup(p, maps, s, false, status, st);
  launch_moe_mid(p, st);
  launch_moe_down(p, maps, s, status, st);
  launch_moe_combine(p, true, st);
  last_rows = rows;
}

}  // namespace ijah

extern "C" {

NE_API int ne_exl3_dequant(const ne_exl3_weight *w, void *w_f16_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(w && w->trellis_dev && w_f16_dev, "null argument");
    launch_dequant(w->trellis_dev, w->in, w->out, w->K, (__half *)w_f16_dev, (cudaStream_t)stream);
  });
}

NE_API int ne_exl3_linear(const ne_exl3_weight *w, const float *x_dev, int rows, float *y_dev, void *stream) {
  return c_call([&] {
    check_weight(w);
    IJ_CHECK(x_dev && y_dev, "null activation pointer");
    const LinearPlan p = plan_linear(w->in, w->out, w->K, rows);
    void *scratch = device_scratch(p.scratch_bytes());
    launch_linear(p, w->trellis_dev, w->suh_dev, w->svh_dev, x_dev, y_dev, scratch, device_status_word(), (cudaStream_t)stream);
  });
}

static Q8Weight q8_from_c(const ne_q8_weight *w) {
  IJ_CHECK(w != nullptr, "null weight");
  Q8Weight q;
  q.w = static_cast<const uint8_t *>(w->weight_dev);
  q.scales = static_cast<const uint16_t *>(w->scales_dev);
  q.biases = static_cast<const uint16_t *>(w->biases_dev);
  q.rows = w->out; q.in = w->in; q.group = w->group;
  return q;
}

NE_API int ne_q8_linear(const ne_q8_weight *w, const float *x_dev, int rows, float *y_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(x_dev && y_dev, "null activation pointer");
    launch_q8_linear(q8_from_c(w), x_dev, rows, y_dev, device_status_word(), (cudaStream_t)stream);
  });
}

NE_API int ne_q8_embed(const ne_q8_weight *w, const int *tokens_dev, int rows, float *x_dev, int round_bf16, void *stream) {
  return c_call([&] {
    IJ_CHECK(tokens_dev && x_dev && rows >= 1, "bad arguments");
    launch_q8_embed(q8_from_c(w), tokens_dev, rows, x_dev, round_bf16 != 0, (cudaStream_t)stream);
  });
}

NE_API int ne_exl3_linear_plan(int n_in, int n_out, int K, int rows, int *info8, uint64_t *scratch_bytes) {
  return c_call([&] {
    const LinearPlan p = plan_linear(n_in, n_out, K, rows);
    if (info8) {
      const int v[8] = {p.S, p.kc, p.lay.stages, p.lay.aslots, p.grid, p.MT, (int)p.lay.total(), p.lay.stage_bytes};
      memcpy(info8, v, sizeof v);
    }
    if (scratch_bytes) *scratch_bytes = p.scratch_bytes();
  });
}
NE_API int ne_moe_plan(int hidden, int inter, int experts, int top_k, int k_expert, int k_shared, int rows, int *info8) {
  return c_call([&] {
    const MoeSplits s = plan_moe(hidden, inter, experts, top_k, k_expert, k_shared, rows, k_shared > 0);
    if (info8) {
      const int v[8] = {s.S_gu, s.kc_gu, s.S_d, s.kc_d, s.lay_gu.stages, s.lay_d.stages, s.grid, (int)std::max(s.lay_gu.total(), s.lay_d.total())};
      memcpy(info8, v, sizeof v);
    }
  });
}

NE_API int ne_exl3_linear_multi(const ne_exl3_weight *w, int n, const float *x_dev, int rows, float *const *y_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(w && x_dev && y_dev && n >= 1 && n <= ML_MAX, "bad arguments (1..%d Linears)", ML_MAX);
    int out[ML_MAX], K[ML_MAX];
    MultiLinearArgs a{};
    for (int m = 0; m < n; m++) {
      check_weight(&w[m]);
      IJ_CHECK(w[m].in == w[0].in, "Linears of one call must share the input width (%d vs %d)", w[m].in, w[0].in);
      IJ_CHECK(y_dev[m] != nullptr, "null output pointer");
      out[m] = w[m].out; K[m] = w[m].K;
      a.trellis[m] = w[m].trellis_dev; a.suh[m] = w[m].suh_dev; a.svh[m] = w[m].svh_dev; a.y[m] = y_dev[m];
    }
    const MultiLinearPlan p = plan_linear_multi(n, w[0].in, out, K, rows);
    launch_linear_multi(p, a, x_dev, device_scratch(p.scratch_bytes()), device_status_word(), (cudaStream_t)stream);
  });
}

NE_API int ne_exl3_linear_prefill(const ne_exl3_weight *w, const float *x_dev, int rows, float *y_dev, void *stream) {
  return c_call([&] {
    check_weight(w);
    IJ_CHECK(x_dev && y_dev, "null activation pointer");
    void *scratch = device_scratch(pf_linear_scratch_bytes(w->in, w->out, rows));
    launch_pf_linear(w->trellis_dev, w->suh_dev, w->svh_dev, w->in, w->out, w->K, x_dev, rows, y_dev, scratch, device_status_word(),
                     (cudaStream_t)stream);
  });
}

NE_API int ne_exl3_linear_host(const ne_exl3_weight *w, const float *x_host, int rows, float *y_host) {
  return c_call([&] {
    check_weight(w);
    IJ_CHECK(x_host && y_host, "null activation pointer");
    const LinearPlan p = plan_linear(w->in, w->out, w->K, rows);
    const size_t xb = (size_t)rows * w->in * 4, yb = (size_t)rows * w->out * 4;
    char *s = (char *)device_scratch(p.scratch_bytes() + xb + yb + 512);
    float *xd = (float *)(s + ((p.scratch_bytes() + 255) & ~(size_t)255));
    float *yd = (float *)((char *)xd + ((xb + 255) & ~(size_t)255));
    IJ_CUDA(cudaMemcpyAsync(xd, x_host, xb, cudaMemcpyHostToDevice, 0));
    launch_linear(p, w->trellis_dev, w->suh_dev, w->svh_dev, xd, yd, s, device_status_word(), 0);
    IJ_CUDA(cudaMemcpyAsync(y_host, yd, yb, cudaMemcpyDeviceToHost, 0));
    IJ_CUDA(cudaStreamSynchronize(0));
  });
}

NE_API ne_moe *ne_moe_create(const ne_moe_desc *d, int max_rows) {
  Moe *m = nullptr;
  const int rc = c_call([&] {
    IJ_CHECK(d != nullptr, "null ne_moe_desc");
    m = new Moe(*d, max_rows);
  });
  return rc == 0 ? reinterpret_cast<ne_moe *>(m) : nullptr;
}
NE_API void ne_moe_free(ne_moe *m) { delete reinterpret_cast<Moe *>(m); }

NE_API int ne_moe_forward(ne_moe *m, const float *x_dev, int rows, float *y_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_dev && y_dev, "null argument");
    reinterpret_cast<Moe *>(m)->forward(x_dev, rows, y_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_forward_host(ne_moe *m, const float *x_host, int rows, float *y_host) {
  return c_call([&] {
    Moe *o = reinterpret_cast<Moe *>(m);
    IJ_CHECK(o && x_host && y_host, "null argument");
    IJ_CHECK(rows >= 1 && rows <= o->max_rows, "rows %d outside 1..%d", rows, o->max_rows);
    const size_t b = (size_t)rows * o->desc.hidden * 4;
    IJ_CUDA(cudaMemcpyAsync(o->x_stage, x_host, b, cudaMemcpyHostToDevice, 0));
    o->forward(o->x_stage, rows, o->y_stage, 0);
    IJ_CUDA(cudaMemcpyAsync(y_host, o->y_stage, b, cudaMemcpyDeviceToHost, 0));
    IJ_CUDA(cudaStreamSynchronize(0));
  });
}
NE_API int ne_moe_stage(ne_moe *m, int stage, const float *x_dev, int rows, float *y_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_dev && y_dev, "null argument");
    reinterpret_cast<Moe *>(m)->stage(stage, x_dev, rows, y_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_forward_routed(ne_moe *m, const float *x_dev, const uint32_t *route_dev, int rows, float *y_partial_dev,
                                 void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_dev && route_dev && y_partial_dev, "null argument");
    reinterpret_cast<Moe *>(m)->forward_routed(x_dev, route_dev, rows, y_partial_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_forward_ep(ne_moe *m, const float *x_all_dev, int rows_all, int own_row0, int own_rows, float *y_part_dev,
                             void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_all_dev && y_part_dev, "null argument");
    reinterpret_cast<Moe *>(m)->forward_ep(x_all_dev, rows_all, own_row0, own_rows, y_part_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_prefill(ne_moe *m, const float *x_dev, int n_tokens, float *y_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_dev && y_dev, "null argument");
    Moe *o = reinterpret_cast<Moe *>(m);
    IJ_CHECK(o->desc.expert_first == 0 && o->desc.expert_count == o->desc.experts,
             "ne_moe_prefill runs on an object that holds all experts (expert parallel: ne_moe_prefill_ep)");
    o->prefill(x_dev, n_tokens, 0, n_tokens, y_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_route(ne_moe *m, const float *x_dev, int rows, uint32_t *route_out_dev, int ld_route, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_dev, "null argument");
    reinterpret_cast<Moe *>(m)->route_rows(x_dev, rows, route_out_dev, ld_route, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_forward_ep_routed(ne_moe *m, const float *x_all_dev, int ld_x, const uint32_t *route_all_dev, int ld_route, int rows_all,
                                    int own_row0, int own_rows, float *y_part_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_all_dev && route_all_dev && y_part_dev, "null argument");
    reinterpret_cast<Moe *>(m)->forward_ep_routed(x_all_dev, ld_x, route_all_dev, ld_route, rows_all, own_row0, own_rows, y_part_dev,
                                                  (cudaStream_t)stream);
  });
}
// ---- expert-parallel exchange context (ep_exchange.cuh)
NE_API ne_ep *ne_ep_create(int rank, int world, int rows_cap, int hidden, int top_k) {
  ne_ep *out = nullptr;
  c_call([&] {
    IJ_CHECK(world >= 1 && world <= EP_MAX_RANKS && rank >= 0 && rank < world, "bad rank %d of %d (at most %d ranks)", rank, world, EP_MAX_RANKS);
    IJ_CHECK(rows_cap >= 1 && hidden % 4 == 0 && top_k >= 1 && (2 * top_k) % 4 == 0, "bad dims (hidden and 2 * top_k must be multiples of 4)");
    auto c = std::make_unique<EpCtx>();
    c->top_k = top_k;
    EpDev &h = c->host;
    h.rank = rank; h.world = world; h.rows_cap = rows_cap; h.H = hidden; h.W = hidden + 2 * top_k;
    auto up = [](size_t b) { return (b + 255) & ~(size_t)255; };
    c->off_gather = 0;
    c->off_part = up((size_t)world * rows_cap * h.W * 4);
    c->off_flags = c->off_part + up((size_t)world * rows_cap * hidden * 4);
    c->bytes = c->off_flags + 256;  // two flag arrays of EP_MAX_RANKS words
    IJ_CUDA(cudaMalloc(&c->local, c->bytes));
    IJ_CUDA(cudaMemset(c->local, 0, c->bytes));
    IJ_CUDA(cudaMalloc((void **)&c->route_own, (size_t)rows_cap * 2 * top_k * 4));
    IJ_CUDA(cudaMalloc((void **)&h.counter, 64));  // counter, epoch, ticket: one word each, 16 bytes apart
    IJ_CUDA(cudaMemset(h.counter, 0, 64));
    h.epoch = reinterpret_cast<uint32_t *>(h.counter + 4);
    h.ticket = h.counter + 8;
    IJ_CUDA(cudaMalloc((void **)&c->dev, sizeof(EpDev)));
    IJ_CUDA(cudaDeviceSynchronize());
    out = reinterpret_cast<ne_ep *>(c.release());
  });
  return out;
}
NE_API int ne_ep_handle(ne_ep *e, void *handle64) {
  return c_call([&] {
    IJ_CHECK(e && handle64, "null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    IJ_CUDA(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(handle64), reinterpret_cast<EpCtx *>(e)->local));
  });
}
NE_API int ne_ep_connect(ne_ep *e, const void *handles64) {
  return c_call([&] {
    EpCtx *c = reinterpret_cast<EpCtx *>(e);
    IJ_CHECK(c && handles64 && !c->connected, "null argument or already connected");
    EpDev &h = c->host;
    for (int r = 0; r < h.world; r++) {
      char *base;
      if (r == h.rank) base = (char *)c->local;
      else {
        cudaIpcMemHandle_t hd;
        memcpy(&hd, (const char *)handles64 + 64 * r, 64);
        IJ_CUDA(cudaIpcOpenMemHandle(&c->peer[r], hd, cudaIpcMemLazyEnablePeerAccess));
        base = (char *)c->peer[r];
      }
      h.gather[r] = (float *)(base + c->off_gather);
      h.part[r] = (float *)(base + c->off_part);
      h.gflag[r] = (uint32_t *)(base + c->off_flags);
      h.pflag[r] = (uint32_t *)(base + c->off_flags + 128);
    }
    IJ_CUDA(cudaMemcpy(c->dev, &h, sizeof h, cudaMemcpyHostToDevice));
    c->connected = true;
  });
}
NE_API int ne_ep_disconnect(ne_ep *e) {
  return c_call([&] {
    EpCtx *c = reinterpret_cast<EpCtx *>(e);
    IJ_CHECK(c != nullptr, "null argument");
    IJ_CUDA(cudaDeviceSynchronize());
    for (int r = 0; r < c->host.world; r++)
      if (c->peer[r]) { cudaIpcCloseMemHandle(c->peer[r]); c->peer[r] = nullptr; }
    c->connected = false;
  });
}
// Teardown order across ranks: every rank calls ne_ep_disconnect (closes its mappings of the peers' buffers), the ranks
// synchronise on the host (a barrier), then each calls ne_ep_free: a buffer must not be freed while a peer still has it
// mapped. ne_ep_free alone (it closes the mappings first) is enough only once every peer has disconnected or exited.
NE_API void ne_ep_free(ne_ep *e) {
  EpCtx *c = reinterpret_cast<EpCtx *>(e);
  if (!c) return;
  cudaDeviceSynchronize();
  for (int r = 0; r < c->host.world; r++)
    if (c->peer[r]) cudaIpcCloseMemHandle(c->peer[r]);
  cudaFree(c->local); cudaFree(c->route_own); cudaFree(c->host.counter); cudaFree(c->dev);
  delete c;
}
NE_API int ne_moe_forward_ep_fused(ne_moe *m, ne_ep *e, const float *x_own_dev, int rows, float *y_own_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && e && x_own_dev && y_own_dev, "null argument");
    reinterpret_cast<Moe *>(m)->forward_ep_fused(*reinterpret_cast<EpCtx *>(e), x_own_dev, rows, y_own_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_prefill_ep(ne_moe *m, const float *x_all_dev, int n_all, int own_row0, int own_rows, float *y_part_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_all_dev && y_part_dev, "null argument");
    reinterpret_cast<Moe *>(m)->prefill(x_all_dev, n_all, own_row0, own_rows, y_part_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_prefill_home(ne_moe *m, const float *x_dev, int n_tokens, float *y_shared_dev, uint32_t *route_out_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_dev && y_shared_dev && route_out_dev, "null argument");
    Moe *o = reinterpret_cast<Moe *>(m);
    o->prefill(x_dev, n_tokens, 0, n_tokens, y_shared_dev, (cudaStream_t)stream, Moe::PF_HOME);
    IJ_CUDA(cudaMemcpyAsync(route_out_dev, o->pf.route, (size_t)n_tokens * 2 * o->desc.top_k * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  });
}
NE_API int ne_moe_prefill_routed(ne_moe *m, const float *x_pairs_dev, const uint32_t *route_pairs_dev, int n_pairs, float *y_pairs_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(m && x_pairs_dev && route_pairs_dev && y_pairs_dev, "null argument");
    reinterpret_cast<Moe *>(m)->prefill(x_pairs_dev, n_pairs, 0, 0, y_pairs_dev, (cudaStream_t)stream, Moe::PF_ROUTED, route_pairs_dev);
  });
}
NE_API int ne_ep_pairs_by_owner(const uint32_t *route_dev, int n_tokens, int top_k, int experts_per_rank, int world, int *send_token_dev,
                                uint32_t *send_route_dev, int *pos_dev, long long *counts_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(route_dev && send_token_dev && send_route_dev && pos_dev && counts_dev, "null argument");
    launch_pairs_by_owner(route_dev, n_tokens, top_k, experts_per_rank, world, send_token_dev, send_route_dev, pos_dev, counts_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_rows_gather(const float *src_dev, const int *index_dev, int n_out, int width, float *dst_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(src_dev && index_dev && dst_dev, "null argument");
    launch_rows_gather(src_dev, index_dev, n_out, width, dst_dev, (cudaStream_t)stream);
  });
}
NE_API int ne_slots_combine(const float *slots_dev, const int *pos_dev, const float *base_dev, float *y_dev, int n_tokens, int top_k, int width,
                            void *stream) {
  return c_call([&] {
    IJ_CHECK(slots_dev && pos_dev && y_dev, "null argument");
    launch_slots_combine(slots_dev, pos_dev, base_dev, y_dev, n_tokens, top_k, width, (cudaStream_t)stream);
  });
}
NE_API int ne_moe_buffer(ne_moe *m, const char *name, void **dev, uint64_t *nbytes) {
  return c_call([&] {
    Moe *o = reinterpret_cast<Moe *>(m);
    IJ_CHECK(o && name && dev && nbytes, "null argument");
    const size_t H = o->desc.hidden, I = o->desc.inter, E = o->desc.experts, k = o->desc.top_k, R = o->last_rows;
    const std::string n = name;
    if (n == "logits") { *dev = o->logits; *nbytes = R * (E + 1) * 4; }
    else if (n == "route") { *dev = o->route; *nbytes = R * 2 * k * 4; }
    else if (n == "shared_gu") { *dev = o->gush; *nbytes = R * 2 * I * 4; }
    else if (n == "shared_down") { *dev = o->sho; *nbytes = R * H * 4; }
    else if (n == "experts_gu_raw") { *dev = o->raw_gu; *nbytes = (size_t)o->splits((int)R).S_gu * R * k * 2 * I * 4; }
    else if (n == "plan") { *dev = o->plan; *nbytes = PlanView::ints((int)(R * k)) * 4; }
    else if (n == "prefill_route") { *dev = o->pf.route; *nbytes = (size_t)o->pf_last_n * 2 * k * 4; }
    else if (n == "prefill_counts") { *dev = o->pf.cnt; *nbytes = E * 4; }
    else if (n == "prefill_logits") { *dev = o->pf.logits; *nbytes = (size_t)o->pf_last_n * (E + 1) * 4; }
    else fail("unknown MoE buffer '%s'", name);
  });
}
NE_API int ne_moe_experts_gu(ne_moe *m, int rows, float *dst_host) {
  return c_call([&] {
    Moe *o = reinterpret_cast<Moe *>(m);
    IJ_CHECK(o && dst_host && rows >= 1 && rows <= o->max_rows, "bad argument");
    const size_t n = (size_t)rows * o->desc.top_k * 2 * o->desc.inter;
    const int S = o->splits(rows).S_gu;
    std::vector<float> tmp(n * S);
    IJ_CUDA(cudaDeviceSynchronize());
    IJ_CUDA(cudaMemcpy(tmp.data(), o->raw_gu, tmp.size() * 4, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < n; i++) {
      float a = 0.0f;
      for (int s = 0; s < S; s++) a += tmp[(size_t)s * n + i];  // split order, as the device sums them
      dst_host[i] = a;
    }
  });
}
NE_API int ne_exl3_set_summand_product(int on) {
  const int was = g_summand_product;
  if (on == 0 || on == 1) g_summand_product = on;
  return was;
}

NE_API int ne_moe_last_bytes(ne_moe *m, int rows, uint64_t *total, uint64_t *gateup, uint64_t *down, int *distinct_experts) {
  return c_call([&] {
    Moe *o = reinterpret_cast<Moe *>(m);
    IJ_CHECK(o && rows >= 1 && rows <= o->max_rows, "bad argument");
    int head[2] = {0, 0};  // entries, distinct experts
    IJ_CUDA(cudaDeviceSynchronize());
    IJ_CUDA(cudaMemcpy(head, o->plan, 8, cudaMemcpyDeviceToHost));
    const int nu = head[1];
    const uint64_t H = o->desc.hidden, I = o->desc.inter, E = o->desc.experts;
    const uint64_t lin_x = H * I * o->desc.k_expert / 8, lin_s = H * I * o->desc.k_shared / 8;
    const uint64_t gu = (uint64_t)nu * 2 * (lin_x + 2 * H + 2 * I) + (o->has_shared ? 2 * (lin_s + 2 * H + 2 * I) : 0);
    const uint64_t dn = (uint64_t)nu * (lin_x + 2 * I + 2 * H) + (o->has_shared ? lin_s + 2 * I + 2 * H : 0);
    uint64_t rt = E * H * 2 + (o->has_shared ? H * 2 : 0);
    if (o->shared_q8)  // three 8-bit affine Linears and the gate vector
      rt += q8_weight_bytes(q8_of(o->desc.sh_gate_q8)) + q8_weight_bytes(q8_of(o->desc.sh_up_q8)) + q8_weight_bytes(q8_of(o->desc.sh_down_q8)) + H * 2;
    if (gateup) *gateup = gu;
    if (down) *down = dn;
    if (total) *total = gu + dn + rt + 2ull * rows * H * 4;
    if (distinct_experts) *distinct_experts = nu;
  });
}

}  // extern "C"
