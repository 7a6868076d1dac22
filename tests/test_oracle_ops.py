"""The numpy restatement of the operator reference against fixtures produced by the reference's own tools/opref.py
(tests/golden/make_golden.py). CPU only."""
import numpy as np

from oracle import opref_port as O
from tests.helpers import MoeView, hc_oracle, hc_small, q8_parts, q8_small, rel_max, small_pack, trunk_linear


def test_router_matches_reference():
    t, g = small_pack()
    mv = MoeView(t)
    logits, p, ids, w = O.moe_route(g["x"], mv.router, int(g["topk"]))
    assert np.array_equal(ids, g["ids"])
    assert np.allclose(logits, g["logits"], rtol=0, atol=1e-6)
    assert np.allclose(w, g["weights"], rtol=1e-6)
    ids2, w2 = O.route_device_order(logits, int(g["topk"]))
    assert np.array_equal(ids2, g["ids"]) and np.allclose(w2, g["weights"], rtol=2e-6)


def test_dense_experts_match_reference():
    t, g = small_pack()
    mv = MoeView(t)
    for e in (int(g["gate_expert_id"]), 31):
        for proj, lin in zip(("gate", "up", "down"), mv.expert(e)):
            assert np.array_equal(lin.inner[::7, ::5], g[f"inner_{proj}_{e}_sub"])
            assert np.allclose(lin.dense[::7, ::5], g[f"W_{proj}_{e}_sub"], rtol=0, atol=1e-7)
            assert abs(lin.dense.astype(np.float64).sum() - float(g[f"W_{proj}_{e}_sum"])) < 1e-5


def test_inner_out_and_finish_match_reference():
    t, g = small_pack()
    lin = MoeView(t).expert(int(g["gate_expert_id"]))[0]
    io = O.exl3_inner_out(g["x"][0], lin.inner, lin.suh.astype(np.float32))
    assert np.allclose(io, g["gate_inner_out"], rtol=0, atol=1e-5)
    assert np.allclose(O.exl3_finish(io, lin.svh.astype(np.float32)), g["gate_finish"], rtol=0, atol=1e-6)


def test_block_matches_reference():
    t, g = small_pack()
    mv = MoeView(t)
    r = O.moe_block_exact(g["x"], mv.router, mv.sgate, mv.expert, mv.shared, int(g["topk"]))
    assert np.array_equal(r["ids"], g["ids"])
    assert rel_max(r["routed"], g["routed"]) < 1e-6
    assert rel_max(r["shared"], g["shared_out"]) < 1e-6
    assert np.allclose(r["shared_scale"], g["shared_scale"], rtol=1e-6)
    assert rel_max(r["out"], g["block_out"]) < 1e-6


def test_device_arithmetic_emulation_is_within_budget_of_reference():
    # The float16 operand preparation is the only systematic difference (the reference measured <= 5.8e-4 for it,
    # docs/trunk6.md:78-84); the acceptance bound for layer outputs is 2e-3 of the output's max-abs.
    t, g = small_pack()
    mv = MoeView(t)
    r = O.moe_block_emul(g["x"], mv.router, mv.sgate, mv.expert, mv.shared, int(g["topk"]))
    assert np.array_equal(r["ids"], g["ids"])
    assert rel_max(r["out"], g["block_out"]) < 2e-3
    assert rel_max(r["shared_gu"][:, 0], g["shared_gate_proj"]) < 2e-3
    assert rel_max(r["shared_down"], g["shared_out"]) < 2e-3


def test_trunk_linears_match_reference():
    t, g = small_pack()
    x = g["x"]
    for layer in (0, 1):
        for proj in ("q", "k", "v", "o"):
            lin = trunk_linear(t, layer, proj)
            xin = x if lin.inner.shape[0] == x.shape[1] else np.tile(x, (1, lin.inner.shape[0] // x.shape[1]))
            assert np.allclose(lin.dense.T[::5, ::7], g[f"trunk_L{layer}_{proj}_Wsub"], rtol=0, atol=1e-7)
            want = g[f"trunk_L{layer}_{proj}_y"]
            assert rel_max(O.exl3_linear_exact(xin, lin.trellis, lin.suh, lin.svh), want) < 1e-5
            assert rel_max(O.exl3_linear_emul(xin, lin.trellis, lin.suh, lin.svh), want) < 2e-3


def test_hc_read_matches_reference():
    # the reference's hc_read (f32 flow) on the small hyper-connection tensors; its bf16 flow differs by bf16 rounding only
    t, g = hc_small()
    r = hc_oracle(t, g["h"])
    for k in ("normed", "mix", "block_in", "inject_w"):
        assert rel_max(r[k], g["f32_" + k]) < 2e-6, k
        assert rel_max(r[k], g["bf16_" + k]) < 2e-2, k


def test_q8_linear_and_embedding_match_reference():
    # the reference's linear_big (f32 flow) and linear_rows (bf16 rows) on the small 8-bit affine head and embedding
    t, g = q8_small()
    assert rel_max(O.q8_linear(g["x"], *q8_parts(t, "language_model.lm_head")), g["head_y"]) < 2e-6
    assert np.array_equal(O.q8_embed(g["ids"], *q8_parts(t, "language_model.model.embed_tokens")), g["embed_rows"])


def test_q8_shared_expert_matches_reference():
    t, g = q8_small()
    pre = "language_model.model.layers.3.mlp."
    gate, up, down = (q8_parts(t, pre + f"shared_expert.{p}_proj") for p in ("gate", "up", "down"))
    gp, upj, out, scale = O.shared_expert_q8(g["x"], gate, up, down, O.bf16_bits_to_f32(t[pre + "shared_expert_gate.weight"][1]))
    assert rel_max(gp, g["sh8_shared_gate_proj"]) < 2e-6 and rel_max(upj, g["sh8_shared_up_proj"]) < 2e-6
    assert rel_max(out, g["sh8_shared_out"]) < 5e-6
    assert rel_max(scale, g["sh8_shared_scale"]) < 2e-6
    # the dense view the float64 block / stack references multiply by gives the same shared expert
    sh, sc = O.shared_expert(g["x"], O.AffineLinear(*gate), O.AffineLinear(*up), O.AffineLinear(*down),
                             O.bf16_bits_to_f32(t[pre + "shared_expert_gate.weight"][1]))
    assert rel_max(sh, g["sh8_shared_out"]) < 5e-6 and rel_max(sc.reshape(-1, 1), g["sh8_shared_scale"]) < 2e-6
