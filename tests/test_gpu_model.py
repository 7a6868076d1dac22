"""The decoder stack behind ne_fn_model_* (graph-replayed decode step) against the CPU restatement of the same stack:
logits within KL < 1e-4 of the float64 operator reference, greedy token = argmax, replays bit-identical."""
import numpy as np
import pytest

from ijah_b200 import packgen
from oracle import c_oracle as CO
from oracle import opref_port as O
from oracle import stack_port as S
from tests.helpers import MoeView, trunk_linear

pytestmark = pytest.mark.gpu

CFG = dict(layers=3, hidden=512, inter=256, experts=32, top_k=4, heads=4, kv_heads=2, head_dim=64, vocab=2048)


def small_model_tensors(rng, fmt="bf16", kv_heads=None):
    t = {}
    kvh = kv_heads or CFG["kv_heads"]
    H, V = CFG["hidden"], CFG["vocab"]
    if fmt in ("q8", "q8all"):  # 8-bit affine embedding and head, the format of the reference's packs
        for name, std in (("language_model.model.embed_tokens", 1.0), ("language_model.lm_head", 0.1)):
            w, sc, bi = packgen.q8_linear(rng, V, H, 64, std=std)
            t[name + ".weight"], t[name + ".scales"], t[name + ".biases"] = ("U32", w), ("BF16", sc), ("BF16", bi)
    else:
        t["language_model.model.embed_tokens.weight"] = ("BF16", packgen.f32_to_bf16_bits(rng.standard_normal((V, H))))
        t["language_model.lm_head.weight"] = ("BF16", packgen.f32_to_bf16_bits(rng.standard_normal((V, H)) * 0.1))
    for l in range(CFG["layers"]):
        t.update(packgen.moe_layer(rng, layer=l, hidden=H, inter=CFG["inter"], experts=CFG["experts"]))
        if fmt == "q8all":  # a pack whose trunk stayed 8-bit affine: attention projections and the shared expert too
            for name in [n for n in t if f"layers.{l}.mlp.shared_expert." in n]:
                del t[name]
            t.update(packgen.shared_expert_q8(rng, layer=l, hidden=H, inter=CFG["inter"], group=64 if l else 32))
            t.update(packgen.trunk_layer_q8(rng, layer=l, hidden=H, q_out=CFG["heads"] * CFG["head_dim"],
                                            kv_out=kvh * CFG["head_dim"], group=64 if l else 128))
            continue
        t.update(packgen.trunk_layer(rng, layer=l, hidden=H, q_out=CFG["heads"] * CFG["head_dim"], kv_out=kvh * CFG["head_dim"],
                                     K=8 if l == 2 else 6))
    return t


class FastView(MoeView):
    def _lin(self, tr, su, sv):
        l = O.Exl3Linear(tr, su, sv)
        l._inner = CO.decode_inner(l.trellis)
        return l

    def expert(self, e):
        if e not in self._cache:
            self._cache[e] = tuple(self._lin(self.raw(f"switch_mlp.{p}_proj.trellis")[e], self.raw(f"switch_mlp.{p}_proj.suh")[e],
                                             self.raw(f"switch_mlp.{p}_proj.svh")[e]) for p in ("gate", "up", "down"))
        return self._cache[e]

    @property
    def shared(self):
        if "s" not in self._cache:
            self._cache["s"] = tuple(self._lin(self.raw(f"shared_expert.{p}_proj.trellis"), self.raw(f"shared_expert.{p}_proj.suh"),
                                               self.raw(f"shared_expert.{p}_proj.svh")) for p in ("gate", "up", "down"))
        return self._cache["s"]


def affine(t, name):
    return O.AffineLinear(*(t[name + s][1] for s in (".weight", ".scales", ".biases")))


class AffineSharedView(FastView):
    @property
    def shared(self):
        if "s" not in self._cache:
            self._cache["s"] = tuple(affine(self.t, f"{self.pre}shared_expert.{p}_proj") for p in ("gate", "up", "down"))
        return self._cache["s"]


@pytest.fixture(scope="module")
def eng():
    import torch
    assert torch.cuda.is_available()
    from ijah_b200 import engine as E
    return E.Engine()


# (weight format, cached positions, KV heads): the long caches make the attention stand-in take its 128- and 256-position blocks
@pytest.mark.parametrize("fmt,tmax,kvh", [("bf16", 128, 2), ("q8", 128, 2), ("q8all", 128, 2), ("bf16", 8192, 2), ("q8", 8192, 4)])
def test_stack_logits_match_the_operator_reference(eng, tmp_path, fmt, tmax, kvh):
    rng = np.random.default_rng(2025)
    t = small_model_tensors(rng, fmt, kvh)
    cfg = {"num_hidden_layers": CFG["layers"], "num_attention_heads": CFG["heads"], "num_key_value_heads": kvh,
           "head_dim": CFG["head_dim"], "num_experts_per_tok": CFG["top_k"], "vocab_size": CFG["vocab"]}
    packgen.write_pack(tmp_path / "model", t, cfg, shards=4, misalign=2)
    p = eng.pack_open(tmp_path / "model")
    m = eng.fn_model(p, tmax=tmax, max_rows=8)
    p.close()  # the model keeps the pack alive
    assert m.desc["layers"] == 3 and m.desc["kv_positions"] == tmax and m.desc["k_trunk"] == (8 if fmt == "q8all" else 6)
    tokens = np.array([5, 77, 1999, 0, 1024], np.int32)
    nxt, logits, ms = m.step_rows(tokens, want_logits=True)
    assert eng.lib.ne_device_wait_status() == 0
    assert np.array_equal(nxt, logits.argmax(1)), "greedy token must be the argmax of the returned logits"
    # CPU restatement of the same stack on the same weights and the KV cache the library generated
    layers = []
    for l in range(CFG["layers"]):
        kv = (tmax, kvh, CFG["head_dim"])
        if fmt == "q8all":
            proj = {n: affine(t, f"{packgen.PFX}{l}.self_attn.{n}_proj") for n in ("q", "k", "v", "o")}
        else:
            proj = {n: trunk_linear(t, l, n) for n in ("q", "k", "v", "o")}
            for n in proj:
                proj[n]._inner = CO.decode_inner(proj[n].trellis)
        layers.append(dict(**proj, view=(AffineSharedView if fmt == "q8all" else FastView)(t, l), kc=m.read("kv_k", l).reshape(kv),
                           vc=m.read("kv_v", l).reshape(kv)))
    q8 = (lambda n: tuple(t[n + s][1] for s in (".weight", ".scales", ".biases"))) if fmt != "bf16" else (lambda n: None)
    want = S.stack_logits(tokens, t["language_model.model.embed_tokens.weight"][1], t["language_model.lm_head.weight"][1], layers,
                          CFG["heads"], kvh, CFG["head_dim"], CFG["top_k"], embed_q8=q8("language_model.model.embed_tokens"),
                          head_q8=q8("language_model.lm_head"))
    kl = S.kl(want, logits)
    assert kl.max() < 1e-4, kl
    assert np.abs(logits - want).max() / np.abs(want).max() < 1e-2
    # replays of the captured step are bit-identical; the one-token entry point of the reference gives row 0
    nxt2, logits2, _ = m.step_rows(tokens, want_logits=True)
    assert np.array_equal(logits, logits2) and np.array_equal(nxt, nxt2)
    lg1, n1, lp1, _ = m.step(int(tokens[0]))
    assert n1 == nxt[0] and S.kl(want[:1], lg1[None])[0] < 1e-4
    lref = want[0] - want[0].max()
    assert abs(lp1 - (lref[n1] - np.log(np.exp(lref).sum()))) < 1e-2
    info = m.info()
    per_layer = 18 if fmt == "q8all" else 16  # four 8-bit Linears instead of two 3-kernel chains; + the shared expert's 4
    assert info["launches_full"] == 1 + CFG["layers"] * per_layer + 1 + (4 if fmt == "bf16" else 3) and info["T"] == tmax
    a, b, c = m.time(reps=3)
    assert 0 < b <= a and c > 0
    m.free()


def test_synthetic_stack_runs_and_is_deterministic(eng):
    d = dict(layers=2, hidden=512, inter=256, experts=32, top_k=4, k_expert=5, k_shared=6, q_out=256, kv_out=128, heads=4, kv_heads=2,
             head_dim=64, k_trunk=6, k_trunk_alt=8, alt_every=2, vocab=1024, kv_positions=64, expert_first=0, expert_count=0)
    a = eng.fn_model(desc=d, seed=7, max_rows=16)
    b = eng.fn_model(desc=d, seed=7, max_rows=16)
    tokens = np.arange(16, dtype=np.int32) * 13 % 1024
    na, la, _ = a.step_rows(tokens, want_logits=True)
    nb, lb, _ = b.step_rows(tokens, want_logits=True)
    assert np.array_equal(la, lb) and np.array_equal(na, nb), "equal seeds must give equal models"
    assert np.isfinite(la).all() and la.std() > 0
    # a row's logits do not depend on which other rows share the step (up to the summation order of the k-splits)
    n1, l1, _ = a.step_rows(tokens[3:4], want_logits=True)
    assert np.abs(l1[0] - la[3]).max() / np.abs(la[3]).max() < 1e-4
    # prompt prefill: chunks of max_rows rows, the head on the last chunk; its last row equals that token's own step
    prompt = (np.arange(37, dtype=np.int32) * 29 + 3) % 1024
    nx, lg, ms = a.prefill(prompt)
    _, l5, _ = a.step_rows(prompt[32:37], want_logits=True)  # the last chunk (37 = 16 + 16 + 5)
    assert np.array_equal(lg, l5[4]) and nx == int(l5[4].argmax()) and ms > 0
    # one speculative round: drafts that are the model's own greedy continuations are all accepted (+ the bonus token),
    # a wrong draft cuts the run there and is replaced by the model's choice
    t1 = int(tokens[0])
    chain = [t1]
    for _ in range(3):
        nj, _, _ = a.step_rows(np.array(chain, np.int32))
        chain.append(int(nj[-1]))
    # (the stand-in attention has no causal state: a row's output depends on its own token only, so chain[j + 1] is what
    # the model picks after chain[j] in any batch)
    acc, emitted, _ = a.verify_greedy(chain)
    assert acc == 3 and list(emitted[:3]) == chain[1:] and len(emitted) == 4
    bad = list(chain)
    bad[2] = (bad[2] + 1) % 1024
    acc, emitted, _ = a.verify_greedy(bad)
    assert acc == 1 and list(emitted) == [chain[1], chain[2]]
    assert a.weight_bytes() > 0 and a.last_bytes(16)["total"] > 0
    assert eng.lib.ne_device_wait_status() == 0
    a.free()
    b.free()
