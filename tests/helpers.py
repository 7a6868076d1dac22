"""Shared test helpers: the seeded small pack of tests/golden and accessors over packgen tensor dicts."""
import importlib.util
from pathlib import Path

import numpy as np

from oracle import opref_port as O

GOLD = Path(__file__).resolve().parent / "golden"
_spec = importlib.util.spec_from_file_location("make_golden", GOLD / "make_golden.py")
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)

PFX = "language_model.model.layers."


def golden():
    return np.load(GOLD / "moe_small.npz")


def small_pack():
    """(tensors, golden) with the random-stream digest verified"""
    g = golden()
    t = make_golden.small_pack_tensors()
    assert make_golden.tensors_digest(t) == str(g["digest"]), "numpy random stream differs from the one that made the golden file"
    return t, g


def hc_small():
    """(hyper-connection tensors of layer 0, their golden file) with the digest verified"""
    g = np.load(GOLD / "hc_small.npz")
    t = make_golden.hc_tensors()
    assert make_golden.tensors_digest(t) == str(g["digest"]), "numpy random stream differs from the one that made the golden file"
    return t, g


def q8_small():
    """(8-bit affine LM head + embedding tensors, their golden file) with the digest verified"""
    g = np.load(GOLD / "q8_small.npz")
    t = make_golden.q8_tensors()
    t.update(make_golden.shared_q8_tensors())
    assert make_golden.tensors_digest(t) == str(g["digest"]), "numpy random stream differs from the one that made the golden file"
    return t, g


def q8_parts(tensors, name):
    return tuple(tensors[name + s][1] for s in (".weight", ".scales", ".biases"))


def hc_oracle(tensors, h, layer=0, which="mlp"):
    """oracle hyper-connection read over a packgen dict"""
    pre = f"{PFX}{layer}.{which}_hyper_connection."
    raw = lambda n: tensors[pre + n][1]  # noqa: E731
    dn = O.affine_dequant(raw("input_mix_weight_down.weight"), raw("input_mix_weight_down.scales"), raw("input_mix_weight_down.biases"))
    up = O.affine_dequant(raw("input_mix_weight_up.weight"), raw("input_mix_weight_up.scales"), raw("input_mix_weight_up.biases"))
    return O.hc_read(h, O.bf16_bits_to_f32(raw("hc_norm.weight")), O.bf16_bits_to_f32(raw("block_inject_weight.weight")), dn, up)


class MoeView:
    """Oracle-side view of one layer's MoE tensors in a packgen dict"""

    def __init__(self, tensors, layer=0):
        self.t, self.pre = tensors, f"{PFX}{layer}.mlp."
        self._cache = {}
        self.router = O.bf16_bits_to_f32(tensors[self.pre + "gate.weight"][1])
        self.sgate = O.bf16_bits_to_f32(tensors[self.pre + "shared_expert_gate.weight"][1])

    def raw(self, name):
        return self.t[self.pre + name][1]

    def expert(self, e):
        if e not in self._cache:
            self._cache[e] = tuple(
                O.Exl3Linear(self.raw(f"switch_mlp.{p}_proj.trellis")[e], self.raw(f"switch_mlp.{p}_proj.suh")[e],
                             self.raw(f"switch_mlp.{p}_proj.svh")[e]) for p in ("gate", "up", "down"))
        return self._cache[e]

    @property
    def shared(self):
        if "s" not in self._cache:
            self._cache["s"] = tuple(
                O.Exl3Linear(self.raw(f"shared_expert.{p}_proj.trellis"), self.raw(f"shared_expert.{p}_proj.suh"),
                             self.raw(f"shared_expert.{p}_proj.svh")) for p in ("gate", "up", "down"))
        return self._cache["s"]


def trunk_linear(tensors, layer, proj):
    pre = f"{PFX}{layer}.self_attn.{proj}_proj."
    return O.Exl3Linear(tensors[pre + "trellis"][1], tensors[pre + "suh"][1], tensors[pre + "svh"][1])


def rel_max(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
