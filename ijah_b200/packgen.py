"""Synthetic EXL3 packs in the reference's on-disk layout (safetensors shards + model.safetensors.index.json +
config.json), for tests and benchmarks when no real pack is at hand.

Tensor names and shapes are the ones the reference's layer loader reads (models/flash_next/layer.mm:136-147,180-197):
  <pre>mlp.gate.weight                                   BF16 [E, H]        router
  <pre>mlp.shared_expert_gate.weight                     BF16 [1, H]
  <pre>mlp.switch_mlp.{gate,up,down}_proj.trellis        U16  [E, in/16, out/16, 16K]
  <pre>mlp.switch_mlp.{gate,up,down}_proj.{suh,svh}      F16  [E, in] / [E, out]
  <pre>mlp.shared_expert.{gate,up,down}_proj.{trellis,suh,svh}   (no leading E)
  <pre>self_attn.{q,k,v,o}_proj.{trellis,suh,svh}
  <pre>mlp_hyper_connection.hc_norm.weight               BF16 [4H]          (layer.mm:81-94)
  <pre>mlp_hyper_connection.block_inject_weight.weight   BF16 [4, 4H]
  <pre>mlp_hyper_connection.input_mix_weight_{down,up}.{weight U32 [rows, in/4], scales BF16 [rows, in/G], biases}
with <pre> = "language_model.model.layers.<L>.". Value distributions: trellis words uniform random (every bit pattern
is a valid tail-biting ring), suh uniform +-1, svh = sign * |N(0,1)| * 0.02 (the format has no separate scale tensor),
router / shared gate ~ N(0, 0.02) rounded to bf16.
"""
import json
import struct
from pathlib import Path

import numpy as np

PFX = "language_model.model.layers."
_DT = {"BF16": np.uint16, "F16": np.float16, "U16": np.uint16, "F32": np.float32, "U32": np.uint32}


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) >> 16).astype(np.uint16)


def exl3_linear(rng, n_in, n_out, K, lead=()):
    """(trellis u16 [*lead, in/16, out/16, 16K], suh f16 [*lead, in], svh f16 [*lead, out])"""
    tr = rng.integers(0, 1 << 16, (*lead, n_in // 16, n_out // 16, 16 * K), dtype=np.uint16)
    suh = rng.choice(np.array([-1.0, 1.0], np.float16), (*lead, n_in))
    svh = (np.where(rng.random((*lead, n_out)) < 0.5, -1.0, 1.0) * np.abs(rng.standard_normal((*lead, n_out))) * 0.02)
    return tr, suh.astype(np.float16), svh.astype(np.float16)


def shared_expert_q8(rng, layer=0, hidden=2048, inter=768, group=64):
    """name -> (dtype, array): the shared expert of one layer as three 8-bit affine Linears + its bf16 sigmoid gate (the
    format of packs whose trunk was not converted to EXL3)"""
    pre = f"{PFX}{layer}.mlp."
    t = {pre + "shared_expert_gate.weight": ("BF16", f32_to_bf16_bits(rng.standard_normal((1, hidden)) * 0.02))}
    for proj, (n_out, n_in) in (("gate", (inter, hidden)), ("up", (inter, hidden)), ("down", (hidden, inter))):
        w, sc, bi = q8_linear(rng, n_out, n_in, group, std=1.0 / np.sqrt(n_in))
        t[f"{pre}shared_expert.{proj}_proj.weight"] = ("U32", w)
        t[f"{pre}shared_expert.{proj}_proj.scales"] = ("BF16", sc)
        t[f"{pre}shared_expert.{proj}_proj.biases"] = ("BF16", bi)
    return t


def moe_layer(rng, layer=0, hidden=2048, inter=768, experts=512, k_expert=5, k_shared=6):
    """name -> (safetensors dtype, array) for the MoE block of one layer"""
    pre = f"{PFX}{layer}.mlp."
    t = {pre + "gate.weight": ("BF16", f32_to_bf16_bits(rng.standard_normal((experts, hidden)) * 0.02)),
         pre + "shared_expert_gate.weight": ("BF16", f32_to_bf16_bits(rng.standard_normal((1, hidden)) * 0.02))}
    for proj, (a, b) in (("gate", (hidden, inter)), ("up", (hidden, inter)), ("down", (inter, hidden))):
        tr, su, sv = exl3_linear(rng, a, b, k_expert, (experts,))
        t[f"{pre}switch_mlp.{proj}_proj.trellis"] = ("U16", tr)
        t[f"{pre}switch_mlp.{proj}_proj.suh"] = ("F16", su)
        t[f"{pre}switch_mlp.{proj}_proj.svh"] = ("F16", sv)
        tr, su, sv = exl3_linear(rng, a, b, k_shared)
        t[f"{pre}shared_expert.{proj}_proj.trellis"] = ("U16", tr)
        t[f"{pre}shared_expert.{proj}_proj.suh"] = ("F16", su)
        t[f"{pre}shared_expert.{proj}_proj.svh"] = ("F16", sv)
    return t


def q8_linear(rng, rows, n_in, group=64, std=0.02):
    """8-bit affine Linear in the MLX layout: (weight u32 [rows, in/4] = bytes little-endian, scales, biases bf16 bits
    [rows, in/group]); w = scale * q + bias, roughly N(0, std)"""
    q = np.clip(np.rint(rng.standard_normal((rows, n_in)) * 32 + 128), 0, 255).astype(np.uint8)
    sc = (std / 32) * (1 + 0.1 * rng.standard_normal((rows, n_in // group)))
    bi = -128 * sc + 0.1 * std * rng.standard_normal((rows, n_in // group))
    return np.ascontiguousarray(q).view(np.uint32), f32_to_bf16_bits(sc), f32_to_bf16_bits(bi)


def hc_block(rng, layer=0, which="mlp", hidden=2048, lr=320, group=64, streams=4):
    """name -> (dtype, array) for one hyper-connection read (the reference's sizes: hidden 2560, lr 320, group 64)"""
    pre = f"{PFX}{layer}.{which}_hyper_connection."
    hcd = streams * hidden
    t = {pre + "hc_norm.weight": ("BF16", f32_to_bf16_bits(1 + 0.1 * rng.standard_normal(hcd))),
         pre + "block_inject_weight.weight": ("BF16", f32_to_bf16_bits(rng.standard_normal((streams, hcd)) * 0.02))}
    for name, (rows, n_in) in (("input_mix_weight_down", (lr, hcd)), ("input_mix_weight_up", (hcd, lr))):
        w, sc, bi = q8_linear(rng, rows, n_in, group, std=2.0 / np.sqrt(n_in))
        t[pre + name + ".weight"] = ("U32", w)
        t[pre + name + ".scales"] = ("BF16", sc)
        t[pre + name + ".biases"] = ("BF16", bi)
    return t


def trunk_layer(rng, layer=0, hidden=2048, q_out=4096, kv_out=512, K=6):
    """name -> (dtype, array) for the attention projections q, k, v, o of one layer"""
    pre = f"{PFX}{layer}.self_attn."
    t = {}
    for proj, (a, b) in (("q", (hidden, q_out)), ("k", (hidden, kv_out)), ("v", (hidden, kv_out)), ("o", (q_out, hidden))):
        tr, su, sv = exl3_linear(rng, a, b, K)
        t[f"{pre}{proj}_proj.trellis"] = ("U16", tr)
        t[f"{pre}{proj}_proj.suh"] = ("F16", su)
        t[f"{pre}{proj}_proj.svh"] = ("F16", sv)
    return t


def trunk_layer_q8(rng, layer=0, hidden=2048, q_out=4096, kv_out=512, group=64):
    """the attention projections of one layer as 8-bit affine Linears (packs whose trunk was not converted to EXL3)"""
    pre = f"{PFX}{layer}.self_attn."
    t = {}
    for proj, (n_in, n_out) in (("q", (hidden, q_out)), ("k", (hidden, kv_out)), ("v", (hidden, kv_out)), ("o", (q_out, hidden))):
        w, sc, bi = q8_linear(rng, n_out, n_in, group, std=1.0 / np.sqrt(n_in))
        t[f"{pre}{proj}_proj.weight"] = ("U32", w)
        t[f"{pre}{proj}_proj.scales"] = ("BF16", sc)
        t[f"{pre}{proj}_proj.biases"] = ("BF16", bi)
    return t


def write_shard(path, tensors, misalign=0):
    """One safetensors file. `misalign` extra header bytes reproduce the real packs' odd data offsets (the reference
    needs Pack::aligned for those, core/pack.mm:254-268)."""
    hdr, off = {}, 0
    for name, (dt, arr) in tensors.items():
        n = int(np.asarray(arr).nbytes)
        hdr[name] = {"dtype": dt, "shape": list(np.shape(arr)), "data_offsets": [off, off + n]}
        off += n
    hdr["__metadata__"] = {"format": "pt"}
    blob = json.dumps(hdr, separators=(",", ":")).encode()
    blob += b" " * ((-len(blob)) % 8 + misalign)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, (dt, arr) in tensors.items():
            f.write(np.ascontiguousarray(arr, dtype=_DT[dt]).tobytes())


def write_pack(directory, tensors, config=None, shards=2, misalign=0):
    """Split `tensors` over `shards` files, write the index and config.json. Returns the directory."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    names = list(tensors)
    per = max(1, -(-len(names) // shards))
    wm = {}
    nsh = -(-len(names) // per)
    for i in range(nsh):
        fn = f"model-{i + 1:05d}-of-{nsh:05d}.safetensors"
        part = {n: tensors[n] for n in names[i * per:(i + 1) * per]}
        write_shard(d / fn, part, misalign)
        wm.update({n: fn for n in part})
    (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}, indent=1))
    cfg = {"expert_quant": {"codebook": "mcg", "window": 15}, "num_experts_per_tok": 10}
    cfg.update(config or {})
    (d / "config.json").write_text(json.dumps(cfg, indent=1))
    return d
