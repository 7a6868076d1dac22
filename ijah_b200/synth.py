"""Synthetic EXL3 MoE / trunk weights generated directly on the GPU (torch is only the allocator and the random
source here), with the same names, shapes and value distributions as ijah_b200.packgen writes to disk. Used by the
benchmark, where a full-size layer (1.5 GB of trellis words) should not cross PCIe."""
import torch

PFX = "language_model.model.layers."


def _exl3(gen, n_in, n_out, K, lead=(), device="cuda"):
    tr = torch.randint(-32768, 32768, (*lead, n_in // 16, n_out // 16, 16 * K), dtype=torch.int16, device=device, generator=gen)
    suh = (torch.randint(0, 2, (*lead, n_in), device=device, generator=gen) * 2 - 1).to(torch.float16)
    sign = (torch.randint(0, 2, (*lead, n_out), device=device, generator=gen) * 2 - 1).to(torch.float32)
    svh = (sign * torch.randn((*lead, n_out), device=device, generator=gen).abs() * 0.02).to(torch.float16)
    return tr, suh, svh


def moe_layer(seed, layer=0, hidden=2048, inter=768, experts=512, k_expert=5, k_shared=6, expert_first=0,
              expert_count=None, router_seed=None, device="cuda"):
    """name -> (dtype, tensor). Only experts [expert_first, expert_first + expert_count) are generated (the stacks have
    that many leading entries); the router covers all experts and depends on router_seed only, so ranks agree on it."""
    count = experts if expert_count is None else expert_count
    gr = torch.Generator(device=device).manual_seed(seed if router_seed is None else router_seed)
    g = torch.Generator(device=device).manual_seed(seed * 1000003 + expert_first + 17)
    pre = f"{PFX}{layer}.mlp."
    t = {pre + "gate.weight": ("BF16", (torch.randn((experts, hidden), device=device, generator=gr) * 0.02).to(torch.bfloat16)),
         pre + "shared_expert_gate.weight": ("BF16", (torch.randn((1, hidden), device=device, generator=gr) * 0.02).to(torch.bfloat16))}
    for proj, (a, b) in (("gate", (hidden, inter)), ("up", (hidden, inter)), ("down", (inter, hidden))):
        tr, su, sv = _exl3(gr, a, b, k_shared, device=device)
        t[f"{pre}shared_expert.{proj}_proj.trellis"] = ("U16", tr)
        t[f"{pre}shared_expert.{proj}_proj.suh"] = ("F16", su)
        t[f"{pre}shared_expert.{proj}_proj.svh"] = ("F16", sv)
        tr, su, sv = _exl3(g, a, b, k_expert, (count,), device=device)
        t[f"{pre}switch_mlp.{proj}_proj.trellis"] = ("U16", tr)
        t[f"{pre}switch_mlp.{proj}_proj.suh"] = ("F16", su)
        t[f"{pre}switch_mlp.{proj}_proj.svh"] = ("F16", sv)
    return t


def trunk_layer(seed, hidden=2048, q_out=4096, kv_out=512, K=6, device="cuda"):
    """the four attention projections of one layer as (trellis, suh, svh) triples: q, k, v (hidden -> q_out / kv_out) and o
    (q_out -> hidden)"""
    g = torch.Generator(device=device).manual_seed(seed * 7919 + 3)
    return {"q": _exl3(g, hidden, q_out, K, device=device), "k": _exl3(g, hidden, kv_out, K, device=device),
            "v": _exl3(g, hidden, kv_out, K, device=device), "o": _exl3(g, q_out, hidden, K, device=device)}


def zipf_router_bias(tensors, layer=0, s=1.1):
    """Skew the routing of a layer in place: router column 0 becomes -s * log(rank of the expert) (centred), so that with
    activations whose channel 0 is 1 the per-expert token counts follow a Zipf(s)-like law (the prefill configuration).
    The same on every rank."""
    w = tensors[f"{PFX}{layer}.mlp.gate.weight"][1]
    bias = -s * torch.log(torch.arange(1, w.shape[0] + 1, device=w.device, dtype=torch.float32))
    # popularity rank -> expert id by a fixed permutation (a popularity that falls with the expert id would put all hot
    # experts on the first expert-parallel rank)
    perm = torch.randperm(w.shape[0], generator=torch.Generator().manual_seed(4242)).to(w.device)
    col = torch.empty_like(bias)
    col[perm] = bias - bias.mean()
    w[:, 0] = col.to(torch.bfloat16)


def to_numpy(tensors):
    """the same dict with numpy arrays (uint16 for U16 / BF16, float16 for F16), for the CPU oracle"""
    import numpy as np
    out = {}
    for k, (dt, v) in tensors.items():
        a = v.cpu()
        if dt == "BF16":
            a = a.view(torch.int16).numpy().view(np.uint16)
        elif dt == "U16":
            a = a.numpy().view(np.uint16)
        else:
            a = a.numpy()
        out[k] = (dt, a)
    return out
