"""Benchmark of the EXL3 MoE decoder hot path on B200 (one JSON line on stdout).

Headline workload (`config.workload`): one decode step of a random-init 48-layer MoE decoder stack -- hidden 2048, vocab
151936 (bf16 embedding and LM head), per layer the trunk projections q 2048->4096, k / v 2048->512, o 4096->2048 at K6
(every fourth layer K8), an attention stand-in over a fixed cache of 8192 random fp16 positions (16 query / 2 KV heads of
dimension 256), and the MoE block: 512 routed experts (top-10, intermediate 768, K5) plus one shared expert (K6) -- for
`--batch` concurrent sequences x `--verify` tokens each (default 2 x 4 = 8 rows per GPU). The whole step runs inside
libijah_b200.so behind ne_fn_model_* and is replayed from a CUDA graph the library owns; weights are generated on the
device by the library (about 75 GB resident on one GPU). value = rows / step time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--verify M] [--impl reference] [--workload stack|block|q8head]

N > 1 (under torchrun): expert parallel, weak scaling. Every rank holds experts/N experts of every layer and B x M rows of
its own; per MoE block the ranks exchange rows and partial outputs over NVLink peer memory (the library's own kernels),
everything else is replicated. value = N * rows / step time. Rank 0 also holds the full model and checks the ranks' logits
against a single-GPU step over all rows (`ep_check`).

`e2e` is the same step through ne_fn_model_step_rows with the token ids in host memory and the sampled ids copied back.
`roofline` is the dominant kernel (the gate/up stream GEMM of the MoE block) timed alone over layers with distinct weights.
`--workload block` times the MoE block alone (the earlier headline; also what the ncu recipes under profiles/ run);
`--workload q8head` the 8-bit affine Linear at the reference's LM head size.

--impl reference: the CPU restatement of the reference's operator path (oracle/, C with all host threads) on a bounded
sample of the same workload; the reference's own code for this path is Metal / numpy-with-a-missing-module and cannot run
on this box.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

DIMS = dict(hidden=2048, inter=768, experts=512, k_expert=5, k_shared=6)
TOPK = 10
STACK = dict(layers=48, hidden=2048, inter=768, experts=512, top_k=TOPK, k_expert=5, k_shared=6, q_out=4096, kv_out=512, heads=16,
             kv_heads=2, head_dim=256, k_trunk=6, k_trunk_alt=8, alt_every=4, vocab=151936, kv_positions=8192)
METRIC = "EXL3 MoE decoder stack decode tok/s"
BLOCK_METRIC = "EXL3 MoE decode tok/s (rows through one MoE block)"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# DRAM bytes (read + write) per algorithmic byte of the gate/up stream launch, from the ncu capture summarised in
# profiles/stream_gemm_moe_decode.md (8 rows, one layer: 153.31 MB read + 4.21 MB written for 152.65 MB of compressed weights;
# the writes are the k-split partial sums). The full-size launch processes the same units, only more of them, so the traffic
# reported beside the roofline is this ratio times the launch's algorithmic bytes.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = (153.31 + 4.21) / 152.65


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed regions (read-only query)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        for line in Path(self.path).read_text().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
                pw.append(float(c[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            busy = [s for s, p in zip(sm, pw) if p > 0.5 * max(pw)]  # samples taken under load
            out = {"sm_mhz": float(np.median(busy or sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                   "samples_under_load": len(busy), "power_w_max": max(pw)}
        return out


# ---------------------------------------------------------------------------------------------- CPU legs (oracle/)
_CPU_LAYER = {}


def cpu_layer():
    """one full-size MoE layer (512 experts) and one trunk layer as host arrays for the CPU legs"""
    if not _CPU_LAYER:
        from ijah_b200 import packgen
        rng = np.random.default_rng(0)
        _CPU_LAYER["moe"] = packgen.moe_layer(rng, **DIMS)
        _CPU_LAYER["trunk"] = packgen.trunk_layer(rng, hidden=STACK["hidden"], q_out=STACK["q_out"], kv_out=STACK["kv_out"], K=6)
    return _CPU_LAYER["moe"], _CPU_LAYER["trunk"]


def cpu_port_layer_seconds(rows, budget_s):
    """The C oracle (device-arithmetic restatement of the reference's operators, all host threads) on ONE decoder layer of
    the workload: the four trunk projections and the MoE block (router, top-10 of 512 experts, shared expert) for `rows`
    rows, repeated until about budget_s seconds have passed. Returns (seconds per layer, threads, layers done)."""
    from oracle import c_oracle as CO
    moe, trunk = cpu_layer()
    pre = "language_model.model.layers.0.self_attn."
    rng = np.random.default_rng(1)
    x = rng.standard_normal((rows, STACK["hidden"])).astype(np.float16).astype(np.float32)
    xo = rng.standard_normal((rows, STACK["q_out"])).astype(np.float16).astype(np.float32)

    def layer():
        for p_ in ("q", "k", "v"):
            CO.linear_emul(trunk[pre + p_ + "_proj.trellis"][1], trunk[pre + p_ + "_proj.suh"][1], trunk[pre + p_ + "_proj.svh"][1], x)
        CO.linear_emul(trunk[pre + "o_proj.trellis"][1], trunk[pre + "o_proj.suh"][1], trunk[pre + "o_proj.svh"][1], xo)
        CO.moe_block_emul(moe, x, top_k=TOPK)

    n, t0 = 0, time.perf_counter()
    while True:
        layer()
        n += 1
        el = time.perf_counter() - t0
        if el > budget_s or n >= 200:
            break
    return el / n, CO.threads(), n


def cpu_numpy_row_seconds():
    """The numpy restatement of the reference's tools/opref.py operators (float64 dense reconstruction of every touched
    expert, BLAS threads as numpy has them) on ONE row of one MoE block. Returns seconds."""
    from oracle import c_oracle as CO
    from oracle import opref_port as O
    moe, _ = cpu_layer()
    pre = "language_model.model.layers.0.mlp."
    rng = np.random.default_rng(2)
    x = rng.standard_normal((1, STACK["hidden"])).astype(np.float16).astype(np.float32)

    def lin(tr, su, sv):
        l = O.Exl3Linear(tr, su, sv)
        l._inner = CO.decode_inner(l.trellis)  # the codec table lookup itself in C: the numpy codec would take most of the time
        return l

    def expert(e):
        return tuple(lin(moe[f"{pre}switch_mlp.{p}_proj.trellis"][1][e], moe[f"{pre}switch_mlp.{p}_proj.suh"][1][e],
                         moe[f"{pre}switch_mlp.{p}_proj.svh"][1][e]) for p in ("gate", "up", "down"))

    shared = tuple(lin(moe[f"{pre}shared_expert.{p}_proj.trellis"][1], moe[f"{pre}shared_expert.{p}_proj.suh"][1],
                       moe[f"{pre}shared_expert.{p}_proj.svh"][1]) for p in ("gate", "up", "down"))
    t0 = time.perf_counter()
    O.moe_block_exact(x, O.bf16_bits_to_f32(moe[pre + "gate.weight"][1]), O.bf16_bits_to_f32(moe[pre + "shared_expert_gate.weight"][1]), expert,
                      shared, TOPK)
    return time.perf_counter() - t0


def arithmetic(a):
    if a.summand_product:
        return "opt-in summand product: weights as their two f16 summands (sum unrounded), f16 activations, f32 accumulate"
    return "weights decoded to f16 (the format's rounded values), f16 activations, f32 accumulate"


def stack_config(a, rows):
    return {"workload": f"decoder stack decode step: {a.layers} layers (EXL3 trunk q/k/v/o K6/K8 + attention stand-in over 8192 cached positions + "
                        f"MoE block 512 experts top-10 K5 + shared K6), bf16 LM head 151936 x 2048; {a.batch} sequences x {a.verify} verify "
                        f"tokens = {rows} rows per GPU",
            "arithmetic": arithmetic(a), "rows": rows, "layers": a.layers,
            "l2": "weights of a step (tens of GB) exceed L2", "parallelism": "single GPU" if a.gpus == 1 else f"ep{a.gpus}"}


def run_reference(a, rank):
    if rank != 0:
        return
    rows = a.batch * a.verify if a.workload == "stack" else a.rows
    per_step = max(2.0, min(20.0, 120.0 / max(a.steps + a.warmup, 1)))
    vals, cores, done = [], 1, 0
    for i in range(a.warmup + a.steps):
        sec, cores, n = cpu_port_layer_seconds(rows, per_step)
        done = n
        if i >= a.warmup:
            vals.append(sec)
    sec = float(np.mean(vals))
    layers = a.layers if a.workload == "stack" else 1
    v = rows / (sec * layers)
    sample = (f"each step: {done} x one decoder layer (4 trunk projections + MoE block on a full 512-expert layer) for {rows} rows in the C "
              f"port; tok/s = rows / (seconds per layer x {layers} layers); LM head and attention stand-in not included")
    print(json.dumps({
        "impl": "reference", "metric": METRIC if a.workload == "stack" else BLOCK_METRIC, "value": v, "unit": "tok/s", "n_gpus": a.gpus,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": 1e3 * rows / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": stack_config(a, rows) if a.workload == "stack" else block_config(a),
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def block_config(a):
    return {"workload": f"MoE block decode: hidden 2048, 512 experts top-10, inter 768, K5 routed + K6 shared, rows {a.rows}",
            "arithmetic": arithmetic(a), "rows": a.rows, "layers": a.layers,
            "l2": "weights of a step exceed L2 (distinct layers cycled)", "parallelism": "single GPU" if a.gpus == 1 else f"ep{a.gpus}"}


# ---------------------------------------------------------------------------------------------- MoE block figures
def block_figures(eng, rows, layers, steps, dev, want_kernels=True):
    """The MoE block alone at `rows` rows over `layers` layers with distinct weights (one CUDA graph per pass): block time and,
    timed alone, the gate/up and down stream-GEMM launches. Returns a dict; frees its weights."""
    import torch
    from ijah_b200 import engine as E
    from ijah_b200 import synth
    peak, which = peaks()
    H = DIMS["hidden"]
    blocks = [E.MoeBlock(eng, synth.moe_layer(1000 + l, router_seed=77 + l, device=dev, **DIMS), top_k=TOPK, max_rows=rows, device=dev)
              for l in range(layers)]
    g = torch.Generator(device=dev).manual_seed(5)
    xs = [torch.randn((rows, H), device=dev, generator=g).to(torch.float16).to(torch.float32) for _ in range(layers)]
    ys = [torch.empty((rows, H), device=dev) for _ in range(layers)]

    def timed_graph(fn, n):
        fn()
        torch.cuda.synchronize()
        gk = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gk):
            fn()
        gk.replay()
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(n):
            gk.replay()
        k1.record()
        torch.cuda.synchronize()
        return k0.elapsed_time(k1) * 1e3 / n / layers

    def fwd():
        for l in range(layers):
            blocks[l].forward(xs[l], out=ys[l])

    def stage(code):
        def f():
            for l in range(layers):
                blocks[l].stage(code, xs[l], ys[l])
        return f

    n = max(5, min(steps, 20))
    out = {"rows": rows, "block_us": timed_graph(fwd, n)}
    lbs = [b.last_bytes(rows) for b in blocks]
    out["block_bytes"] = float(np.mean([x["total"] for x in lbs]))
    out["block_gbs"] = out["block_bytes"] / out["block_us"] / 1e3
    out["distinct_experts_mean"] = float(np.mean([x["distinct_experts"] for x in lbs]))
    if want_kernels:
        for c in (7, 80):
            stage(c)()
        gu_us = timed_graph(stage(81), n)
        for c in (81, 90):
            stage(c)()
        dn_us = timed_graph(stage(91), n)
        gu_b = float(np.mean([x["gateup"] for x in lbs]))
        dn_b = float(np.mean([x["down"] for x in lbs]))
        out.update(gateup_us=gu_us, gateup_bytes=gu_b, gateup_gbs=gu_b / gu_us / 1e3, gateup_frac=gu_b / gu_us / 1e3 / peak,
                   down_us=dn_us, down_bytes=dn_b, down_gbs=dn_b / dn_us / 1e3, down_frac=dn_b / dn_us / 1e3 / peak)
    status = eng.lib.ne_device_wait_status()
    assert status == 0, f"a device-side bounded wait gave up ({status})"
    for b in blocks:
        b.free()
    del blocks, xs, ys
    torch.cuda.empty_cache()
    return out


def prefill_figure(eng, n_pf, dev):
    import torch
    from ijah_b200 import engine as E
    from ijah_b200 import synth
    last = synth.moe_layer(1007, router_seed=84, device=dev, **DIMS)
    synth.zipf_router_bias(last)
    pblk = E.MoeBlock(eng, last, top_k=TOPK, max_rows=16, device=dev)
    gp = torch.Generator(device=dev).manual_seed(99)
    xp = torch.randn((n_pf, DIMS["hidden"]), device=dev, generator=gp).to(torch.float16).to(torch.float32)
    xp[:, 0] = 1.0
    yp = torch.empty_like(xp)
    for _ in range(3):
        pblk.prefill(xp, out=yp)
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for _ in range(5):
        pblk.prefill(xp, out=yp)
    p1.record()
    torch.cuda.synchronize()
    pms = p0.elapsed_time(p1) / 5
    flop = n_pf * TOPK * 3 * 2 * DIMS["hidden"] * DIMS["inter"]
    tpeak = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"] if (ROOT / "MEASURED_PEAKS.json").exists() else 1590.0
    pblk.free()
    return {"tokens": n_pf, "ms": pms, "tok_per_s": n_pf / pms * 1e3, "routed_tflops": flop / pms / 1e9,
            "frac_of_dense_f16_peak": flop / pms / 1e9 / tpeak, "routing": "Zipf(1.1) bias on the router logits"}


def prefill_ep_figure(eng, dev, rank, world, n_total):
    """Expert-parallel prefill of n_total tokens split evenly over the ranks (strong scaling against the single-GPU
    `prefill` figure): the all-to-all form (ep.prefill_a2a) and the all-gather + reduce-scatter form, device-timed, max
    over ranks. Every rank calls this."""
    import torch
    import torch.distributed as dist
    from ijah_b200 import engine as E
    from ijah_b200 import ep, synth
    per, n = DIMS["experts"] // world, n_total // world
    last = synth.moe_layer(1007, router_seed=84, device=dev, expert_first=rank * per, expert_count=per, **DIMS)
    synth.zipf_router_bias(last)
    blk = E.MoeBlock(eng, last, top_k=TOPK, max_rows=16, expert_first=rank * per, expert_count=per, device=dev)
    par = ep.ExpertParallelMoe(blk, dist.group.WORLD)
    gp = torch.Generator(device=dev).manual_seed(99 + rank)
    xp = torch.randn((n, DIMS["hidden"]), device=dev, generator=gp).to(torch.float16).to(torch.float32)
    xp[:, 0] = 1.0
    yp = torch.empty_like(xp)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(5):
            fn()
        t1.record()
        torch.cuda.synchronize()
        tt = torch.tensor([t0.elapsed_time(t1) / 5], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt[0])

    a2a = timed(lambda: par.prefill_a2a(xp, out=yp))
    gat = timed(lambda: par.forward(xp, out=yp, prefill=True))
    # one more all-to-all call with a device synchronisation after every stage: where the time goes on each rank
    marks = [("start", time.perf_counter())]

    def mark(name):
        torch.cuda.synchronize()
        marks.append((name, time.perf_counter()))

    par.prefill_a2a(xp, out=yp)  # the other form ran last: let the block's prefill scratch settle at this form's sizes again
    torch.cuda.synchronize()
    dist.barrier()
    marks[0] = ("start", time.perf_counter())
    par.prefill_a2a(xp, out=yp, mark=mark)
    mine = {"pairs_received": par.last_pairs_received}
    mine.update({nm: round((t - marks[i][1]) * 1e3, 3) for i, (nm, t) in enumerate(marks[1:])})
    stages = [None] * world
    dist.all_gather_object(stages, mine)
    blk.free()
    return {"tokens_total": n * world, "tokens_per_rank": n, "all_to_all_ms": a2a, "all_to_all_tok_per_s": n * world / a2a * 1e3,
            "allgather_reduce_ms": gat, "routing": "Zipf(1.1) bias on the router logits",
            "all_to_all_stage_ms_per_rank": stages,
            "note": "the single-GPU time of the same token count is extra.prefill.ms of the N = 1 line"}


# ---------------------------------------------------------------------------------------------- the stack (headline)
def run_stack(a, rank, world):
    import torch
    import torch.distributed as dist
    from ijah_b200 import engine as E
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE {world}"
    eng = E.Engine()
    if a.summand_product:
        eng.lib.ne_exl3_set_summand_product(1)
    N, rows = world, a.batch * a.verify
    assert rows * N <= 64, f"{rows} rows x {N} ranks: the decode-width MoE block takes at most 64 gathered rows"
    per = STACK["experts"] // N
    desc = dict(STACK, layers=a.layers, expert_first=rank * per, expert_count=per, ep_world=N)
    max_rows = 64 if N == 1 else rows
    model = eng.fn_model(desc=desc, seed=a.seed, max_rows=max_rows)
    xchg = None
    if N > 1:
        from ijah_b200 import ep
        xchg = ep.ExpertParallelMoe.make_exchange(eng, dist.group.WORLD, rows, STACK["hidden"], TOPK)
        assert xchg is not None, "the NVLink peer-memory exchange could not be set up on every rank"
        model.set_ep(xchg)

    def barrier():
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()

    rng = np.random.default_rng(100 + rank)
    tokens = rng.integers(0, STACK["vocab"], rows).astype(np.int32)
    for _ in range(a.warmup):
        model.step_rows(tokens)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- value: exactly K replays of the captured step, inputs resident, device-timed on the model's stream
    barrier()
    ms = model.replay(rows, a.steps)
    barrier()
    # ---- e2e: K steps through the host-buffer entry point (token ids in, sampled ids out), wall clock
    t0 = time.perf_counter()
    for _ in range(a.steps):
        nxt, _, _ = model.step_rows(tokens)
    barrier()
    e2e_s = time.perf_counter() - t0
    # ---- sustained: at least about 2 s of back-to-back replays (clocks settle under load)
    k_sus = max(a.steps, int(2000.0 / max(ms / a.steps, 1e-3)) + 1) if a.sustain else 0
    ms_sus = model.replay(rows, k_sus) if k_sus else None
    barrier()
    # ---- strong scaling: the SAME total number of rows as one GPU's step (rows), split over the N ranks
    ms_strong, rs = None, max(1, rows // N)
    if N > 1 and a.extras and rs * N == rows:
        model.step_rows(tokens[:rs])
        barrier()
        ms_strong = model.replay(rs, a.steps)
        barrier()
        model.step_rows(tokens)  # the byte accounting below reads the last step's routing: make that the headline step again
        barrier()
    if N > 1:
        tt = torch.tensor([ms, e2e_s, ms_sus or 0.0, ms_strong or 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_s, ms_sus, ms_strong = float(tt[0]), float(tt[1]), float(tt[2]) or None, float(tt[3]) or None
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / a.steps
    value = N * rows / (ms_per_step * 1e-3)
    info = model.info()
    lb = model.last_bytes(rows)
    wbytes = model.weight_bytes()
    status = eng.lib.ne_device_wait_status()
    peak, which = peaks()
    extra = {"weights_gb_resident": wbytes / 1e9, "distinct_experts_per_layer": lb["distinct_experts_mean"],
             "step": {"bytes": lb["total"], "gbs": lb["total"] / (ms_per_step * 1e-3) / 1e9, "frac_of_hbm": lb["total"] / (ms_per_step * 1e-3) / 1e9 / peak},
             "graph": True, "exchange": "nvlink peer memory (own kernels)" if N > 1 else None}
    if ms_strong:
        extra["strong_scaling"] = {"total_rows": rs * N, "rows_per_rank": rs, "ms_per_step": ms_strong / a.steps,
                                   "tok_per_s": rs * N * a.steps / (ms_strong * 1e-3),
                                   "note": f"the same {rs * N} rows as the N = 1 line's step, split over {N} ranks (its value is the reference point)"}
    if ms_sus:
        extra["sustained"] = {"steps": k_sus, "seconds": ms_sus * 1e-3, "tok_per_s": N * rows * k_sus / (ms_sus * 1e-3)}
        if clocks and clocks.get("sm_mhz"):
            extra["sustained"]["sm_mhz_median_under_load"] = clocks["sm_mhz"]
            extra["sustained"]["mcycles_per_step"] = ms_sus / k_sus * 1e-3 * clocks["sm_mhz"]

    # ---- expert parallel: the ranks' results against a single GPU holding all experts (rank 0), outside the timed regions.
    # Checked on a ONE-layer stack of the same dims, where the only differences are the order in which the k-splits and a
    # row's slots are summed (1e-7 in the gate / up products, which flips a few fp16 roundings of the down operands: 1e-5 to
    # 1e-4 in the output). Over many layers two valid summation orders drift apart (each layer's input differences flip more
    # roundings, then routing decisions of near ties), so the 48-layer difference is reported for information only.
    if N > 1:
        def gathered_logits(m):
            nx_, lg_, _ = m.step_rows(tokens, want_logits=True)
            box = [None] * N
            dist.gather_object(lg_, box if rank == 0 else None, dst=0)
            return np.concatenate(box) if rank == 0 else None

        all_tok = [None] * N
        dist.gather_object(tokens, all_tok if rank == 0 else None, dst=0)
        deep = gathered_logits(model)
        model.free()
        one = eng.fn_model(desc=dict(desc, layers=1), seed=a.seed, max_rows=rows)
        one.set_ep(xchg)
        shallow = gathered_logits(one)
        if rank == 0:
            chk = {"rows": int(rows * N)}
            for name, L, got in (("one_layer", 1, shallow), ("full_depth", a.layers, deep)):
                # the single-GPU model takes each rank's rows as a step of their own, so that the replicated parts (trunk, attention,
                # head) run with the same launch plans as on the ranks and only the MoE block differs
                full = eng.fn_model(desc=dict(STACK, layers=L, expert_first=0, expert_count=0, ep_world=1), seed=a.seed, max_rows=rows)
                parts = [full.step_rows(t_, want_logits=True) for t_ in all_tok]
                fnx, flg = np.concatenate([p_[0] for p_ in parts]), np.concatenate([p_[1] for p_ in parts])
                chk[name] = {"max_rel_err": float(np.abs(got - flg).max() / np.abs(flg).max()), "next_equal": bool(np.array_equal(got.argmax(1), fnx))}
                full.free()
            chk["max_rel_err"], chk["next_equal"] = chk["one_layer"]["max_rel_err"], chk["one_layer"]["next_equal"]
            extra["ep_check"] = chk
        dist.barrier()
        one.free()
    else:
        model.free()
    if xchg is not None:
        xchg.free(barrier=lambda: dist.barrier())
    torch.cuda.empty_cache()
    if N > 1 and a.extras:
        pe = prefill_ep_figure(eng, dev, rank, N, 4096)
        if rank == 0:
            extra["prefill_ep"] = pe

    roof, cpu = None, None
    if N == 1 and rank == 0:
        # ---- roofline of the dominant kernel: the gate/up stream-GEMM launch at this row count, timed alone over 8 layers
        bf = block_figures(eng, rows, 8, a.steps, dev)
        roof = {"bound": "hbm", "kernel": "stream_gemm_kernel<MoeGateUpProblem> (gate/up of routed + shared experts)",
                "achieved": bf["gateup_gbs"], "peak": peak, "unit": "GB/s", "frac": bf["gateup_frac"], "peak_source": which + " (stream copy)",
                "traffic": bf["gateup_bytes"] * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE, "traffic_source": "ncu capture of a one-layer case, scaled by bytes",
                "bytes_per_launch": bf["gateup_bytes"], "us_per_launch": bf["gateup_us"]}
        if clocks and clocks.get("sm_mhz"):
            roof["kcycles_per_launch_at_median_mhz"] = bf["gateup_us"] * clocks["sm_mhz"] * 1e-3
        extra["block"] = {str(rows): bf}
        if a.extras:
            for r in (1, 4, 16):
                if r != rows:
                    extra["block"][str(r)] = block_figures(eng, r, 8, a.steps, dev)
            extra["prefill"] = prefill_figure(eng, 4096, dev)
            q8 = q8head_figure(eng, dev, 1, (248320, 2560), a.seed, 10, 3)  # the reference's 8-bit LM head (not part of the step above)
            q8["frac_of_hbm"] = q8["gbs"] / peak
            extra["q8_lm_head"] = q8
            big = eng.fn_model(desc=dict(STACK, layers=a.layers, ep_world=1, expert_first=0, expert_count=0), seed=a.seed, max_rows=64)
            extra["stack_rows"] = {}
            for r in (4, 64):
                big.step_rows(np.random.default_rng(100).integers(0, STACK["vocab"], r).astype(np.int32))  # distinct rows, as in the headline
                t = big.replay(r, 5) / 5
                extra["stack_rows"][str(r)] = {"ms_per_step": t, "tok_per_s": r / t * 1e3}
            big.free()
            # the opt-in summand product (every weight multiplied as its two fp16 summands, sum unrounded): same figures
            if not a.summand_product:
                eng.lib.ne_exl3_set_summand_product(1)
                try:
                    sbf = block_figures(eng, rows, 8, a.steps, dev)
                    sm = eng.fn_model(desc=dict(STACK, layers=a.layers, ep_world=1, expert_first=0, expert_count=0), seed=a.seed, max_rows=rows)
                    sm.step_rows(tokens)
                    t = sm.replay(rows, 5) / 5
                    sm.free()
                    extra["summand_product"] = {"note": "ne_exl3_set_summand_product(1); off in every other figure of this line",
                                                "rows": rows, "stack_ms_per_step": t, "stack_tok_per_s": rows / t * 1e3,
                                                "block_us": sbf["block_us"], "gateup_us": sbf["gateup_us"], "gateup_frac": sbf["gateup_frac"],
                                                "down_us": sbf["down_us"], "down_frac": sbf["down_frac"]}
                finally:
                    eng.lib.ne_exl3_set_summand_product(0)
        if a.cpu_seconds > 0:
            sec, cores, n = cpu_port_layer_seconds(rows, a.cpu_seconds)
            cpu = {"value": rows / (sec * a.layers), "unit": "tok/s", "cores": cores, "kind": "port",
                   "sample": f"{n} x one decoder layer (4 trunk projections + MoE block on a full 512-expert layer) for {rows} rows in the C port; "
                             f"tok/s = rows / (seconds per layer x {a.layers} layers); LM head and attention stand-in not included"}
            t_np = cpu_numpy_row_seconds()
            extra["cpu_numpy"] = {"seconds_per_block_row": t_np, "tok_per_s": 1.0 / (t_np * a.layers), "threads": os.cpu_count(),
                                  "sample": "one row of one MoE block in the numpy restatement of the reference's tools/opref.py operators "
                                            "(float64 dense reconstruction of the 11 touched experts); tok/s = 1 / (seconds x layers), MoE blocks only"}
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": N, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": stack_config(a, rows),
            "e2e": {"value": N * rows * a.steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": rows * 4, "d2h_bytes_per_step": rows * 4},
            "gpu_launches": info["launches_full"] * a.steps, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu, "extra": extra,
            "wait_status": status}))
    if N > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------- the MoE block alone
def run_block(a, rank, world):
    import torch
    from ijah_b200 import engine as E
    assert world == 1, "--workload block is a single-GPU measurement"
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    eng = E.Engine()
    if a.summand_product:
        eng.lib.ne_exl3_set_summand_product(1)
    peak, which = peaks()
    sampler = ClockSampler(0)
    sampler.start()
    bf = block_figures(eng, a.rows, a.layers, a.steps, dev)
    clocks = sampler.stop()
    extra = {"block": bf}
    if a.prefill_tokens > 0:
        extra["prefill"] = prefill_figure(eng, a.prefill_tokens, dev)
    print(json.dumps({
        "metric": BLOCK_METRIC, "value": a.rows / (bf["block_us"] * 1e-6), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": bf["block_us"] * a.layers * 1e-3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": block_config(a), "e2e": None, "gpu_launches": 6 * a.layers * a.steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "stream_gemm_kernel<MoeGateUpProblem> (gate/up of routed + shared experts)", "achieved": bf["gateup_gbs"],
                     "peak": peak, "unit": "GB/s", "frac": bf["gateup_frac"], "peak_source": which + " (stream copy)",
                     "traffic": bf["gateup_bytes"] * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE, "traffic_source": "ncu capture of a one-layer case, scaled by bytes",
                     "bytes_per_launch": bf["gateup_bytes"], "us_per_launch": bf["gateup_us"]},
        "cpu_baseline": None, "extra": extra, "wait_status": eng.lib.ne_device_wait_status()}))


# ---------------------------------------------------------------------------------------------- the 8-bit affine LM head alone
def q8head_figure(eng, dev, rows, dims, seed, steps, warmup):
    """ne_q8_linear at `dims` = (outputs, inputs), group 64: seeded random bytes / scales generated on the device, CUDA events
    around `steps` launches; returns microseconds per launch, GB/s of algorithmic bytes and a spot check against f64"""
    import torch
    from ijah_b200 import engine as E
    V, H = dims
    G = 64
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    w = torch.randint(0, 256, (V, H), dtype=torch.uint8, device=dev, generator=g)
    sc = (torch.randn((V, H // G), device=dev, generator=g) * 1e-4 + 6e-4).to(torch.bfloat16).view(torch.int16)
    bi = (sc.view(torch.bfloat16).float() * -128).to(torch.bfloat16).view(torch.int16)
    x = torch.randn((rows, H), device=dev, generator=g)
    y = torch.empty((rows, V), device=dev)
    c = E.Q8WeightC(w.data_ptr(), sc.data_ptr(), bi.data_ptr(), H, V, G)
    st = torch.cuda.current_stream().cuda_stream

    def launch():
        eng._ok(eng.lib.ne_q8_linear(ctypes.byref(c), x.data_ptr(), rows, y.data_ptr(), ctypes.c_void_p(st)), "ne_q8_linear")

    for _ in range(warmup):
        launch()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        launch()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / steps
    # spot check against f64 arithmetic on 64 output rows
    idx = torch.arange(0, V, max(V // 64, 1), device=dev)[:64]
    n = len(idx)
    wd = w[idx].float().view(n, H // G, G) * sc.view(torch.bfloat16)[idx].float()[..., None] + bi.view(torch.bfloat16)[idx].float()[..., None]
    want = x.double() @ wd.view(n, H).double().T
    err = float((y[:, idx].double() - want).abs().max() / want.abs().max())
    nbytes = V * H + 4 * V * (H // G) + rows * H * 4 + rows * V * 4
    return {"rows": rows, "outputs": V, "inputs": H, "group": G, "us_per_launch": us, "bytes_per_launch": nbytes, "gbs": nbytes / (us * 1e-6) / 1e9,
            "max_rel_err_vs_f64_on_64_rows": err}


def run_q8head(a, rank, world):
    """--workload q8head: the 8-bit affine Linear at the reference's LM head size (248320 x 2560 bytes, group 64: 636 MB per
    launch, larger than L2) for --rows activation rows"""
    import torch
    from ijah_b200 import engine as E
    assert world == 1, "--workload q8head is a single-GPU measurement"
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    eng = E.Engine()
    if a.summand_product:
        eng.lib.ne_exl3_set_summand_product(1)
    peak, which = peaks()
    V, H = (int(v) for v in a.q8_dims.split("x"))
    sampler = ClockSampler(0)
    sampler.start()
    f = q8head_figure(eng, dev, a.rows, (V, H), a.seed, a.steps, a.warmup)
    clocks = sampler.stop()
    us, gbs = f["us_per_launch"], f["gbs"]
    print(json.dumps({
        "metric": "8-bit affine LM head tok/s", "value": a.rows / (us * 1e-6), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": us * 1e-3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 weights, f16 hi+lo activations, f32 accumulate",
        "data": "synthetic", "config": {"workload": f"ne_q8_linear {V} x {H}, group 64, rows {a.rows}", "l2": "636 MB of weights per launch exceed L2"},
        "e2e": None, "gpu_launches": a.steps * ((a.rows + 7) // 8), "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "q8_stream_kernel", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "peak_source": which + " (stream copy)", "traffic": f["bytes_per_launch"] * 1.01, "traffic_source": "ncu capture of a smaller case, scaled by bytes",
                     "bytes_per_launch": f["bytes_per_launch"], "us_per_launch": us},
        "cpu_baseline": None, "extra": {"max_rel_err_vs_f64_on_64_rows": f["max_rel_err_vs_f64_on_64_rows"]}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=2, help="concurrent sequences per GPU")
    ap.add_argument("--verify", type=int, default=4, help="verify tokens per sequence (rows per GPU = batch x verify)")
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--summand-product", action="store_true",
                    help="run everything under ne_exl3_set_summand_product(1) (opt-in arithmetic: weights as their two fp16 summands)")
    ap.add_argument("--no-extras", dest="extras", action="store_false", help="skip the extra block / prefill / other-row-count figures")
    ap.add_argument("--no-sustain", dest="sustain", action="store_false", help="skip the >= 2 s sustained replay")
    ap.add_argument("--workload", default="stack", choices=["stack", "block", "q8head"])
    ap.add_argument("--q8-dims", default="248320x2560", help="--workload q8head: output rows x inputs (default: the reference's LM head)")
    ap.add_argument("--rows", type=int, default=4, help="--workload block: activation rows")
    ap.add_argument("--prefill-tokens", type=int, default=0, help="--workload block: tokens of a prefill figure (0 = skip)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if a.workload == "block" and "--layers" not in " ".join(sys.argv):
        a.layers = 8
    if a.impl == "reference":
        return run_reference(a, rank)
    if a.workload == "block":
        return run_block(a, rank, world)
    if a.workload == "q8head":
        return run_q8head(a, rank, world)
    return run_stack(a, rank, world)


if __name__ == "__main__":
    main()
