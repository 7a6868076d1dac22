"""Benchmark of the EXL3 MoE decode hot path on B200 (one JSON line on stdout).

Workload (named in `config.workload`): the MoE block of the decoder at decode width -- hidden 2048, 512 experts, top-10,
expert intermediate 768, routed experts K=5, shared expert K=6 -- for `--rows` activation rows, run over `--layers`
layers with distinct random weights (so the weights of one step are far larger than L2). A step is one pass of the rows
through all those layers. value = rows * layers / step time = tokens per second through one MoE block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rows M] [--layers L] [--impl reference]

N > 1 (under torchrun): expert parallel. Every rank holds experts/N experts of every layer and `rows` rows of its own;
rows are all-gathered, each rank runs the routed experts it owns for all rows, partial outputs are reduce-scattered
(NCCL) and the shared expert runs on the rank's own rows. value = N * rows * layers / step time (weak scaling).

--impl reference: the CPU restatement of the reference's operator path (oracle/, C with all host threads) on a bounded
sample of the same workload; the reference's own code for this path is Metal / numpy-with-a-missing-module and cannot
run on this box.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

DIMS = dict(hidden=2048, inter=768, experts=512, k_expert=5, k_shared=6)
TOPK = 10
METRIC = "EXL3 MoE decode tok/s (rows through one MoE block)"
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up stream_gemm launch by rows, from the ncu captures
# summarised under profiles/ (rows without a capture report null)
NCU_TRAFFIC = {4: 79.48e6 + 3.25e6}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region (read-only query)."""

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
        sm, mx, reasons = [], [], set()
        for line in Path(self.path).read_text().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def cpu_port_tokens_per_s(rows, budget_s):
    """The C oracle (device-arithmetic restatement) on the host cores: MoE blocks of `rows` rows on a 64-expert layer
    of the benchmark's dims (the work per row is the same: 10 routed experts + the shared expert), repeated until
    about `budget_s` seconds have passed."""
    from ijah_b200 import packgen
    from oracle import c_oracle as CO
    rng = np.random.default_rng(0)
    t = packgen.moe_layer(rng, hidden=DIMS["hidden"], inter=DIMS["inter"], experts=64, k_expert=DIMS["k_expert"], k_shared=DIMS["k_shared"])
    x = rng.standard_normal((rows, DIMS["hidden"])).astype(np.float16).astype(np.float32)
    CO.moe_block_emul(t, x[:1], top_k=TOPK)
    n, t0 = 0, time.perf_counter()
    while True:
        CO.moe_block_emul(t, x, top_k=TOPK)
        n += 1
        el = time.perf_counter() - t0
        if el > budget_s or n >= 1000:
            break
    return rows * n / el, CO.threads(), f"{n} MoE blocks of {rows} rows on a 64-expert layer of the same dims ({el:.1f} s)"


def run_reference(a, rank):
    if rank != 0:
        return
    per_step = max(2.0, min(20.0, 120.0 / max(a.steps + a.warmup, 1)))
    vals = []
    for i in range(a.warmup + a.steps):
        v, cores, sample = cpu_port_tokens_per_s(a.rows, per_step)
        if i >= a.warmup:
            vals.append(v)
    v = float(np.mean(vals))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tok/s", "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": 1e3 * a.rows / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(a),
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def workload_config(a):
    return {"workload": f"MoE block decode: hidden 2048, 512 experts top-10, inter 768, K5 routed + K6 shared, rows {a.rows}",
            "arithmetic": "weights decoded to f16, f16 activations, f32 accumulate", "rows": a.rows, "layers": a.layers, "l2": "weights of a step exceed L2 (distinct layers cycled)",
            "parallelism": "single GPU" if a.gpus == 1 else f"ep{a.gpus}"}


def run_stack(a, rank, world):
    """--workload stack: one decode step of `--rows` rows through a random-init decoder stack of `--layers` layers (default
    48): per layer the four trunk projections (q 2048->4096, k, v 2048->512, o 4096->2048; K6, every fourth layer K8), a
    stand-in for attention (the o projection takes the q output), the MoE block with residual adds, and at the end the bf16
    LM head (151936 x 2048, a library GEMM). N > 1: experts sharded, everything else replicated, M rows per rank."""
    import torch
    import torch.distributed as dist
    from ijah_b200 import engine as E
    from ijah_b200 import synth
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    eng = E.Engine()
    N, M, L = world, a.rows, a.layers
    H, Ex, V = DIMS["hidden"], DIMS["experts"], 151936
    per = Ex // N
    blocks, trunks, wbytes = [], [], 0
    for l in range(L):
        t = synth.moe_layer(1000 + l, expert_first=rank * per, expert_count=per, router_seed=77 + l, device=dev, **DIMS)
        blocks.append(E.MoeBlock(eng, t, top_k=TOPK, max_rows=M * N, expert_first=rank * per, expert_count=per, device=dev))
        K = 8 if l % 4 == 3 else 6
        tl = synth.trunk_layer(500 + l, K=K, device=dev)
        trunks.append({n: E.Exl3Linear.from_device(eng, *w) for n, w in tl.items()})
        wbytes += sum(w[0].numel() * 2 + w[1].numel() * 2 + w[2].numel() * 2 for w in tl.values())
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    head = (torch.randn((V, H), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    x0 = torch.randn((M, H), device=dev, generator=g).to(torch.float16).to(torch.float32)
    x, q, kk, vv, o, y = (torch.empty((M, n), device=dev) for n in (H, 4096, 512, 512, H, H))
    logits = torch.empty((M, V), device=dev, dtype=torch.bfloat16)
    tok = torch.empty((M,), device=dev, dtype=torch.int64)
    if N > 1:
        from ijah_b200 import ep
        eps = [ep.ExpertParallelMoe(b, dist.group.WORLD) for b in blocks]

    xn = torch.empty_like(x)
    norm = torch.nn.functional.rms_norm

    def step():
        x.copy_(x0)
        for l in range(L):
            tr = trunks[l]
            xn.copy_(norm(x, (H,)))     # the two RMS norms of a layer are stand-ins too (no learned scale)
            E.linear_multi(eng, (tr["q"], tr["k"], tr["v"]), xn, (q, kk, vv))  # one launch chain for the three
            tr["o"].into(q, o)          # attention stand-in: its output has the q width
            x.add_(o)
            xn.copy_(norm(x, (H,)))
            if N == 1:
                blocks[l].forward(xn, out=y)
            else:
                eps[l].forward(xn, out=y)
            x.add_(y)
        torch.matmul(norm(x, (H,)).to(torch.bfloat16), head.t(), out=logits)
        torch.argmax(logits, dim=1, out=tok)

    def barrier():
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        step()
    barrier()
    graph = None
    if N == 1:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        graph.replay()
    run = graph.replay if graph is not None else step
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(a.steps):
        run()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # end to end: the step's input rows from pinned host memory, the sampled token ids back
    xh, th = x0.cpu().pin_memory(), torch.empty((M,), dtype=torch.int64).pin_memory()
    for _ in range(2):
        x0.copy_(xh, non_blocking=True); run(); th.copy_(tok, non_blocking=True); torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        x0.copy_(xh, non_blocking=True); run(); th.copy_(tok, non_blocking=True); torch.cuda.synchronize()
    barrier()
    e2e_s = time.perf_counter() - t0
    if N > 1:
        tt = torch.tensor([ms, e2e_s], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(tt[0].item()), float(tt[1].item())
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / a.steps
    moe_bytes = float(np.mean([b.last_bytes(M * N if N > 1 else M)["total"] for b in blocks])) * L
    total_bytes = moe_bytes + wbytes + V * H * 2
    peak, which = peaks()
    status = eng.lib.ne_device_wait_status()
    if rank == 0:
        per_layer = 6 + 2 * 3  # MoE block, q/k/v chain, o chain
        print(json.dumps({
            "metric": "EXL3 MoE decoder stack decode tok/s", "value": N * M / (ms_per_step * 1e-3), "unit": "tok/s", "n_gpus": N,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"decoder stack decode step: {L} layers (trunk q/k/v/o K6/K8 + MoE block 512 experts top-10 K5 + shared K6), "
                                   f"bf16 LM head 151936 x 2048, rows {M}, attention left as a stand-in",
                       "rows": M, "layers": L, "l2": "weights of a step exceed L2", "graph": graph is not None,
                       "parallelism": "single GPU" if N == 1 else f"ep{N}"},
            "e2e": {"value": N * M * a.steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": M * H * 4, "d2h_bytes_per_step": M * 8},
            "gpu_launches": per_layer * L * a.steps, "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "whole step (all launches)", "achieved": total_bytes / (ms_per_step * 1e-3) / 1e9, "peak": peak,
                         "unit": "GB/s", "frac": total_bytes / (ms_per_step * 1e-3) / 1e9 / peak, "peak_source": which + " (stream copy)",
                         "traffic": None, "bytes_per_step": total_bytes},
            "cpu_baseline": None, "extra": {"weights_gb_resident": (wbytes + V * H * 2 + L * per * 2966016) / 1e9}, "wait_status": status}))
    if N > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rows", type=int, default=4)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--prefill-tokens", type=int, default=4096, help="tokens of the prefill figure in extra (0 = skip)")
    ap.add_argument("--nccl-exchange", action="store_true", help="N > 1: exchange rows and partial outputs with NCCL collectives "
                    "instead of the peer-memory kernels")
    ap.add_argument("--workload", default="block", choices=["block", "stack"],
                    help="block: the MoE block (headline); stack: a whole random-init decoder stack step (see run_stack)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if a.impl == "reference":
        return run_reference(a, rank)
    if a.workload == "stack":
        if "--layers" not in sys.argv:
            a.layers = 48
        return run_stack(a, rank, world)

    import torch
    import torch.distributed as dist
    from ijah_b200 import engine as E
    from ijah_b200 import synth
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE {world}"
    eng = E.Engine()
    N, M, L = world, a.rows, a.layers
    H, Ex = DIMS["hidden"], DIMS["experts"]
    per = Ex // N
    blocks = []
    for l in range(L):
        t = synth.moe_layer(1000 + l, expert_first=rank * per, expert_count=per, router_seed=77 + l, device=dev, **DIMS)
        blocks.append(E.MoeBlock(eng, t, top_k=TOPK, max_rows=M * N, expert_first=rank * per, expert_count=per, device=dev))
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    xs = [torch.randn((M, H), device=dev, generator=g).to(torch.float16).to(torch.float32) for _ in range(L)]
    ys = [torch.empty((M, H), device=dev) for _ in range(L)]
    launches_per_block = 6  # router + plan, operand prep, gate/up, SwiGLU + prep, down, combine

    if N == 1:
        def step():
            for l in range(L):
                blocks[l].forward(xs[l], out=ys[l])
    else:
        from ijah_b200 import ep
        eps = [ep.ExpertParallelMoe(blocks[l], dist.group.WORLD) for l in range(L)]
        launches_per_block = eps[0].launches
        if not a.nccl_exchange:
            # both exchange steps of a block over NVLink peer memory (no library collective in the block): + dispatch and sum kernels
            xchg = ep.ExpertParallelMoe.make_exchange(eng, dist.group.WORLD, M, H, TOPK)
            if xchg is not None:
                launches_per_block += 2
                for e_ in eps:
                    e_.use_exchange(xchg)
            else:
                a.nccl_exchange = True
        exchange = "nccl" if a.nccl_exchange else "nvlink peer memory (own kernels)"

        def step():
            for l in range(L):
                eps[l].forward(xs[l], out=ys[l])

    def barrier():
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        step()
    barrier()
    graph = None
    if N == 1:  # one captured graph per step: launch gaps of the 6-kernel block are what a graph removes
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        graph.replay()
    # N > 1: eager steps. Capturing the step with its two NCCL collectives per block into a CUDA graph did not come back
    # on 2 GPUs (the call ran into its time limit), so the expert-parallel step is not captured.
    run = graph.replay if graph is not None else step
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(a.steps):
        run()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if N > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / a.steps
    value = N * M * L / (ms_per_step * 1e-3)

    # ---- end to end through the host-buffer entry point: pinned x in, y out, every block
    xh = [x.cpu().pin_memory() for x in xs]
    yh = [torch.empty((M, H)).pin_memory() for _ in range(L)]
    if N == 1:
        def e2e_step():
            for l in range(L):
                blocks[l].forward_host(xh[l], out=yh[l])
    else:
        def e2e_step():
            for l in range(L):
                xs[l].copy_(xh[l], non_blocking=True)
                eps[l].forward(xs[l], out=ys[l])
                yh[l].copy_(ys[l], non_blocking=True)
            torch.cuda.synchronize()
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    if N > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": N * M * L * a.steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": M * H * 4 * L, "d2h_bytes_per_step": M * H * 4 * L}
    clocks = sampler.stop() if rank == 0 else None

    # ---- roofline of the dominant kernel: the gate/up stream_gemm launch (routed experts + shared expert), timed alone.
    # The router and the operand prep of every layer run first (untimed), then one graph holding only the L gate/up
    # launches (L distinct weight sets, far larger than L2) is replayed between CUDA events on its stream.
    roof, extra = None, {}
    if N == 1:
        peak, which = peaks()

        def kernel_us(code, before):
            for l in range(L):
                for c in before:
                    blocks[l].stage(c, xs[l], ys[l])
            torch.cuda.synchronize()
            gk = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gk):
                for l in range(L):
                    blocks[l].stage(code, xs[l], ys[l])
            gk.replay()
            torch.cuda.synchronize()
            n = max(3, min(a.steps, 10))
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record()
            for _ in range(n):
                gk.replay()
            k1.record()
            torch.cuda.synchronize()
            return k0.elapsed_time(k1) * 1e3 / n / L

        gu_us = kernel_us(81, (7, 80))
        dn_us = kernel_us(91, (81, 90))
        lbs = [blocks[l].last_bytes(M) for l in range(L)]
        gu_b = float(np.mean([x["gateup"] for x in lbs]))
        dn_b = float(np.mean([x["down"] for x in lbs]))
        tot = float(np.mean([x["total"] for x in lbs]))
        ach = gu_b / gu_us / 1e3
        traffic = NCU_TRAFFIC.get(M)
        roof = {"bound": "hbm", "kernel": "stream_gemm_kernel<MoeGateUpProblem> (gate/up of routed + shared experts)",
                "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_source": which + " (stream copy)",
                "traffic": traffic, "bytes_per_launch": gu_b, "us_per_launch": gu_us}
        extra = {"down_kernel": {"achieved": dn_b / dn_us / 1e3, "us": dn_us, "bytes_per_launch": dn_b},
                 "distinct_experts_mean": float(np.mean([x["distinct_experts"] for x in lbs])),
                 "block": {"bytes": tot, "us": ms_per_step * 1e3 / L, "achieved": tot / (ms_per_step * 1e-3 / L) / 1e9,
                           "frac": tot / (ms_per_step * 1e-3 / L) / 1e9 / peak}}
    # ---- prefill (config 4): one block over 4096 tokens with Zipf(1.1)-skewed routing; N > 1: the same 4096 tokens split
    # over the ranks (strong scaling), all-gather + expert-parallel prefill + reduce-scatter
    n_pf = a.prefill_tokens
    if n_pf > 0:
        last = synth.moe_layer(1000 + L - 1, expert_first=rank * per, expert_count=per, router_seed=77 + L - 1, device=dev, **DIMS)
        synth.zipf_router_bias(last)
        pblk = E.MoeBlock(eng, last, top_k=TOPK, max_rows=16, expert_first=rank * per, expert_count=per, device=dev)
        gp = torch.Generator(device=dev).manual_seed(99 + rank)
        xp = torch.randn((n_pf // N, H), device=dev, generator=gp).to(torch.float16).to(torch.float32)
        xp[:, 0] = 1.0
        yp = torch.empty_like(xp)
        if N == 1:
            def pf_step():
                pblk.prefill(xp, out=yp)
        else:
            pep = ep.ExpertParallelMoe(pblk, dist.group.WORLD)

            def pf_step():
                pep.forward(xp, out=yp, prefill=True)
        for _ in range(3):
            pf_step()
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(5):
            pf_step()
        p1.record()
        barrier()
        pms = p0.elapsed_time(p1) / 5
        if N > 1:
            tt = torch.tensor([pms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            pms = float(tt.item())
        flop = n_pf * TOPK * 3 * 2 * DIMS["hidden"] * DIMS["inter"]
        tpeak = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"] if (ROOT / "MEASURED_PEAKS.json").exists() else 1590.0
        extra["prefill"] = {"tokens": n_pf, "ms": pms, "tok_per_s": n_pf / pms * 1e3, "routed_tflops": flop / pms / 1e9,
                            "frac_of_dense_f16_peak": flop / pms / 1e9 / tpeak / N, "scaling": "strong" if N > 1 else None,
                            "routing": "Zipf(1.1) bias on the router logits"}
    status = eng.lib.ne_device_wait_status()
    if rank == 0:
        cpu = None
        if N == 1:
            v, cores, sample = cpu_port_tokens_per_s(M, a.cpu_seconds)
            cpu = {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": N, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic", "config": dict(workload_config(a), graph=graph is not None, **({"exchange": exchange} if N > 1 else {})),
            "e2e": e2e, "gpu_launches": launches_per_block * L * a.steps, "clocks": clocks, "roofline": roof,
            "cpu_baseline": cpu, "extra": extra, "wait_status": status}))
    if N > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
