"""Expert parallel over NCCL on two GPUs (skipped on a single-GPU box): decode widths and prefill against the single-GPU block."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["IJAH_ROOT"])
from ijah_b200 import engine as E, ep, packgen
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
eng = E.Engine()
rng = np.random.default_rng(5)
t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
per = 32 // world
x_all = rng.standard_normal((world * 40, 512)).astype(np.float16).astype(np.float32)
full = E.MoeBlock(eng, t, top_k=4, max_rows=16, device=dev)
blk = E.MoeBlock(eng, t, top_k=4, max_rows=16 * world, expert_first=rank * per, expert_count=per, device=dev)
par = ep.ExpertParallelMoe(blk, dist.group.WORLD)
# decode widths: 6 rows per rank
xs = torch.from_numpy(x_all[rank * 6:(rank + 1) * 6]).to(dev)
want = full.forward(torch.from_numpy(x_all[:world * 6]).to(dev))[rank * 6:(rank + 1) * 6]
got = par.forward(xs)                      # few rows: routing replicated on every rank
err_d = float((got - want).abs().max() / want.abs().max())
par.own_routing_min_rows = 0               # every row routed on its home rank, routes all-gathered
got2 = par.forward(xs)
err_d = max(err_d, float((got2 - want).abs().max() / want.abs().max()))
# the same block with both exchange steps over NVLink peer memory (two layers share one context; repeated calls)
xchg = ep.ExpertParallelMoe.make_exchange(eng, dist.group.WORLD, 16, 512, 4)
assert xchg is not None, "the peer-memory exchange must come up on a box whose GPUs see each other (else this test would only repeat the NCCL path)"
par.use_exchange(xchg)
for _ in range(3):
    got3 = par.forward(xs)
    err_d = max(err_d, float((got3 - want).abs().max() / want.abs().max()))
par.use_exchange(None)
# prefill: 40 tokens per rank
xp = torch.from_numpy(x_all[rank * 40:(rank + 1) * 40]).to(dev)
wantp = full.prefill(torch.from_numpy(x_all).to(dev))[rank * 40:(rank + 1) * 40]
gotp = par.forward(xp, prefill=True)
err_p = float((gotp - wantp).abs().max() / wantp.abs().max())
# the same as an all-to-all (each pair computed once, by the owner of its expert; unequal token counts per rank): bit-identical
n0 = 40 + 13 * rank
lo = 0 if rank == 0 else 40
xa = torch.from_numpy(x_all[lo:lo + n0]).to(dev)
wanta = full.prefill(torch.from_numpy(x_all[lo:lo + n0]).to(dev))
gota = par.prefill_a2a(xa)
a2a_equal = bool(torch.equal(gota, wanta))
# the whole decoder stack, expert parallel, replayed from the library's CUDA graph: logits of this rank's rows against a
# single-GPU model over the rows of both ranks (synthetic weights do not depend on which slice a rank holds)
d = dict(layers=2, hidden=512, inter=256, experts=32, top_k=4, k_expert=5, k_shared=6, q_out=256, kv_out=128, heads=4, kv_heads=2,
         head_dim=64, k_trunk=6, k_trunk_alt=8, alt_every=2, vocab=1024, kv_positions=64)
xm = ep.ExpertParallelMoe.make_exchange(eng, dist.group.WORLD, 3, 512, 4)
assert xm is not None
mp = eng.fn_model(desc=dict(d, expert_first=rank * per, expert_count=per, ep_world=world), seed=3, max_rows=3)
mp.set_ep(xm)
mf = eng.fn_model(desc=dict(d, expert_first=0, expert_count=0, ep_world=1), seed=3, max_rows=3 * world)
toks = (np.arange(3 * world, dtype=np.int32) * 37 + 11) % 1024
_, lf, _ = mf.step_rows(toks, want_logits=True)
err_m = 0.0
for _ in range(3):  # the first call captures the step, the others replay it
    nx, lp, _ = mp.step_rows(toks[rank * 3:(rank + 1) * 3], want_logits=True)
    err_m = max(err_m, float(np.abs(lp - lf[rank * 3:(rank + 1) * 3]).max() / np.abs(lf).max()))
assert np.array_equal(nx, lf[rank * 3:(rank + 1) * 3].argmax(1))
torch.cuda.synchronize()
status = eng.lib.ne_device_wait_status()
dist.barrier()
mp.free(); mf.free()
xm.free(barrier=dist.barrier); xchg.free(barrier=dist.barrier)
dist.destroy_process_group()
assert err_d < 1e-5 and err_p < 1e-5 and err_m < 1e-4 and status == 0 and a2a_equal, (err_d, err_p, err_m, status, a2a_equal)
print("EP_OK", rank, err_d, err_p, err_m)
"""


def test_expert_parallel_matches_single_gpu_on_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, IJAH_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", str(port), str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count("EP_OK") == 2
