"""Host logic of the expert-parallel wrapper (ijah_b200/ep.py) on CPU: 2 gloo ranks, each with half the experts; the
block is an oracle-backed stand-in with the interface of engine.MoeBlock.forward_ep. The combined output must equal the
single-rank oracle block."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ijah_b200 import packgen
from oracle import c_oracle as CO

DIMS = dict(hidden=256, inter=128, experts=16)
TOPK = 4
ROWS = 3


def _tensors():
    return packgen.moe_layer(np.random.default_rng(123), **DIMS)


def _x(rank):
    return np.random.default_rng(50 + rank).standard_normal((ROWS, DIMS["hidden"])).astype(np.float16).astype(np.float32)


class OracleBlock:
    def __init__(self, tensors, e0, e1):
        self.t, self.e0, self.e1, self.H, self.k, self.E = tensors, e0, e1, DIMS["hidden"], TOPK, DIMS["experts"]

    # the pieces of the all-to-all prefill, with the interface of engine.MoeBlock
    def prefill_home(self, x):
        r = CO.moe_block_emul(self.t, x.numpy(), top_k=TOPK, expert_range=(0, 0))  # no routed expert: the shared term alone
        route = np.concatenate([r["ids"].astype(np.int32), r["weights"].astype(np.float32).view(np.int32)], 1)
        return torch.from_numpy(r["out"]), torch.from_numpy(route)

    def prefill_routed(self, x_pairs, route_pairs):
        n = x_pairs.shape[0]
        if n == 0:
            return torch.empty((0, self.H))
        ids = route_pairs[:, :1].contiguous().numpy().astype(np.int64)
        assert ((ids >= self.e0) & (ids < self.e1)).all(), "a pair reached a rank that does not own its expert"
        w = route_pairs[:, 1:].contiguous().numpy().view(np.float32)
        r = CO.moe_block_emul(self.t, x_pairs.contiguous().numpy(), top_k=1, ids=ids, weights=w, shared_rows=(0, 0))
        return torch.from_numpy(r["out"])

    def pairs_by_owner(self, route, world):
        ids = route[:, :TOPK].reshape(-1)
        dest = torch.div(ids, self.E // world, rounding_mode="floor")
        perm = torch.argsort(dest, stable=True)
        pos = torch.empty(ids.numel(), dtype=torch.int32)
        pos[perm] = torch.arange(ids.numel(), dtype=torch.int32)
        send_r = torch.stack((ids[perm], route[:, TOPK:].reshape(-1)[perm]), 1).contiguous()
        return (perm // TOPK).to(torch.int32), send_r, pos.view(-1, TOPK), torch.bincount(dest, minlength=world).to(torch.int64)

    def gather_rows(self, src, index):
        return src[index.long()].contiguous()

    def combine_slots(self, slots, pos, base, out=None):
        y = torch.zeros_like(base)
        for s_ in range(pos.shape[1]):  # slot order, the shared term last
            y = y + slots[pos[:, s_].long()]
        return y + base

    def forward_ep(self, x_all, own_row0, own_rows, out=None):
        r = CO.moe_block_emul(self.t, x_all.numpy(), top_k=TOPK, expert_range=(self.e0, self.e1), shared_rows=(own_row0, own_rows))
        out.copy_(torch.from_numpy(r["out"]))
        return out

    # home-rank routing: routes as int32 [rows, 2 top_k] (ids, then the float weights' bits), as engine.MoeBlock has them
    def route_rows(self, x, route_out):  # route_out: a column slice of the packed rows
        r = CO.moe_block_emul(self.t, x.numpy(), top_k=TOPK)
        route_out[:, :TOPK] = torch.from_numpy(r["ids"].astype(np.int32))
        route_out[:, TOPK:] = torch.from_numpy(r["weights"].astype(np.float32).view(np.int32))
        return route_out

    def forward_ep_routed(self, x_all, route_all, own_row0, own_rows, out=None):
        ids = route_all[:, :TOPK].contiguous().numpy().astype(np.int64)
        w = route_all[:, TOPK:].contiguous().numpy().view(np.float32)
        r = CO.moe_block_emul(self.t, x_all.contiguous().numpy(), top_k=TOPK, ids=ids, weights=w, expert_range=(self.e0, self.e1),
                              shared_rows=(own_row0, own_rows))
        out.copy_(torch.from_numpy(r["out"]))
        return out


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ijah_b200 import ep
        per = DIMS["experts"] // world
        m = ep.ExpertParallelMoe(OracleBlock(_tensors(), rank * per, (rank + 1) * per))
        y = m.forward(torch.from_numpy(_x(rank)))
        y2 = m.forward(torch.from_numpy(_x(rank)))  # buffers are reused on the second call
        assert torch.equal(y, y2)
        assert m.own_routing
        m.own_routing_min_rows = 0                  # every row routed on its home rank, routes all-gathered beside the rows
        y3 = m.forward(torch.from_numpy(_x(rank)))
        assert float((y3 - y).abs().max() / y.abs().max()) < 1e-6
        # the all-to-all prefill: a different token count per rank, every pair computed by the rank owning its expert
        xa = np.random.default_rng(70 + rank).standard_normal((5 + 4 * rank, DIMS["hidden"])).astype(np.float16).astype(np.float32)
        ya = m.prefill_a2a(torch.from_numpy(xa))
        q.put((rank, (y.numpy(), xa, ya.numpy())))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_block():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    t = _tensors()
    for rank in range(2):
        y, xa, ya = got[rank]
        want = CO.moe_block_emul(t, _x(rank), top_k=TOPK)["out"]
        assert np.abs(y - want).max() / np.abs(want).max() < 1e-5
        want = CO.moe_block_emul(t, xa, top_k=TOPK)["out"]
        assert np.abs(ya - want).max() / np.abs(want).max() < 1e-5
