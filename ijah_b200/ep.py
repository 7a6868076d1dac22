"""Expert-parallel MoE block over torch.distributed (one process per GPU; NCCL on GPUs, gloo in the CPU tests).

The reference is single-device; this is the sharding BASELINE's north star asks for. Rank g holds experts
[g * E/N, (g+1) * E/N) of the layer (a MoeBlock created with expert_first / expert_count) and `rows` rows of its own.

    route      block.route_rows(x)                                     -> routes of the rank's own rows (decode widths)
    dispatch   all_gather of the ranks' rows (and routes)             -> x_all [N * rows, H] on every rank
    compute    block.forward_ep_routed(x_all, route_all, row0, rows)  -> this rank's summand y_part [N * rows, H]:
               the routed slots whose expert this rank owns (each distinct expert streamed once for all rows that
               use it, slots summed per row in slot order) and the shared expert for the rank's own rows.
               (Blocks without route_rows, and the prefill path, route all rows on every rank: forward_ep / prefill_ep.)
    combine    reduce_scatter (sum) of y_part                          -> y [rows, H] of the rank's own rows

At decode widths the payload is tiny (rows * H * 4 bytes per rank each way), so both collectives are latency-bound and
the win is the N-fold drop in weight bytes per GPU. The sum over ranks changes the order in which a row's slots are
added (per-rank partial sums in slot order, then ranks in the collective's order); the result stays within the 2e-3
output bound and is noted as a deviation from the single-GPU slot order.

`block` only needs `forward_ep(x_all, own_row0, own_rows, out=None)` and `H`; the CPU tests pass an oracle-backed
stand-in, the GPU path passes ijah_b200.engine.MoeBlock.
"""
import torch
import torch.distributed as dist


class ExpertParallelMoe:
    # kernels of this library per forward (router, prep, gate/up, mid, down, combine); the two collectives are NCCL's
    launches = 6

    def __init__(self, block, group=None):
        self.block = block
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.backend = dist.get_backend(group)
        self._x_all = None
        self._y_part = None
        self._route = self._route_all = None
        # blocks that can route alone (engine.MoeBlock) route each row on its home rank; others replicate the routing
        self.own_routing = hasattr(block, "route_rows") and hasattr(block, "forward_ep_routed")
        # ... once the gathered rows exceed this count: below it the replicated router costs less than a second all-gather plus
        # a separate router launch (measured on 2 GPUs: +24 us per block; the replicated router takes 11 / 23 / 42 us at 4 / 16 / 32 rows)
        self.own_routing_min_rows = 32

    def _buffers(self, x):
        rows, H = x.shape
        if self._x_all is None or self._x_all.shape[0] != rows * self.world or self._x_all.device != x.device:
            self._x_all = torch.empty((rows * self.world, H), dtype=torch.float32, device=x.device)
            self._y_part = torch.empty((rows * self.world, H), dtype=torch.float32, device=x.device)
        return self._x_all, self._y_part

    def forward(self, x, out=None, prefill=False):
        """x [rows, H] float32 (every rank the same row count) -> y [rows, H]; prefill: the many-token path
        (block.prefill_ep: sorted slots, grouped tensor-core GEMM) instead of the decode-width kernels"""
        rows, H = x.shape
        x_all, y_part = self._buffers(x)
        x = x.contiguous()
        if not prefill and self.own_routing and rows * self.world > self.own_routing_min_rows:
            # every row is routed on its home rank only; rows and routes travel together (two small all-gathers)
            k2 = 2 * self.block.k
            if self._route is None or self._route.shape[0] != rows or self._route.device != x.device:
                self._route = torch.empty((rows, k2), dtype=torch.int32, device=x.device)
                self._route_all = torch.empty((rows * self.world, k2), dtype=torch.int32, device=x.device)
            self.block.route_rows(x, self._route)
            dist.all_gather_into_tensor(x_all, x, group=self.group)
            dist.all_gather_into_tensor(self._route_all, self._route, group=self.group)
            self.block.forward_ep_routed(x_all, self._route_all, self.rank * rows, rows, out=y_part)
        else:
            dist.all_gather_into_tensor(x_all, x, group=self.group)
            (self.block.prefill_ep if prefill else self.block.forward_ep)(x_all, self.rank * rows, rows, out=y_part)
        y = torch.empty_like(x) if out is None else out
        if self.backend == "gloo":  # gloo has no reduce_scatter: all_reduce and keep the own slice
            dist.all_reduce(y_part, group=self.group)
            y.copy_(y_part[self.rank * rows:(self.rank + 1) * rows])
        else:
            dist.reduce_scatter_tensor(y, y_part, group=self.group)
        return y
