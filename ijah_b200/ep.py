"""Expert-parallel MoE block over torch.distributed (one process per GPU; NCCL on GPUs, gloo in the CPU tests).

The reference is single-device; expert parallelism is this library's addition. Rank g holds experts
[g * E/N, (g+1) * E/N) of the layer (a MoeBlock created with expert_first / expert_count) and `rows` rows of its own.

    route      block.route_rows(x)                                     -> routes of the rank's own rows (decode widths)
    dispatch   all_gather of the ranks' rows (with their routes       -> x_all [N * rows, H] on every rank
               packed beside them: one collective)
    compute    block.forward_ep_routed(x_all, route_all, row0, rows)  -> this rank's summand y_part [N * rows, H]:
               the routed slots whose expert this rank owns (each distinct expert streamed once for all rows that
               use it, slots summed per row in slot order) and the shared expert for the rank's own rows.
               (Blocks without route_rows, and the prefill path, route all rows on every rank: forward_ep / prefill_ep.)
    combine    reduce_scatter (sum) of y_part                          -> y [rows, H] of the rank's own rows

The many-token prefill has a second form, prefill_a2a: a true all-to-all. Each token is routed on its home rank, every
(token, slot) pair is sent to the one rank that owns its expert (all_to_all_single with the pair counts exchanged first),
the owner runs its pairs through the grouped tensor-core GEMM, the per-pair outputs return by the mirrored all-to-all and
the home rank adds a token's slots in slot order and the shared expert last: bit-identical to the single-GPU prefill.

At decode widths the payload is tiny (rows * H * 4 bytes per rank each way), so both collectives are latency-bound and
the win is the N-fold drop in weight bytes per GPU. The sum over ranks changes the order in which a row's slots are
added (per-rank partial sums in slot order, then ranks in the collective's order); the result stays within the 2e-3
output bound and is noted as a deviation from the single-GPU slot order.

With use_exchange(make_exchange(...)) both exchange steps run over NVLink peer memory instead (ijah_b200/csrc/
ep_exchange.cuh): packed rows are written straight into every peer's gather area, the combine kernel stores each finished
row into the owning rank's memory, flags signal arrival; no library collective remains in the block.

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
        self._pack = self._pack_all = self._views = None
        self.xchg = None
        # blocks that can route alone (engine.MoeBlock) route each row on its home rank; others replicate the routing
        self.own_routing = hasattr(block, "route_rows") and hasattr(block, "forward_ep_routed")
        # ... once the gathered rows exceed this count (the replicated router takes 11 / 14 / 23 / 42 us at 4 / 8 / 16 / 32 rows,
        # home-rank routing 11 us plus a small copy)
        self.own_routing_min_rows = 8

    @staticmethod
    def make_exchange(eng, group, rows_cap, hidden, top_k):
        """an NVLink peer-memory exchange context shared by all layers (engine.EpExchange), connected across `group`;
        attach it to wrappers with use_exchange(). Returns None on every rank if any rank could not set it up (the
        wrappers then keep the NCCL exchange)."""
        from . import engine as E
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        x, err = None, None
        try:
            x = E.EpExchange(eng, rank, world, rows_cap, hidden, top_k)
            mine = x.handle()
        except Exception as ex:  # keep taking part in the collectives below so that no rank is left waiting
            mine, err = b"\0" * 64, ex
        handles = [None] * world
        dist.all_gather_object(handles, mine, group=group)
        if err is None:
            try:
                x.connect(handles)
            except Exception as ex:
                err = ex
        oks = [None] * world
        dist.all_gather_object(oks, err is None, group=group)
        if not all(oks):  # one rank could not set up peer access: every rank falls back (returns None)
            if x is None:
                dist.barrier(group)  # the barrier the ranks that do hold a context run between disconnect and free
            if x is not None:
                x.free(barrier=lambda: dist.barrier(group))
            if err is not None:
                import sys
                print(f"[rank {rank}] peer-memory exchange unavailable: {err}", file=sys.stderr)
            return None
        return x

    def use_exchange(self, xchg):
        """decode-width forwards go through block.forward_ep_fused: no library collective in the block"""
        self.xchg = xchg
        return self

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
        x = x.contiguous()
        if not prefill and self.xchg is not None:
            y = torch.empty_like(x) if out is None else out
            return self.block.forward_ep_fused(self.xchg, x, out=y)
        x_all, y_part = self._buffers(x)
        if not prefill and self.own_routing and rows * self.world > self.own_routing_min_rows:
            # every row is routed on its home rank only; a row and its route travel side by side in ONE all-gather:
            # packed row = [x (H floats) | ids (k) | weights (k)], the kernels read both parts with the packed row stride
            k2, W = 2 * self.block.k, H + 2 * self.block.k
            if self._pack is None or self._pack.shape != (rows, W) or self._pack.device != x.device:
                self._pack = torch.empty((rows, W), dtype=torch.float32, device=x.device)
                self._pack_all = torch.empty((rows * self.world, W), dtype=torch.float32, device=x.device)
                self._views = (self._pack[:, :H], self._pack[:, H:].view(torch.int32),
                               self._pack_all[:, :H], self._pack_all[:, H:].view(torch.int32))
            own_x, own_r, all_x, all_r = self._views
            own_x.copy_(x)
            self.block.route_rows(x, own_r)
            dist.all_gather_into_tensor(self._pack_all, self._pack, group=self.group)
            self.block.forward_ep_routed(all_x, all_r, self.rank * rows, rows, out=y_part)
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

    def prefill_a2a(self, x, out=None, mark=None):
        """x [n, H] float32, the rank's own tokens (any count per rank, zero excluded) -> y [n, H]. The block needs
        prefill_home, pairs_by_owner, gather_rows, prefill_routed, combine_slots and k (engine.MoeBlock has them).
        mark(name), if given, is called after each stage (a timing hook: bench.py synchronises in it)."""
        b, N, k = self.block, self.world, self.block.k
        mark = mark or (lambda name: None)
        n, H = x.shape
        x = x.contiguous()
        y_sh, route = b.prefill_home(x)                      # routing + shared expert of the own tokens
        mark("home")
        tok, send_r, pos, counts = b.pairs_by_owner(route, N)  # pairs grouped by owner, (token, slot) order inside a group
        send_x = b.gather_rows(x, tok)
        mark("pack")
        got = torch.empty_like(counts)
        dist.all_to_all_single(got, counts, group=self.group)
        send_n, recv_n = counts.tolist(), got.tolist()       # the one host synchronisation of the call
        mark("counts")
        recv_x = torch.empty((sum(recv_n), H), dtype=torch.float32, device=x.device)
        recv_r = torch.empty((sum(recv_n), 2), dtype=torch.int32, device=x.device)
        dist.all_to_all_single(recv_x, send_x, recv_n, send_n, group=self.group)
        dist.all_to_all_single(recv_r, send_r, recv_n, send_n, group=self.group)
        mark("dispatch")
        y_pairs = b.prefill_routed(recv_x, recv_r)           # this rank's experts on everybody's pairs
        mark("owner")
        back = torch.empty((n * k, H), dtype=torch.float32, device=x.device)
        dist.all_to_all_single(back, y_pairs, send_n, recv_n, group=self.group)
        mark("return")
        y = b.combine_slots(back, pos, y_sh, out=out)        # slots in slot order, the shared term last
        mark("combine")
        self.last_pairs_received = sum(recv_n)
        return y
