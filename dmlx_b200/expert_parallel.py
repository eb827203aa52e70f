"""Expert-parallel MoE layer: tokens stay data-parallel, routed experts are sharded across ranks,
one all-to-all each way (dispatch, combine) over torch.distributed.

The reference has no expert parallelism (it streams experts from SSD on one device,
src/models/expert_stream.zig:400-613); the layer arithmetic is DSV4MoE.forward
(src/models/deepseek_v4.zig:1010-1056) with DSV4SwitchGLU split at the exchange points
(:747-819): sort assignments by expert -> [dispatch] -> grouped gate/up + clipped SwiGLU x score
-> grouped down -> [combine] -> unsort and sum over k.

Layout facts
  * global expert e lives on rank e // experts_per_rank.
  * A rank sorts its N*k assignments by global expert (stable), so its send buffer is already
    ordered by destination rank and, inside a destination, by local expert.
  * Counts travel first as an [W, experts_per_rank] matrix; split sizes for the row exchange are
    its row sums (host integers, as the all-to-all needs them).
  * Received rows are source-major; `regroup_index` gives the gather that makes them expert-major
    (the order the grouped matmul wants) and its inverse puts results back for the return trip.

The planning functions work on CPU tensors (tested with gloo); `ExpertParallelMoE.forward` runs
the kernels of libdmlx_b200 on the GPU around the two collectives.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def send_splits(counts_by_expert: torch.Tensor, world: int) -> List[int]:
    """Rows this rank sends to each rank: sums of its per-expert counts over that rank's experts."""
    e = counts_by_expert.numel()
    assert e % world == 0, "experts must divide evenly over ranks"
    return counts_by_expert.view(world, e // world).sum(1).tolist()


def exchange_counts(counts_by_expert: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """all-to-all of the count matrix: returns recv_counts [W, E_local] — rows source s will send
    to each of this rank's local experts."""
    e = counts_by_expert.numel()
    send = counts_by_expert.view(world, e // world).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def regroup_index(recv_counts: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """recv_counts [W, E_local] (host or device integers) -> (gather index that turns the
    source-major receive buffer into expert-major order, expert offsets [E_local + 1])."""
    rc = recv_counts.to("cpu", torch.int64)
    w, el = rc.shape
    # start of segment (s, e) in the receive buffer: sources in order, experts in order inside
    seg_start = torch.zeros(w * el + 1, dtype=torch.int64)
    seg_start[1:] = rc.reshape(-1).cumsum(0)
    seg_start = seg_start[:-1].view(w, el)
    idx = []
    for e in range(el):
        for s in range(w):
            n = int(rc[s, e])
            if n:
                idx.append(torch.arange(int(seg_start[s, e]), int(seg_start[s, e]) + n))
    index = torch.cat(idx) if idx else torch.zeros(0, dtype=torch.int64)
    offsets = torch.zeros(el + 1, dtype=torch.int64)
    offsets[1:] = rc.sum(0).cumsum(0)
    return index.to(torch.int32), offsets.to(torch.int32)


def work_items(offsets: torch.Tensor, tile_rows: int) -> torch.Tensor:
    """{expert, first row, rows, 0} per token tile of every local expert (host integers)."""
    items = []
    off = offsets.tolist()
    for e in range(len(off) - 1):
        for r0 in range(off[e], off[e + 1], tile_rows):
            items.append((e, r0, min(tile_rows, off[e + 1] - r0), 0))
    return torch.tensor(items if items else [(0, 0, 0, 0)], dtype=torch.int32).view(-1, 4)


def all_to_all_rows(rows: torch.Tensor, send: List[int], recv: List[int], group=None) -> torch.Tensor:
    out = torch.empty((sum(recv),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
    return out


class ExpertParallelMoE:
    """One MoE layer with its routed experts sharded over the ranks of `group`."""

    def __init__(self, hidden: int, n_experts: int, inter: int, top_k: int, gate, local_gate_up, local_down,
                 shared_gate_up=None, shared_down=None, bias: Optional[torch.Tensor] = None, route_scale: float = 1.0,
                 swiglu_limit: float = 10.0, tile_rows: int = 128, group=None):
        self.hidden, self.n_experts, self.inter, self.k = hidden, n_experts, inter, top_k
        self.gate, self.gu, self.down, self.sgu, self.sdown = gate, local_gate_up, local_down, shared_gate_up, shared_down
        self.bias, self.route_scale, self.limit, self.tile = bias, route_scale, swiglu_limit, tile_rows
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        assert n_experts % self.world == 0 and local_gate_up.n_experts == n_experts // self.world

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """One host synchronisation per layer (the split sizes the all-to-all needs as integers);
        everything else, including the regrouping of received rows by local expert, runs on the
        device: rows travel with their local expert id and routing weight, and the receiver sorts
        them with the same stable counting sort the single-GPU layer uses."""
        from . import device as dev

        n, k, w = x.shape[0], self.k, self.world

        def shared_expert():
            return dev.qmm(self.sdown, dev.qmm(self.sgu, x, dev.EPI_SWIGLU)) if self.sgu is not None else None

        logits = dev.qmm(self.gate, x)
        idx, wts, counts = dev.moe_route(logits, k, self.bias, dev.SCORE_SOFTMAX, self.route_scale)
        _, order, inv, items, n_items = dev.moe_group(idx, counts, self.tile)
        x_sorted, scales = dev.moe_gather(x, order, wts, k)
        if w == 1:
            act = dev.moe_grouped_qmm(self.gu, x_sorted, items, n_items, self.tile, dev.EPI_SWIGLU, scales, self.limit)
            y_sorted = dev.moe_grouped_qmm(self.down, act, items, n_items, self.tile)
            return dev.moe_combine(y_sorted, inv, n, k, shared_expert())
        el = self.n_experts // w
        recv_counts = exchange_counts(counts, w, self.group)  # [W, E_local] on the device
        splits = torch.stack([counts.view(w, el).sum(1), recv_counts.sum(1)]).to("cpu")  # the layer's one sync
        send, recv = splits[0].tolist(), splits[1].tolist()
        # per sorted row: (local expert id, routing weight bits)
        eid = torch.remainder(idx.view(-1)[order.long()], el).to(torch.int32)
        meta = torch.stack([eid, scales.view(torch.int32)], 1).contiguous()
        rows = torch.empty((sum(recv), x.shape[1]), dtype=x_sorted.dtype, device=x.device)
        rmeta = torch.empty((sum(recv), 2), dtype=torch.int32, device=x.device)
        pending = [dist.all_to_all_single(rows, x_sorted, recv, send, group=self.group, async_op=True),
                   dist.all_to_all_single(rmeta, meta, recv, send, group=self.group, async_op=True)]
        shared = shared_expert()  # runs while the rows travel
        for work in pending:
            work.wait()
        m = rows.shape[0]
        if m > 0:
            ids = rmeta[:, 0].contiguous().view(m, 1)
            lcounts = recv_counts.sum(0).to(torch.int32)
            _, lorder, linv, litems, ln_items = dev.moe_group(ids, lcounts, self.tile)
            xe = dev.gather_rows(rows, lorder)
            se = rmeta[:, 1].contiguous().view(torch.float32)[lorder.long()].contiguous()
            act = dev.moe_grouped_qmm(self.gu, xe, litems, ln_items, self.tile, dev.EPI_SWIGLU, se, self.limit)
            ye = dev.moe_grouped_qmm(self.down, act, litems, ln_items, self.tile)
            y_recv_order = dev.gather_rows(ye, linv)
        else:
            y_recv_order = torch.empty((0, self.hidden), dtype=torch.bfloat16, device=x.device)
        y_sorted = all_to_all_rows(y_recv_order, recv, send, self.group)
        return dev.moe_combine(y_sorted, inv, n, k, shared)
