"""Expert-parallel MoE layer: thin host wrapper over the library's b200_ep_* / b200_moe_forward_ep.

Tokens stay data-parallel, the routed experts are sharded over the ranks (global expert e lives on rank
e // experts_per_rank), and the layer runs two collectives on the caller's stream: an all-gather of the
token rows (dispatch) and an f32 reduce-scatter of the per-rank expert sums (combine).  Routing is
replicated: every rank routes the tokens of all ranks with the same deterministic kernel and keeps the
assignments that fall on its own experts, so nothing has to be counted on the host and the step never
synchronises.  The reference has no expert parallelism (it streams experts from SSD on one device,
src/models/expert_stream.zig:400-613); the arithmetic is DSV4MoE.forward
(src/models/deepseek_v4.zig:1010-1056) cut at the two argsorts of DSV4SwitchGLU (:747-784, :809-819).

The communicator is created from a 128-byte NCCL id that rank 0 makes and `torch.distributed` (any
backend) carries to the other ranks; torch is plumbing here, the exchange itself is the library's.

`StepGuard` is the host-side failure detector used between steps: every rank announces the step it is
about to run in the process group's store and waits, with a time limit, for the others; a rank that has
gone is noticed here, on the host, before any collective is queued.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from ._lib import lib


class PeerLost(RuntimeError):
    """A rank did not reach the step within the time limit."""


class StepGuard:
    """Store-based arrival check: call `arrive(step)` on every rank before the step's first launch."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "ep_step"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def arrive(self, step: int) -> None:
        self.store.set(f"{self.prefix}/{step}/{self.rank}", b"1")
        deadline = time.monotonic() + self.timeout_s
        missing = [r for r in range(self.world) if r != self.rank]
        while missing:
            missing = [r for r in missing if not self.store.check([f"{self.prefix}/{step}/{r}"])]
            if not missing:
                return
            if time.monotonic() >= deadline:
                raise PeerLost(f"rank(s) {missing} did not reach step {step} within {self.timeout_s} s")
            time.sleep(0.005)


class Communicator:
    """b200_ep: the NCCL communicator of the expert-parallel group (collective construction)."""

    def __init__(self, rank: int, world: int, group=None):
        ident = torch.zeros(_lib.EP_UNIQUE_ID_BYTES, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_uint8 * _lib.EP_UNIQUE_ID_BYTES)()
            _lib.check(lib.b200_ep_unique_id(buf))
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        if world > 1:
            backend = dist.get_backend(group)
            carrier = ident.cuda() if backend == "nccl" else ident
            dist.broadcast(carrier, src=0, group=group)
            ident = carrier.cpu()
        raw = (C.c_uint8 * _lib.EP_UNIQUE_ID_BYTES)(*ident.tolist())
        h = C.c_void_p()
        _lib.check(lib.b200_ep_create(rank, world, raw, C.byref(h)))
        self._h, self.rank, self.world = h.value, rank, world

    def wait(self, timeout_ms: int = 10000) -> None:
        """Wait for the work queued so far on the current stream; aborts the communicator on timeout."""
        _lib.check(lib.b200_ep_wait(self._h, torch.cuda.current_stream().cuda_stream, timeout_ms))

    def close(self):
        if getattr(self, "_h", None):
            lib.b200_ep_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


class ExpertParallelMoE:
    """One MoE layer with its routed experts sharded over the ranks of `comm`."""

    def __init__(self, comm: Communicator, hidden: int, n_experts: int, inter: int, top_k: int, gate, local_gate_up,
                 local_down, shared_gate_up=None, shared_down=None, bias: Optional[np.ndarray] = None, scoring: int = 0,
                 route_scale: float = 1.0, swiglu_limit: float = 10.0, shared_swiglu_limit: float = 0.0, tile_rows: int = 112,
                 max_tokens: int = 4096):
        assert n_experts % comm.world == 0 and local_gate_up.n_experts == n_experts // comm.world
        self.comm = comm
        self.cfg = _lib.MoeConfig(hidden, n_experts, inter, top_k, scoring, tile_rows, max_tokens, route_scale, swiglu_limit,
                                  shared_swiglu_limit, comm.rank, comm.world)
        self._keep = (gate, local_gate_up, local_down, shared_gate_up, shared_down)
        b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
        h = C.c_void_p()
        _lib.check(lib.b200_moe_create(C.byref(self.cfg), gate._h, b.ctypes.data_as(C.POINTER(C.c_float)) if b is not None else None,
                                       local_gate_up._h, local_down._h, shared_gate_up._h if shared_gate_up else None,
                                       shared_down._h if shared_down else None, C.byref(h)))
        self._h = h.value

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = out if out is not None else torch.empty_like(x)
        _lib.check(lib.b200_moe_forward_ep(self._h, self.comm._h, x.data_ptr(), x.shape[0], out.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream))
        return out

    def close(self):
        if getattr(self, "_h", None):
            lib.b200_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()
