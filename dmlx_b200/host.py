"""Host-side mirror of the reference's scheduler / batch builder / block manager API.

Thin wrappers over the C++ host layer in libdmlx_b200 (same names and argument meaning as
src/scheduler.zig, src/batch_builder.zig and paged.BlockManager in src/kvcache/paged.zig), so the
reference's own tests can be restated against it.  All state lives in the C++ objects; Python
holds handles only.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import B200Error, InsufficientBlocks, InvalidBatchIndex, InvalidBlockId, lib

WAITING, PREFILLING, DECODING, DONE = 0, 1, 2, 3
PAGE_SIZE = 32


def _u32(xs) -> Tuple[C.Array, int]:
    arr = (C.c_uint32 * max(len(xs), 1))(*[int(x) & 0xFFFFFFFF for x in xs])
    return arr, len(xs)


def hash_block(prev_hash: int, token_ids: Sequence[int]) -> int:
    arr, n = _u32(token_ids)
    return int(lib.b200_hash_block(int(prev_hash) & 0xFFFFFFFFFFFFFFFF, arr, n))


class Prng:
    """std.Random.DefaultPrng as SamplerConfig.init(seed) creates it (src/sampling.zig:287-296)."""

    def __init__(self, seed: int):
        self._s = (C.c_uint64 * 4)()
        lib.b200_prng_seed(int(seed) & 0xFFFFFFFFFFFFFFFF, self._s)

    def set_state(self, words: Sequence[int]):
        for i in range(4):
            self._s[i] = int(words[i])

    def next_u64(self) -> int:
        return int(lib.b200_prng_next_u64(self._s))

    def next_f32(self) -> float:
        return float(lib.b200_prng_next_f32(self._s))


class PagedBlockManager:
    """paged.BlockManager (src/kvcache/paged.zig:44-273)."""

    def __init__(self, total_blocks: int):
        self._h = lib.b200_bm_create(total_blocks)
        self.total_blocks = total_blocks

    def __del__(self):
        if getattr(self, "_h", None):
            lib.b200_bm_destroy(self._h)
            self._h = None

    def can_allocate(self, n: int) -> bool:
        return bool(lib.b200_bm_can_allocate(self._h, n))

    def allocate_blocks(self, req_id: int, n: int) -> List[int]:
        out = (C.c_uint64 * max(n, 1))()
        _lib.check(lib.b200_bm_allocate_blocks(self._h, req_id, n, out))
        return [int(out[i]) for i in range(n)]

    def free_blocks_of(self, req_id: int) -> None:
        lib.b200_bm_free_blocks(self._h, req_id)

    def copy_on_write(self, block_id: int) -> int:
        out = C.c_uint64()
        _lib.check(lib.b200_bm_copy_on_write(self._h, block_id, C.byref(out)))
        return int(out.value)

    def free_count(self) -> int:
        return int(lib.b200_bm_free_count(self._h))

    def used_count(self) -> int:
        return int(lib.b200_bm_used_count(self._h))

    def find_cached_prefix(self, token_ids: Sequence[int], block_size: int) -> List[int]:
        arr, n = _u32(token_ids)
        cap = n // block_size + 1 if block_size else 1
        out = (C.c_uint64 * cap)()
        cnt = C.c_uint64()
        _lib.check(lib.b200_bm_find_cached_prefix(self._h, arr, n, block_size, out, cap, C.byref(cnt)))
        return [int(out[i]) for i in range(cnt.value)]

    def register_block_hash(self, block_id: int, h: int) -> None:
        _lib.check(lib.b200_bm_register_block_hash(self._h, block_id, h))

    def get_ref(self, bid: int) -> int:
        return int(lib.b200_bm_get_ref(self._h, bid))

    def set_ref(self, bid: int, n: int) -> None:
        lib.b200_bm_set_ref(self._h, bid, n)

    def is_used(self, bid: int) -> bool:
        return bool(lib.b200_bm_is_used(self._h, bid))

    def get_tokens_used(self, bid: int) -> int:
        return int(lib.b200_bm_get_tokens_used(self._h, bid))

    def set_tokens_used(self, bid: int, n: int) -> None:
        lib.b200_bm_set_tokens_used(self._h, bid, n)

    def share(self, req_id: int, bid: int) -> None:
        lib.b200_bm_share(self._h, req_id, bid)

    def blocks_of(self, req_id: int) -> List[int]:
        n = int(lib.b200_bm_blocks_of(self._h, req_id, None, 0))
        out = (C.c_uint64 * max(n, 1))()
        lib.b200_bm_blocks_of(self._h, req_id, out, n)
        return [int(out[i]) for i in range(n)]


class Request:
    """scheduler.Request (src/scheduler.zig:108-187)."""

    def __init__(self, id: int, prompt_tokens: Sequence[int], max_tokens: int, stop_tokens: Sequence[int] = ()):
        p, n = _u32(prompt_tokens)
        s, ns = _u32(stop_tokens)
        self._h = lib.b200_request_create(id, p, n, max_tokens, s, ns)
        self.id = id
        self.max_tokens = max_tokens
        self.stop_tokens = list(stop_tokens)

    def __del__(self):
        if getattr(self, "_h", None):
            lib.b200_request_destroy(self._h)
            self._h = None

    @property
    def state(self) -> int:
        return int(lib.b200_request_state(self._h))

    @property
    def prefill_offset(self) -> int:
        return int(lib.b200_request_prefill_offset(self._h))

    @property
    def generated_tokens(self) -> List[int]:
        n = int(lib.b200_request_generated(self._h, None, 0))
        out = (C.c_uint32 * max(n, 1))()
        lib.b200_request_generated(self._h, out, n)
        return [int(out[i]) for i in range(n)]

    @property
    def block_ids(self) -> List[int]:
        n = int(lib.b200_request_block_ids(self._h, None, 0))
        out = (C.c_uint64 * max(n, 1))()
        lib.b200_request_block_ids(self._h, out, n)
        return [int(out[i]) for i in range(n)]

    @property
    def kv_slot(self) -> int:
        return int(lib.b200_request_kv_slot(self._h))

    @property
    def error(self) -> int:
        return int(lib.b200_request_error(self._h))

    @property
    def prompt_tokens(self) -> List[int]:
        n = int(lib.b200_request_prompt(self._h, None, 0))
        out = (C.c_uint32 * max(n, 1))()
        lib.b200_request_prompt(self._h, out, n)
        return [int(out[i]) for i in range(n)]

    def seq_len(self) -> int:
        return int(lib.b200_request_seq_len(self._h))

    def is_stop_token(self, t: int) -> bool:
        return bool(lib.b200_request_is_stop_token(self._h, t))

    def has_pending_prefill(self) -> bool:
        return bool(lib.b200_request_has_pending_prefill(self._h))

    def current_prefill_chunk_len(self, max_prefill_tokens: int) -> int:
        return int(lib.b200_request_current_prefill_chunk_len(self._h, max_prefill_tokens))

    def force_state(self, state: int, prefill_offset: int, generated: Sequence[int]) -> None:
        g, n = _u32(generated)
        lib.b200_request_force_state(self._h, state, prefill_offset, g, n)


class SchedBlockManager:
    """scheduler.BlockManager (src/scheduler.zig:22-95): bump counter, a view of a
    PagedBlockManager (initWithReal), or a view of a device page pool (``kv=``)."""

    def __init__(self, total_blocks: int = 0, real: Optional[PagedBlockManager] = None, kv=None):
        self._real, self._kv = real, kv
        if real is not None:
            self._h = lib.b200_sched_bm_create_with_real(real._h)
        elif kv is not None:
            self._h = lib.b200_sched_bm_create_with_kv(kv._h)
            if not self._h:
                raise B200Error(_lib.ERR_CUDA)
        else:
            self._h = lib.b200_sched_bm_create(total_blocks)

    def __del__(self):
        if getattr(self, "_h", None):
            lib.b200_sched_bm_destroy(self._h)
            self._h = None

    def can_allocate(self, n: int) -> bool:
        return bool(lib.b200_sched_bm_can_allocate(self._h, n))

    def free_count(self) -> int:
        return int(lib.b200_sched_bm_free_count(self._h))

    @property
    def total_blocks(self) -> int:
        return int(lib.b200_sched_bm_total_blocks(self._h))

    @property
    def used_blocks(self) -> int:
        return int(lib.b200_sched_bm_used_blocks(self._h))


class ScheduleResult:
    """scheduler.ScheduleResult (src/scheduler.zig:202-216)."""

    def __init__(self, prefill_requests: List[Request], decode_requests: List[Request], blocks_needed: int):
        self.prefill_requests = list(prefill_requests)
        self.decode_requests = list(decode_requests)
        self.blocks_needed = blocks_needed

    def total_requests(self) -> int:
        return len(self.prefill_requests) + len(self.decode_requests)

    def is_empty(self) -> bool:
        return self.total_requests() == 0


class Scheduler:
    """scheduler.Scheduler (src/scheduler.zig:222-387)."""

    def __init__(self, block_manager: SchedBlockManager, max_prefill_tokens: int):
        self.block_manager = block_manager
        self.max_prefill_tokens = max_prefill_tokens
        self._h = lib.b200_scheduler_create(block_manager._h, max_prefill_tokens)
        self._by_handle = {}

    def __del__(self):
        if getattr(self, "_h", None):
            lib.b200_scheduler_destroy(self._h)
            self._h = None

    def add_request(self, req: Request) -> None:
        self._by_handle[req._h] = req
        _lib.check(lib.b200_scheduler_add_request(self._h, req._h))

    def schedule(self) -> ScheduleResult:
        cap = max(len(self._by_handle), 1)
        pre, dec = (C.c_void_p * cap)(), (C.c_void_p * cap)()
        n_pre, n_dec, need = C.c_uint64(), C.c_uint64(), C.c_uint64()
        _lib.check(lib.b200_scheduler_schedule(self._h, pre, C.byref(n_pre), dec, C.byref(n_dec), cap, C.byref(need)))
        return ScheduleResult([self._by_handle[pre[i]] for i in range(n_pre.value)],
                              [self._by_handle[dec[i]] for i in range(n_dec.value)], int(need.value))

    def postprocess(self, outputs: Sequence[Tuple[int, int]]) -> None:
        arr = (_lib.TokenOutput * max(len(outputs), 1))()
        for i, (rid, tok) in enumerate(outputs):
            arr[i].request_id, arr[i].token = rid, tok
        _lib.check(lib.b200_scheduler_postprocess(self._h, arr, len(outputs)))
        for h in [h for h, r in self._by_handle.items() if r.state == DONE]:
            del self._by_handle[h]

    def active_count(self) -> int:
        return int(lib.b200_scheduler_active_count(self._h))

    def remove(self, req: Request, error: int) -> None:
        _lib.check(lib.b200_scheduler_remove(self._h, req._h, error))
        self._by_handle.pop(req._h, None)

    def preempt(self, req: Request) -> None:
        _lib.check(lib.b200_scheduler_preempt(self._h, req._h))

    def hold_admission(self, on: bool) -> None:
        lib.b200_scheduler_hold_admission(self._h, int(on))

    def set_admission_budget(self, pages: Optional[int]) -> None:
        lib.b200_scheduler_set_admission_budget(self._h, 2 ** 64 - 1 if pages is None else int(pages))

    def waiting_count(self) -> int:
        return int(lib.b200_scheduler_waiting_count(self._h))

    def running_count(self) -> int:
        return int(lib.b200_scheduler_running_count(self._h))


class BatchResult:
    """batch_builder.BatchResult (src/batch_builder.zig:24-42) plus the ragged descriptors."""

    def __init__(self, tokens, positions, cu, row_to_req, total, n_req):
        self.batched_tokens = tokens
        self.position_ids = positions
        self.cu_seqlens = cu
        self.row_to_req = row_to_req
        self.total_tokens = total
        self.num_requests = n_req
        self._mask = None

    @property
    def attention_mask(self) -> np.ndarray:
        if self._mask is None:
            t = self.total_tokens
            m = np.zeros((t, t), np.float32)
            if t:
                cu = np.ascontiguousarray(self.cu_seqlens, np.int32)
                _lib.check(lib.b200_batch_mask(cu.ctypes.data_as(C.POINTER(C.c_int32)), self.num_requests,
                                               m.ctypes.data_as(C.POINTER(C.c_float)), t))
            self._mask = m
        return self._mask


def build_batch(sched: ScheduleResult, chunked: bool = False, max_prefill_tokens: int = 0) -> BatchResult:
    """batch_builder.build (src/batch_builder.zig:90-214)."""
    pre, dec = sched.prefill_requests, sched.decode_requests
    cap = sum(len(r.prompt_tokens) for r in pre) + len(pre) + len(dec) + 1
    pa = (C.c_void_p * max(len(pre), 1))(*[r._h for r in pre])
    da = (C.c_void_p * max(len(dec), 1))(*[r._h for r in dec])
    tokens = np.zeros(cap, np.uint32)
    positions = np.zeros(cap, np.int32)
    row_to_req = np.zeros(cap, np.int32)
    cu = np.zeros(len(pre) + len(dec) + 1, np.int32)
    total, n_req = C.c_uint64(), C.c_uint64()
    _lib.check(lib.b200_batch_build(pa, len(pre), da, len(dec), int(chunked), max_prefill_tokens,
                                    tokens.ctypes.data_as(C.POINTER(C.c_uint32)),
                                    positions.ctypes.data_as(C.POINTER(C.c_int32)),
                                    row_to_req.ctypes.data_as(C.POINTER(C.c_int32)), cap,
                                    cu.ctypes.data_as(C.POINTER(C.c_int32)), C.byref(total), C.byref(n_req)))
    t = int(total.value)
    if t == 0:
        cu = np.zeros(1, np.int32)
    return BatchResult(tokens[:t], positions[:t], cu, row_to_req[:t], t, int(n_req.value))


def is_attending(mask: np.ndarray, row: int, col: int) -> bool:
    """batch_builder.isAttending (src/batch_builder.zig:253-256)."""
    return bool(mask[row, col] == 0.0)


def is_attending_ragged(cu_seqlens: np.ndarray, row: int, col: int) -> bool:
    cu = np.ascontiguousarray(cu_seqlens, np.int32)
    return bool(lib.b200_is_attending(cu.ctypes.data_as(C.POINTER(C.c_int32)), len(cu) - 1, row, col))


def greedy(logits: np.ndarray) -> int:
    """sampling.greedy (src/sampling.zig:22-39)."""
    a = np.ascontiguousarray(logits, np.float32)
    return int(lib.b200_greedy_host(a.ctypes.data_as(C.POINTER(C.c_float)), a.size))
