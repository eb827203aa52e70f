"""CPU restatement of the reference's host-side (integer) semantics.

TEST INFRASTRUCTURE ONLY.  Nothing under ``dmlx_b200/`` may import this module; it is the
checker the CUDA/C++ product is compared against, never the thing shipped or measured.

Each class cites the reference file:line it follows (paths relative to the reference tree).

Pinning status: the reference's own integer tests for this path (scheduler_tests.zig,
batch_builder_tests.zig, kvcache_tests.zig, integration_tests.zig) are restated as
known-answer cases in ``tests/test_oracle_host.py``; this module must pass them before it is
used as a checker.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

PAGE_SIZE = 32  # src/kvcache/paged.zig:24  default_page_size


class InsufficientBlocks(Exception):
    """src/kvcache/paged.zig:109,174 / src/scheduler.zig:64  error.InsufficientBlocks"""


class InvalidBlockId(Exception):
    """src/kvcache/paged.zig:168,269  error.InvalidBlockId"""


class InvalidBatchIndex(Exception):
    """src/kvcache/paged.zig:904  error.InvalidBatchIndex"""


# ---------------------------------------------------------------------------
# paged.BlockManager  (src/kvcache/paged.zig:44-273)
# ---------------------------------------------------------------------------


def hash_block(prev_hash: int, token_ids: Sequence[int]) -> int:
    """Chained 64-bit block hash (src/kvcache/paged.zig:224-230).

    The reference uses Zig's std.hash.Wyhash seeded with the previous block's hash over the raw
    little-endian bytes of the u32 token ids.  Its tests pin determinism and chain sensitivity only
    (src/tests/kvcache_tests.zig:654-669), never a hash value, so any collision-free chained 64-bit
    hash yields the same block tables.  This oracle and the product both use FNV-1a-64 over the
    8 seed bytes followed by the token bytes.
    """
    h = 0xCBF29CE484222325
    data = int(prev_hash & 0xFFFFFFFFFFFFFFFF).to_bytes(8, "little") + np.asarray(
        token_ids, dtype="<u4"
    ).tobytes()
    for b in data:
        h ^= b
        h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


@dataclass
class Block:
    """src/kvcache/paged.zig:30-38 (array payload omitted: data lives on the device)."""

    used: bool = False
    ref_count: int = 0
    hash: Optional[int] = None
    last_access: int = 0
    tokens_used: int = 0


class PagedBlockManager:
    """LIFO free-stack page allocator with ref-counts, CoW and prefix hashes.

    Follows src/kvcache/paged.zig:44-273.  ``free_blocks`` is a stack initialised so that the first
    pops return 0,1,2,... (:61-73); frees push on top (:156).
    """

    def __init__(self, total_blocks: int):
        self.total_blocks = total_blocks
        self.free_blocks: List[int] = [total_blocks - 1 - i for i in range(total_blocks)]
        self.block_pool: List[Block] = [Block() for _ in range(total_blocks)]
        self.req_to_blocks: Dict[int, List[int]] = {}
        self.block_hashes: Dict[int, int] = {}
        self.access_counter = 0

    def can_allocate(self, n: int) -> bool:  # :102-104
        return len(self.free_blocks) >= n

    def allocate_blocks(self, req_id: int, n: int) -> List[int]:  # :108-137
        if not self.can_allocate(n):
            raise InsufficientBlocks()
        self.access_counter += 1
        out = []
        for _ in range(n):
            bid = self.free_blocks.pop()
            b = self.block_pool[bid]
            b.used, b.ref_count, b.last_access = True, 1, self.access_counter
            b.tokens_used, b.hash = 0, None
            out.append(bid)
        self.req_to_blocks.setdefault(req_id, []).extend(out)
        return out

    def free_blocks_of(self, req_id: int) -> None:  # :142-162
        lst = self.req_to_blocks.pop(req_id, None)
        if lst is None:
            return
        for bid in lst:
            if bid < len(self.block_pool):
                b = self.block_pool[bid]
                if b.ref_count > 1:
                    b.ref_count -= 1
                else:
                    b.ref_count, b.used, b.hash, b.tokens_used = 0, False, None, 0
                    self.free_blocks.append(bid)

    def copy_on_write(self, block_id: int) -> int:  # :167-206
        if block_id >= len(self.block_pool):
            raise InvalidBlockId()
        b = self.block_pool[block_id]
        if b.ref_count <= 1:
            return block_id
        if not self.free_blocks:
            raise InsufficientBlocks()
        new_id = self.free_blocks.pop()
        nb = self.block_pool[new_id]
        nb.used, nb.ref_count, nb.hash = True, 1, b.hash
        nb.last_access, nb.tokens_used = self.access_counter, b.tokens_used
        b.ref_count -= 1
        return new_id

    def free_count(self) -> int:  # :209-211
        return len(self.free_blocks)

    def used_count(self) -> int:  # :214-216
        return self.total_blocks - len(self.free_blocks)

    def find_cached_prefix(self, token_ids: Sequence[int], block_size: int) -> List[int]:  # :234-265
        if block_size == 0:
            return []
        out: List[int] = []
        prev, off = 0, 0
        while off + block_size <= len(token_ids):
            h = hash_block(prev, token_ids[off : off + block_size])
            bid = self.block_hashes.get(h)
            if bid is not None:
                b = self.block_pool[bid]
                if b.used and b.tokens_used == block_size:
                    b.ref_count += 1
                    self.access_counter += 1
                    b.last_access = self.access_counter
                    out.append(bid)
                    prev = h
                    off += block_size
                    continue
            break
        return out

    def register_block_hash(self, block_id: int, h: int) -> None:  # :268-272
        if block_id >= len(self.block_pool):
            raise InvalidBlockId()
        self.block_pool[block_id].hash = h
        self.block_hashes[h] = block_id

    # -- field access used by the reference's tests (they poke block_pool.items[i] directly) --
    def get_ref(self, bid: int) -> int:
        return self.block_pool[bid].ref_count

    def set_ref(self, bid: int, n: int) -> None:
        self.block_pool[bid].ref_count = n

    def is_used(self, bid: int) -> bool:
        return self.block_pool[bid].used

    def get_tokens_used(self, bid: int) -> int:
        return self.block_pool[bid].tokens_used

    def set_tokens_used(self, bid: int, n: int) -> None:
        self.block_pool[bid].tokens_used = n

    def share(self, req_id: int, bid: int) -> None:
        """Append an already-owned block to another request's list (kvcache_tests.zig:608-616)."""
        self.req_to_blocks.setdefault(req_id, []).append(bid)

    def blocks_of(self, req_id: int) -> List[int]:
        return list(self.req_to_blocks.get(req_id, []))


# ---------------------------------------------------------------------------
# scheduler.zig
# ---------------------------------------------------------------------------

WAITING, PREFILLING, DECODING, DONE = 0, 1, 2, 3  # src/scheduler.zig:101-106


@dataclass
class Request:
    """src/scheduler.zig:108-187"""

    id: int
    prompt_tokens: List[int]
    max_tokens: int
    stop_tokens: List[int] = field(default_factory=list)
    generated_tokens: List[int] = field(default_factory=list)
    state: int = WAITING
    block_ids: List[int] = field(default_factory=list)
    prefill_offset: int = 0
    folded: int = 0  # generated tokens a preemption appended to the prompt (extension, see Scheduler.preempt)
    error: int = 0   # why the request ended early (extension, see Scheduler.remove)

    def seq_len(self) -> int:  # :165-167 (minus the generated tokens that now sit in the prompt)
        return self.prefill_offset + len(self.generated_tokens) - self.folded

    def is_stop_token(self, t: int) -> bool:  # :170-175
        return t in self.stop_tokens

    def has_pending_prefill(self) -> bool:  # :178-180
        return self.prefill_offset < len(self.prompt_tokens)

    def current_prefill_chunk_len(self, max_prefill_tokens: int) -> int:  # :183-186
        return min(len(self.prompt_tokens) - self.prefill_offset, max_prefill_tokens)

    def force_state(self, state: int, prefill_offset: int, generated: Sequence[int]) -> None:
        """Test helper: the reference's tests build requests mid-flight by writing the fields
        (src/tests/batch_builder_tests.zig:27-42)."""
        self.state, self.prefill_offset = state, prefill_offset
        self.generated_tokens = list(generated)


class SchedBlockManager:
    """Scheduler-side wrapper (src/scheduler.zig:22-95): bump counter, or a view of the real pool."""

    def __init__(self, total_blocks: int = 0, real: Optional[PagedBlockManager] = None):
        self.real = real
        self.total_blocks = real.total_blocks if real else total_blocks
        self.used_blocks = real.used_count() if real else 0

    def can_allocate(self, n: int) -> bool:  # :46-51
        if self.real:
            return self.real.can_allocate(n)
        return self.free_count() >= n

    def allocate_blocks(self, req: Request, n: int) -> None:  # :54-70
        if self.real:
            req.block_ids.extend(self.real.allocate_blocks(req.id, n))
            self.used_blocks = self.real.used_count()
            return
        if not self.can_allocate(n):
            raise InsufficientBlocks()
        for _ in range(n):
            req.block_ids.append(self.used_blocks)
            self.used_blocks += 1

    def free_blocks(self, req: Request) -> None:  # :73-87
        if self.real:
            self.real.free_blocks_of(req.id)
            self.used_blocks = self.real.used_count()
            req.block_ids.clear()
            return
        freed = len(req.block_ids)
        self.used_blocks = self.used_blocks - freed if freed <= self.used_blocks else 0
        req.block_ids.clear()

    def free_count(self) -> int:  # :89-94
        if self.real:
            return self.real.free_count()
        return self.total_blocks - self.used_blocks


@dataclass
class ScheduleResult:  # src/scheduler.zig:202-216
    prefill_requests: List[Request]
    decode_requests: List[Request]
    blocks_needed: int

    def total_requests(self) -> int:
        return len(self.prefill_requests) + len(self.decode_requests)

    def is_empty(self) -> bool:
        return self.total_requests() == 0


class Scheduler:
    """src/scheduler.zig:222-387"""

    def __init__(self, block_manager: SchedBlockManager, max_prefill_tokens: int):
        self.waiting: List[Request] = []
        self.running: List[Request] = []
        self.block_manager = block_manager
        self.max_prefill_tokens = max_prefill_tokens
        self.blocks_per_request = 1  # :242
        self.hold = False  # extension: schedule() promotes nobody while set
        self.admission_budget: Optional[int] = None  # extension: pages one schedule() may promise to newcomers

    def add_request(self, req: Request) -> None:  # :252-255
        req.state = WAITING
        self.waiting.append(req)

    def schedule(self) -> ScheduleResult:  # :267-315
        decode_list, prefill_list = [], []
        for req in self.running:
            if req.state == PREFILLING and req.has_pending_prefill():
                prefill_list.append(req)
            else:
                decode_list.append(req)
        still_waiting, blocks_needed = [], 0
        budget, closed = self.admission_budget, self.hold
        for req in self.waiting:
            prompt_pages = -(-(len(req.prompt_tokens) + 1) // PAGE_SIZE)
            if not closed and budget is not None and prompt_pages > budget:
                closed = True  # arrival order: nobody overtakes the first request that does not fit
            if not closed and self.block_manager.can_allocate(self.blocks_per_request):
                if budget is not None:
                    budget -= prompt_pages
                self.block_manager.allocate_blocks(req, self.blocks_per_request)
                req.state = PREFILLING
                prefill_list.append(req)
                self.running.append(req)
            else:
                blocks_needed += self.blocks_per_request
                still_waiting.append(req)
        self.waiting = still_waiting
        return ScheduleResult(prefill_list, decode_list, blocks_needed)

    def postprocess(self, outputs: Sequence[Tuple[int, int]]) -> None:  # :328-381
        for rid, token in outputs:
            for req in self.running:
                if req.id != rid:
                    continue
                if req.state == PREFILLING:
                    req.prefill_offset += req.current_prefill_chunk_len(self.max_prefill_tokens)
                    if not req.has_pending_prefill():
                        req.state = DECODING
                        req.generated_tokens.append(token)
                        if req.is_stop_token(token) or len(req.generated_tokens) >= req.max_tokens:
                            req.state = DONE
                else:
                    req.generated_tokens.append(token)
                    if req.is_stop_token(token) or len(req.generated_tokens) >= req.max_tokens:
                        req.state = DONE
                break
        i = 0
        while i < len(self.running):
            if self.running[i].state == DONE:
                self.block_manager.free_blocks(self.running[i])
                self.running.pop(i)
            else:
                i += 1

    def active_count(self) -> int:  # :384-386
        return len(self.running) + len(self.waiting)

    # ---- extensions with no counterpart in scheduler.zig (the engine loop's handleBatchError and
    # cancel flag, src/engine/engine_loop.zig:687-754, src/engine/request_state.zig:182-189, and a
    # preemption rule for an exhausted pool) -----------------------------------------------------
    def remove(self, req: Request, error: int) -> None:
        if req in self.running:
            self.running.remove(req)
            self.block_manager.free_blocks(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        else:
            raise ValueError("request is not active")
        req.state, req.error = DONE, error

    def preempt(self, req: Request) -> None:
        self.running.remove(req)
        self.block_manager.free_blocks(req)
        req.prompt_tokens = list(req.prompt_tokens) + list(req.generated_tokens[req.folded:])
        req.folded = len(req.generated_tokens)
        req.prefill_offset = 0
        req.state = WAITING
        self.waiting.insert(0, req)

    def hold_admission(self, on: bool) -> None:
        self.hold = bool(on)

    def set_admission_budget(self, pages: Optional[int]) -> None:
        self.admission_budget = pages


# ---------------------------------------------------------------------------
# batch_builder.zig
# ---------------------------------------------------------------------------


def get_request_tokens(req: Request, chunked: bool = False, max_prefill_tokens: int = 0) -> List[int]:
    """src/batch_builder.zig:47-83.  ``chunked`` caps a prefilling request at its current chunk
    (src/scheduler.zig:183-186); the reference itself never caps (pinned by
    src/tests/integration_tests.zig:833-838)."""
    if req.state in (PREFILLING, WAITING):
        start, end = req.prefill_offset, len(req.prompt_tokens)
        if start >= end:
            return [req.prompt_tokens[end - 1]] if end > 0 else []
        if chunked:
            end = start + req.current_prefill_chunk_len(max_prefill_tokens)
        return list(req.prompt_tokens[start:end])
    if req.state == DECODING:
        if req.generated_tokens:
            return [req.generated_tokens[-1]]
        if req.prompt_tokens:
            return [req.prompt_tokens[-1]]
        return []
    return []


@dataclass
class BatchResult:
    """src/batch_builder.zig:24-42, plus the ragged descriptors the product emits in place of the
    T x T mask (cu_seqlens / row_to_req); the mask is derivable from them (see is_attending)."""

    batched_tokens: np.ndarray  # [T] u32
    position_ids: np.ndarray  # [T] i32
    attention_mask: np.ndarray  # [T,T] f32, 0 / -inf
    total_tokens: int
    num_requests: int
    cu_seqlens: np.ndarray  # [R+1] i32
    row_to_req: np.ndarray  # [T] i32


def build_batch(sched: ScheduleResult, chunked: bool = False, max_prefill_tokens: int = 0,
                with_mask: bool = True) -> BatchResult:
    """src/batch_builder.zig:90-214: prefill requests first, then decode requests."""
    reqs = list(sched.prefill_requests) + list(sched.decode_requests)
    toks = [get_request_tokens(r, chunked, max_prefill_tokens) for r in reqs]
    total = sum(len(t) for t in toks)
    if not reqs or total == 0:
        return BatchResult(np.zeros(0, np.uint32), np.zeros(0, np.int32), np.zeros((0, 0), np.float32),
                           0, 0, np.zeros(1, np.int32), np.zeros(0, np.int32))
    all_tok = np.zeros(total, np.uint32)
    all_pos = np.zeros(total, np.int32)
    row_to_req = np.zeros(total, np.int32)
    cu = np.zeros(len(reqs) + 1, np.int32)
    mask = np.full((total, total), -np.inf, np.float32) if with_mask else np.zeros((0, 0), np.float32)
    off = 0
    for i, (req, t) in enumerate(zip(reqs, toks)):
        n = len(t)
        all_tok[off : off + n] = t
        if req.state in (PREFILLING, WAITING):
            base = req.prefill_offset  # :160
        elif req.state == DECODING:
            base = req.seq_len() - n if req.seq_len() > 0 else 0  # :161
        else:
            base = 0
        all_pos[off : off + n] = base + np.arange(n)
        row_to_req[off : off + n] = i
        if with_mask:
            for row in range(n):
                mask[off + row, off : off + row + 1] = 0.0  # :170-177
        off += n
        cu[i + 1] = off
    return BatchResult(all_tok, all_pos, mask, total, len(reqs), cu, row_to_req)


def is_attending(mask: np.ndarray, row: int, col: int) -> bool:  # src/batch_builder.zig:253-256
    return bool(mask[row, col] == 0.0)


def is_attending_ragged(cu_seqlens: np.ndarray, row: int, col: int) -> bool:
    """The same predicate computed from cu_seqlens: same segment and col <= row."""
    seg_r = int(np.searchsorted(cu_seqlens, row, side="right")) - 1
    seg_c = int(np.searchsorted(cu_seqlens, col, side="right")) - 1
    return seg_r == seg_c and col <= row


# ---------------------------------------------------------------------------
# Paged KV page tables (src/kvcache/paged.zig:505-531, 842-945) on the LIFO pool
# ---------------------------------------------------------------------------


class PagedKVTables:
    """Integer state of the Paged strategy: per-sequence page tables over one shared pool.

    Page growth follows src/kvcache/paged.zig:525-531 (ensure ceil((len+S)/page) pages, in batch
    order) with page ids drawn from the LIFO stack of paged.BlockManager (:116-118) — the
    allocator whose free list the product keeps in device memory.  Before a sequence writes into a
    partially filled last page that is shared (ref_count > 1) it takes a private copy
    (copyOnWrite, :167-206).  ``release`` is freeBlocks (:142-162); ``rollback`` pops pages
    (:864-877); ``fork`` shares a prefix by ref-count (the effect of findCachedPrefix :247-256).
    """

    def __init__(self, total_pages: int, max_seqs: int, page_size: int = PAGE_SIZE):
        self.page_size = page_size
        self.free: List[int] = [total_pages - 1 - i for i in range(total_pages)]
        self.ref = [0] * total_pages
        self.tokens_used = [0] * total_pages
        self.tables: List[List[int]] = [[] for _ in range(max_seqs)]
        self.lens = [0] * max_seqs
        self.cow_log: List[Tuple[int, int]] = []  # (src page, dst page) in order

    def free_count(self) -> int:
        return len(self.free)

    def alloc(self, seq: int, n: int) -> List[int]:
        if len(self.free) < n:
            raise InsufficientBlocks()
        out = []
        for _ in range(n):
            p = self.free.pop()
            self.ref[p] = 1
            self.tokens_used[p] = 0
            out.append(p)
        self.tables[seq].extend(out)
        return out

    def reserve(self, seqs: Sequence[int], n_new: Sequence[int]) -> None:
        """Grow the page tables for one packed step; requests in batch order."""
        ps = self.page_size
        # all-or-nothing check first so a failed step leaves the state untouched
        need = 0
        ref_sim: Dict[int, int] = {}
        for s, n in zip(seqs, n_new):
            if n <= 0:
                continue
            ln = self.lens[s]
            if ln % ps != 0 and self.tables[s]:
                last = self.tables[s][ln // ps]
                r = ref_sim.get(last, self.ref[last])
                if r > 1:
                    need += 1
                    ref_sim[last] = r - 1
            need += max(0, -(-(ln + n) // ps) - len(self.tables[s]))
        if need > len(self.free):
            raise InsufficientBlocks()
        for s, n in zip(seqs, n_new):
            if n <= 0:
                continue
            ln = self.lens[s]
            if ln % ps != 0:
                idx = ln // ps
                last = self.tables[s][idx]
                if self.ref[last] > 1:
                    new = self.free.pop()
                    self.ref[new] = 1
                    self.tokens_used[new] = self.tokens_used[last]
                    self.ref[last] -= 1
                    self.tables[s][idx] = new
                    self.cow_log.append((last, new))
            pages_needed = -(-(ln + n) // ps)
            while len(self.tables[s]) < pages_needed:
                p = self.free.pop()
                self.ref[p] = 1
                self.tokens_used[p] = 0
                self.tables[s].append(p)
            # per-page fill counts
            for pos in range(ln, ln + n):
                self.tokens_used[self.tables[s][pos // ps]] = pos % ps + 1
            self.lens[s] = ln + n

    def release(self, seq: int) -> None:
        for p in self.tables[seq]:
            if self.ref[p] > 1:
                self.ref[p] -= 1
            else:
                self.ref[p] = 0
                self.tokens_used[p] = 0
                self.free.append(p)
        self.tables[seq] = []
        self.lens[seq] = 0

    def fork(self, src: int, dst: int, n_tokens: int) -> None:
        """dst shares the pages covering src's first n_tokens tokens (ref_count += 1 each)."""
        assert not self.tables[dst] and n_tokens <= self.lens[src]
        n_pages = -(-n_tokens // self.page_size)
        for p in self.tables[src][:n_pages]:
            self.ref[p] += 1
        self.tables[dst] = list(self.tables[src][:n_pages])
        self.lens[dst] = n_tokens

    def rollback(self, seq: int, to_len: int) -> None:  # paged.zig:864-877 on one sequence
        need = -(-to_len // self.page_size)
        while len(self.tables[seq]) > need:
            p = self.tables[seq].pop()
            if self.ref[p] > 1:
                self.ref[p] -= 1
            else:
                self.ref[p] = 0
                self.tokens_used[p] = 0
                self.free.append(p)
        self.lens[seq] = min(self.lens[seq], to_len)

    def current_len(self) -> int:  # paged.zig:842-849
        return max(self.lens) if self.lens else 0

    def filter(self, keep: Sequence[int]) -> None:
        """paged.zig:879-945: reference counts are derived afresh from the page tables of the
        sequences that stay (:898-914); pages nobody references any more are free again (:939-944).
        Sequence slots keep their numbers here (the reference compacts them to 0..n-1), and a freed
        page returns to the LIFO stack at the (slot, table position) of the last dropped sequence that
        listed it."""
        for s in keep:
            if s < 0 or s >= len(self.tables):
                raise InvalidBatchIndex()  # :904
        kept = set(keep)
        new_ref = [0] * len(self.ref)
        for s in kept:
            for p in self.tables[s]:
                new_ref[p] += 1
        dropped = [s for s in range(len(self.tables)) if s not in kept]
        holders = [0] * len(self.ref)  # dropped tables that still list the page
        for s in dropped:
            for p in self.tables[s]:
                holders[p] += 1
        for s in dropped:
            for p in self.tables[s]:
                holders[p] -= 1
                if new_ref[p] == 0 and holders[p] == 0:  # freed where its last holder goes
                    self.tokens_used[p] = 0
                    self.free.append(p)
            self.tables[s] = []
            self.lens[s] = 0
        for p in range(len(self.ref)):
            if self.ref[p] > 0:
                self.ref[p] = new_ref[p]

    def reset(self) -> None:
        """paged.zig:851-862: every page unused, every sequence empty.  The pool is as new: pages pop
        in the order 0, 1, 2, ... again."""
        n = len(self.ref)
        self.free = [n - 1 - i for i in range(n)]
        self.ref = [0] * n
        self.tokens_used = [0] * n
        self.tables = [[] for _ in self.tables]
        self.lens = [0] * len(self.lens)


def greedy(logits: np.ndarray) -> int:
    """First strict maximum (src/sampling.zig:22-39)."""
    best, idx = logits[0], 0
    for i in range(1, len(logits)):
        if logits[i] > best:
            best, idx = logits[i], i
    return idx
