"""Device-side Python surface: torch tensors carry device memory and streams, every operation
is a call into libdmlx_b200 through the C-ABI.  There is no torch or CPU implementation behind
these calls — without the library or without a GPU they raise.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import KvConfig, PackDesc, lib

KV_BF16, KV_FP8_E4M3 = 0, 1
Q_AFFINE4_G64, Q_MXFP4_G32 = 0, 1
EPI_NONE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
QMM_AUTO, QMM_SIMT, QMM_TCGEN05, QMM_MMA, QMM_TCGEN05_X2, QMM_TCGEN05_TMEM_A, QMM_MXFP4_BLOCK_SCALED, QMM_MMA_I8 = 0, 1, 2, 3, 4, 5, 6, 7


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device tensors must be contiguous CUDA tensors"
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def pack_desc_array(descs: Sequence[Sequence[int]]) -> torch.Tensor:
    """[(seq_slot, count, base_pos, src_offset)] -> pinned int32 [R,4] host tensor."""
    a = torch.tensor(list(descs), dtype=torch.int32).reshape(-1, 4)
    return a.pin_memory() if torch.cuda.is_available() else a


class PackedBatch:
    """Device-resident result of pack_batch (the ragged stand-in for BatchResult)."""

    def __init__(self, n_req: int, total_rows: int, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.n_req, self.total_rows = n_req, total_rows
        self.cu_seqlens = torch.empty(n_req + 1, **i32)
        self.token_ids = torch.empty(max(total_rows, 1), dtype=torch.int32, device=device)  # u32 payload
        self.position_ids = torch.empty(max(total_rows, 1), **i32)
        self.row_to_req = torch.empty(max(total_rows, 1), **i32)
        self.row_seq = torch.empty(max(total_rows, 1), **i32)
        self.row_ctx = torch.empty(max(total_rows, 1), **i32)
        self.last_row = torch.empty(max(n_req, 1), **i32)


def pack_batch(d_desc: torch.Tensor, total_rows: int, prefill_tokens: Optional[torch.Tensor],
               last_token: Optional[torch.Tensor], out: Optional[PackedBatch] = None) -> PackedBatch:
    """b200_pack_batch: builds cu_seqlens / positions / flat tokens on the GPU."""
    n_req = d_desc.shape[0]
    out = out or PackedBatch(n_req, total_rows, d_desc.device)
    _lib.check(lib.b200_pack_batch(_ptr(d_desc), n_req, _ptr(prefill_tokens), _ptr(last_token),
                                   _ptr(out.cu_seqlens), _ptr(out.token_ids), _ptr(out.position_ids),
                                   _ptr(out.row_to_req), _ptr(out.row_seq), _ptr(out.row_ctx), _ptr(out.last_row),
                                   total_rows, _stream()))
    return out


class PagedKVCache:
    """The Paged KVCacheStrategy on a device page pool (src/kvcache/paged.zig:305-1139).

    updateAndFetch becomes reserve() + append(): pages are written in place and attention reads
    them in place; gather() returns the contiguous view for tests.
    """

    def __init__(self, n_layers: int, n_kv_heads: int, head_dim: int, n_pages: int, max_seqs: int,
                 max_pages_per_seq: int, n_q_heads: int, max_rows: int = 4096, kv_dtype: int = KV_BF16,
                 page_size: int = 32, attn_scratch_chunks: int = 0):
        cfg = KvConfig(n_layers, n_kv_heads, head_dim, page_size, n_pages, max_seqs, max_pages_per_seq, kv_dtype,
                       max_rows, n_q_heads, attn_scratch_chunks)
        h = C.c_void_p()
        _lib.check(lib.b200_kv_create(C.byref(cfg), C.byref(h)))
        self._h = h.value
        self.cfg = cfg

    def close(self):
        if getattr(self, "_h", None):
            lib.b200_kv_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    # -- allocator surface --
    def reset(self):
        _lib.check(lib.b200_kv_reset(self._h))

    def set_free_order(self, ids: Sequence[int]):
        arr = (C.c_int32 * len(ids))(*ids)
        _lib.check(lib.b200_kv_set_free_order(self._h, arr, len(ids)))

    def free_count(self) -> int:
        out = C.c_int32()
        _lib.check(lib.b200_kv_free_count(self._h, C.byref(out)))
        return out.value

    def alloc(self, seq: int, n: int) -> List[int]:
        out = (C.c_int32 * max(n, 1))()
        _lib.check(lib.b200_kv_alloc(self._h, seq, n, out))
        return [out[i] for i in range(n)]

    def release(self, seqs: Sequence[int]):
        arr = (C.c_int32 * max(len(seqs), 1))(*seqs)
        _lib.check(lib.b200_kv_release(self._h, arr, len(seqs)))

    def fork(self, src: int, dst: int, n_tokens: int):
        _lib.check(lib.b200_kv_fork(self._h, src, dst, n_tokens))

    def extend(self, dst_seq: int, src: "PagedKVCache", src_seq: int):
        """VTable.extend: copy sequence src_seq of another pool into the empty slot dst_seq."""
        _lib.check(lib.b200_kv_extend(self._h, dst_seq, src._h, src_seq))

    def rollback(self, seq: int, to_len: int):
        _lib.check(lib.b200_kv_rollback(self._h, seq, to_len))

    def filter(self, keep: Sequence[int]):
        arr = (C.c_int32 * max(len(keep), 1))(*keep)
        _lib.check(lib.b200_kv_filter(self._h, arr, len(keep)))

    # -- step surface --
    def reserve(self, d_desc: torch.Tensor):
        _lib.check(lib.b200_kv_reserve(self._h, _ptr(d_desc), d_desc.shape[0], _stream()))

    def rope_append(self, layer: int, q: torch.Tensor, k_rows: torch.Tensor, v_rows: torch.Tensor, positions: torch.Tensor,
                    row_seq: torch.Tensor, theta: float = 10000.0):
        """b200_kv_rope_append: rotate q and k in place, then append k and v to the pages reserved for this step."""
        _lib.check(lib.b200_kv_rope_append(self._h, layer, _ptr(q), _ptr(k_rows), _ptr(v_rows), _ptr(positions), _ptr(row_seq),
                                           q.shape[0], q.shape[1], theta, _stream()))

    def rope_append_partials(self, layer: int, parts, q_buf: torch.Tensor, q_stride: int, positions: torch.Tensor, row_seq: torch.Tensor,
                             n_q_heads: int, theta: float = 10000.0):
        """b200_kv_rope_append_partials: RoPE + append fed from the split-K partial sums of the q/k/v projection."""
        _lib.check(lib.b200_kv_rope_append_partials(self._h, layer, C.byref(parts), _ptr(q_buf), q_stride, _ptr(positions), _ptr(row_seq),
                                                    positions.shape[0], n_q_heads, theta, _stream()))

    def append(self, layer: int, k_rows: torch.Tensor, v_rows: torch.Tensor):
        assert k_rows.dtype == torch.bfloat16 and v_rows.dtype == torch.bfloat16
        _lib.check(lib.b200_kv_append(self._h, layer, _ptr(k_rows), _ptr(v_rows), k_rows.shape[0], _stream()))

    def attention(self, layer: int, q: torch.Tensor, row_seq: torch.Tensor, row_ctx: torch.Tensor,
                  out: Optional[torch.Tensor] = None, prefill: bool = False) -> torch.Tensor:
        """b200_paged_attn_decode (or b200_paged_attn_prefill: same results, rows of a prefill chunk
        served in groups). q: [T, Hq, D] bf16."""
        out = out if out is not None else torch.empty_like(q)
        fn = lib.b200_paged_attn_prefill if prefill else lib.b200_paged_attn_decode
        _lib.check(fn(self._h, layer, _ptr(q), _ptr(row_seq), _ptr(row_ctx), q.shape[0], _ptr(out), _stream()))
        return out

    # -- introspection --
    def seq_len(self, seq: int) -> int:
        out = C.c_int32()
        _lib.check(lib.b200_kv_seq_len(self._h, seq, C.byref(out)))
        return out.value

    def current_len(self) -> int:
        out = C.c_int32()
        _lib.check(lib.b200_kv_current_len(self._h, C.byref(out)))
        return out.value

    def block_table(self, seq: int) -> List[int]:
        cap = self.cfg.max_pages_per_seq
        out = (C.c_int32 * cap)()
        n = C.c_int32()
        _lib.check(lib.b200_kv_block_table(self._h, seq, out, cap, C.byref(n)))
        return [out[i] for i in range(n.value)]

    def ref_counts(self) -> np.ndarray:
        out = np.zeros(self.cfg.n_pages, np.int32)
        _lib.check(lib.b200_kv_ref_counts(self._h, out.ctypes.data_as(C.POINTER(C.c_int32)), out.size))
        return out

    def error_word(self) -> int:
        out = C.c_int32()
        _lib.check(lib.b200_kv_error_word(self._h, C.byref(out)))
        return out.value

    def gather(self, layer: int, seq: int):
        n = self.seq_len(seq)
        shape = (max(n, 1), self.cfg.n_kv_heads, self.cfg.head_dim)
        k = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
        v = torch.empty_like(k)
        _lib.check(lib.b200_kv_gather(self._h, layer, seq, _ptr(k), _ptr(v), n, _stream()))
        return k[:n], v[:n]

    def page_raw(self, layer: int, page: int):
        c = self.cfg
        eb = 2 if c.kv_dtype == KV_BF16 else 1
        nbytes = c.n_kv_heads * c.page_size * c.head_dim * eb
        k, v = np.zeros(nbytes, np.uint8), np.zeros(nbytes, np.uint8)
        ks, vs = np.zeros(c.n_kv_heads, np.float32), np.zeros(c.n_kv_heads, np.float32)
        _lib.check(lib.b200_kv_page_raw(self._h, layer, page, k.ctypes.data, v.ctypes.data,
                                        ks.ctypes.data_as(C.POINTER(C.c_float)), vs.ctypes.data_as(C.POINTER(C.c_float))))
        shape = (c.n_kv_heads, c.page_size, c.head_dim)
        if eb == 2:
            return k.view(np.uint16).reshape(shape), v.view(np.uint16).reshape(shape), ks, vs
        return k.reshape(shape), v.reshape(shape), ks, vs

    def page_load(self, layer: int, page: int, k: np.ndarray, v: np.ndarray, k_scales=None, v_scales=None):
        """Inverse of page_raw: host page bytes (and, for FP8 pools, per-head scales) into the pool."""
        k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
        fp = lambda a: None if a is None else np.ascontiguousarray(a, np.float32)
        ks, vs = fp(k_scales), fp(v_scales)
        pf = lambda a: None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))
        _lib.check(lib.b200_kv_page_load(self._h, layer, page, k.ctypes.data, v.ctypes.data, pf(ks), pf(vs)))

    def set_len(self, seq: int, n_tokens: int):
        _lib.check(lib.b200_kv_set_len(self._h, seq, n_tokens))


def set_attn_pages_per_chunk(n: int):
    lib.b200_set_attn_pages_per_chunk(n)


def set_attn_prefill_direct(on: bool):
    lib.b200_set_attn_prefill_direct(1 if on else 0)


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib.b200_launch_count())


def set_qmm_grouped_tmem_a(on: bool):
    lib.b200_set_qmm_grouped_tmem_a(int(on))


def set_qmm_grouped_block_scaled(on: bool):
    """MXFP4 grouped matmuls on tcgen05.mma kind::mxf8f6f4 (hardware block scaling)."""
    lib.b200_set_qmm_grouped_block_scaled(int(on))


def set_attn_path(path: int):
    """0 = automatic (tensor-core kernel for bf16 pools), 1 = force the CUDA-core kernel."""
    lib.b200_set_attn_path(path)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    out = out if out is not None else torch.empty_like(x)
    _lib.check(lib.b200_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), x.shape[0], x.shape[1], eps, _stream()))
    return out


def rope_(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int,
          theta: float = 10000.0, q_stride: Optional[int] = None, k_stride: Optional[int] = None):
    """In-place RoPE on q [T, Hq*D] and k [T, Hkv*D] rows (strides in elements)."""
    rows = positions.shape[0]
    q_stride = q_stride if q_stride is not None else n_q_heads * head_dim
    k_stride = k_stride if k_stride is not None else n_kv_heads * head_dim
    _lib.check(lib.b200_rope(q.data_ptr(), k.data_ptr(), _ptr(positions), rows, n_q_heads, n_kv_heads, head_dim,
                             q_stride, k_stride, theta, _stream()))


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows = ids.shape[0]
    out = out if out is not None else torch.empty((rows, table.shape[1]), dtype=torch.bfloat16, device=table.device)
    _lib.check(lib.b200_embed_gather(_ptr(table), _ptr(ids), _ptr(out), rows, table.shape[1], _stream()))
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    out = out if out is not None else torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _lib.check(lib.b200_argmax(_ptr(logits), logits.shape[0], logits.shape[1], _ptr(out), _stream()))
    return out


def sample_params_array(rows) -> np.ndarray:
    """rows of (temperature, top_k, top_p, uniform[, repetition_penalty]) -> the 24-byte records of
    b200_sample_params as a [n, 6] float32 array (top_k stored by its bits)."""
    out = np.zeros((len(rows), 6), np.float32)
    for i, r in enumerate(rows):
        out[i, 0], out[i, 1], out[i, 3] = r[0], r[2], r[3]
        out[i, 2] = r[4] if len(r) > 4 else 1.0
    out.view(np.int32)[:, 4] = [int(r[1]) for r in rows]
    return out


def sample_rows(logits: torch.Tensor, rows, context: Optional[Sequence[Sequence[int]]] = None, logprobs: bool = True):
    """SamplerConfig.sample per row (src/sampling.zig:298-322) on bf16 or f32 logits [R, V].
    Returns (tokens int32 [R], logprobs float32 [R] or None)."""
    assert logits.dtype in (torch.bfloat16, torch.float32) and logits.is_contiguous()
    n, v = logits.shape
    d_params = torch.from_numpy(sample_params_array(rows)).to(logits.device)
    tokens = torch.empty(n, dtype=torch.int32, device=logits.device)
    lp = torch.empty(n, dtype=torch.float32, device=logits.device) if logprobs else None
    d_ctx = d_off = scratch = None
    if context is not None:
        flat = [int(t) for c in context for t in c]
        offs = np.concatenate([[0], np.cumsum([len(c) for c in context])]).astype(np.int32)
        d_ctx = torch.tensor(flat + [0], dtype=torch.int64).to(torch.int32).to(logits.device)
        d_off = torch.from_numpy(offs).to(logits.device)
        scratch = torch.empty((n, v), dtype=torch.float32, device=logits.device)
    _lib.check(lib.b200_sample_rows(_ptr(logits), int(logits.dtype == torch.float32), n, v, _ptr(d_params), _ptr(d_ctx),
                                    _ptr(d_off), _ptr(scratch), _ptr(tokens), _ptr(lp), _stream()))
    return tokens, lp


class QWeight:
    """A quantised weight repacked into the library's tile-major device layout."""

    def __init__(self, mode: int, packed: np.ndarray, scales: np.ndarray, biases: Optional[np.ndarray], n: int, k: int,
                 n_experts: int = 1):
        packed = np.ascontiguousarray(packed)
        scales = np.ascontiguousarray(scales)
        biases = np.ascontiguousarray(biases) if biases is not None else None
        h = C.c_void_p()
        _lib.check(lib.b200_qweight_create(mode, n_experts, n, k, packed.ctypes.data, scales.ctypes.data,
                                           biases.ctypes.data if biases is not None else None, C.byref(h)))
        self._h, self.mode, self.n, self.k, self.n_experts = h.value, mode, n, k, n_experts

    @classmethod
    def random(cls, mode: int, n: int, k: int, n_experts: int = 1, seed: int = 1) -> "QWeight":
        """Synthetic weights generated on the device (b200_qweight_random)."""
        h = C.c_void_p()
        _lib.check(lib.b200_qweight_random(mode, n_experts, n, k, seed, C.byref(h)))
        w = cls.__new__(cls)
        w._h, w.mode, w.n, w.k, w.n_experts = h.value, mode, n, k, n_experts
        return w

    def export(self, expert: int = 0):
        """(packed, scales, biases) of one expert in the layouts the constructor takes (b200_qweight_export)."""
        n, k = self.n, self.k
        if self.mode == Q_AFFINE4_G64:
            packed, scales, biases = np.zeros((n, k // 8), np.uint32), np.zeros((n, k // 64), np.uint16), np.zeros((n, k // 64), np.uint16)
        elif self.mode == Q_MXFP4_G32:
            packed, scales, biases = np.zeros((n, k // 2), np.uint8), np.zeros((n, k // 32), np.uint8), None
        else:
            packed, scales, biases = np.zeros((n, k), np.uint16), np.zeros(1, np.uint8), None
        _lib.check(lib.b200_qweight_export(self._h, expert, packed.ctypes.data, scales.ctypes.data,
                                           biases.ctypes.data if biases is not None else None))
        return packed, scales, biases

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.b200_qweight_destroy(self._h)
            self._h = None


def qmm_deferred(w: "QWeight", x: torch.Tensor, out: torch.Tensor, defer: bool = True):
    """b200_qmm_deferred: the matmul with its split-K finish pass left to the caller; returns the partial-sum record."""
    parts = _lib.QmmPartials()
    _lib.check(lib.b200_qmm_deferred(w._h, _ptr(x), x.shape[0], _ptr(out), 1 if defer else 0, _stream(), C.byref(parts)))
    return parts


def qmm(w: QWeight, x: torch.Tensor, epilogue: int = EPI_NONE, residual: Optional[torch.Tensor] = None,
        swiglu_limit: float = 0.0, path: int = QMM_AUTO, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """b200_qmm: y = x . dequant(W)^T with a fused epilogue."""
    rows = x.shape[0]
    n_out = w.n // 2 if epilogue == EPI_SWIGLU else w.n
    out = out if out is not None else torch.empty((rows, n_out), dtype=torch.bfloat16, device=x.device)
    _lib.check(lib.b200_qmm(w._h, _ptr(x), rows, _ptr(out), epilogue, _ptr(residual), swiglu_limit, path, _stream()))
    return out


def qmm_residual_norm(w: QWeight, x: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float = 1e-5):
    """b200_qmm_residual_norm: y = residual + x W^T and rmsnorm(y) * norm_weight.  Returns (y, normed)."""
    y = torch.empty((x.shape[0], w.n), dtype=torch.bfloat16, device=x.device)
    h = torch.empty_like(y)
    _lib.check(lib.b200_qmm_residual_norm(w._h, _ptr(x), x.shape[0], _ptr(y), _ptr(residual), _ptr(norm_weight), eps, _ptr(h),
                                          _stream()))
    return y, h


def qmm_error_word() -> int:
    out = C.c_int32()
    _lib.check(lib.b200_qmm_error_word(C.byref(out)))
    return out.value


Q_BF16 = 2
W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_LM_HEAD = range(8)


class LlamaModel:
    """The LLaMA layer stack behind b200_llama_step (ModelVTable.forward + greedy sampling,
    src/generation.zig:47-53,104-145)."""

    def __init__(self, n_layers: int, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, ffn: int, vocab: int,
                 max_rows: int, max_reqs: int, max_seqs: int, rms_eps: float = 1e-5, rope_theta: float = 10000.0):
        self.cfg = _lib.LlamaConfig(n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_rows, max_reqs,
                                    max_seqs, rms_eps, rope_theta)
        h = C.c_void_p()
        _lib.check(lib.b200_llama_create(C.byref(self.cfg), C.byref(h)))
        self._h = h.value

    def close(self):
        if getattr(self, "_h", None):
            lib.b200_llama_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def set_linear(self, layer: int, which: int, mode: int, packed: np.ndarray, scales: Optional[np.ndarray] = None,
                   biases: Optional[np.ndarray] = None):
        packed = np.ascontiguousarray(packed)
        scales = np.ascontiguousarray(scales) if scales is not None else None
        biases = np.ascontiguousarray(biases) if biases is not None else None
        _lib.check(lib.b200_llama_set_linear(self._h, layer, which, mode, packed.ctypes.data,
                                             scales.ctypes.data if scales is not None else None,
                                             biases.ctypes.data if biases is not None else None))

    def set_embedding(self, table_bf16_bits: np.ndarray):
        t = np.ascontiguousarray(table_bf16_bits, np.uint16)
        _lib.check(lib.b200_llama_set_embedding(self._h, t.ctypes.data))

    def set_norm(self, layer: int, which: int, w_bf16_bits: np.ndarray):
        t = np.ascontiguousarray(w_bf16_bits, np.uint16)
        _lib.check(lib.b200_llama_set_norm(self._h, layer, which, t.ctypes.data))

    def finalize(self):
        _lib.check(lib.b200_llama_finalize(self._h))

    def random_init(self, mode: int, seed: int = 1):
        _lib.check(lib.b200_llama_random_init(self._h, mode, seed))

    def step(self, kv: PagedKVCache, descs: Sequence[Sequence[int]], prefill_tokens: Sequence[int] = ()):
        """b200_llama_step with host buffers.  Returns (next token per request, free pages)."""
        n = len(descs)
        d = (PackDesc * max(n, 1))()
        for i, (slot, count, base, src) in enumerate(descs):
            d[i].seq_slot, d[i].count, d[i].base_pos, d[i].src_offset = slot, count, base, src
        pt = (C.c_uint32 * max(len(prefill_tokens), 1))(*[int(t) for t in prefill_tokens])
        out = (C.c_uint32 * max(n, 1))()
        free = C.c_int32()
        _lib.check(lib.b200_llama_step(self._h, kv._h, d, n, pt, len(prefill_tokens), out, C.byref(free), _stream()))
        return np.array([out[i] for i in range(n)], np.uint32), free.value

    def forward_device(self, kv: PagedKVCache, d_desc: torch.Tensor, total_rows: int,
                       d_prefill: Optional[torch.Tensor] = None):
        """b200_llama_forward on device-resident descriptors (asynchronous)."""
        _lib.check(lib.b200_llama_forward(self._h, kv._h, _ptr(d_desc), d_desc.shape[0], total_rows, _ptr(d_prefill),
                                          _stream()))

    def set_samplers(self, rows):
        """Sampler rows (temperature, top_k, top_p, uniform) for the requests of the next step()."""
        arr = sample_params_array(rows)
        _lib.check(lib.b200_llama_set_samplers(self._h, arr.ctypes.data_as(C.POINTER(_lib.SampleParams)), len(rows)))

    def last_logprobs(self, n_req: int) -> np.ndarray:
        out = np.zeros(n_req, np.float32)
        _lib.check(lib.b200_llama_last_logprobs(self._h, out.ctypes.data_as(C.POINTER(C.c_float)), n_req))
        return out

    def last_logits(self, n_req: int) -> np.ndarray:
        out = np.zeros((n_req, self.cfg.vocab), np.uint16)
        _lib.check(lib.b200_llama_last_logits(self._h, out.ctypes.data, n_req))
        return (out.astype(np.uint32) << 16).view(np.float32)

    def launch_count(self) -> int:
        return int(lib.b200_llama_launch_count(self._h))

    def enable_graphs(self, on: bool = True):
        lib.b200_llama_enable_graphs(self._h, int(on))

    def set_fused_qkv_rope(self, on: bool = True):
        lib.b200_llama_set_fused_qkv_rope(self._h, int(on))

    def profile_enable(self, on: bool = True):
        lib.b200_llama_profile_enable(self._h, int(on))

    def profile_collect(self):
        """{category: (milliseconds, calls)} for attention / matmul / rope+append / other."""
        ms, calls = (C.c_double * 4)(), (C.c_int64 * 4)()
        _lib.check(lib.b200_llama_profile_collect(self._h, ms, calls))
        names = ("attention", "matmul", "rope_append", "other")
        return {n: (ms[i], calls[i]) for i, n in enumerate(names)}


# ---------------------------------------------------------------------------------------------
# mixture of experts
# ---------------------------------------------------------------------------------------------
SCORE_SOFTMAX, SCORE_SIGMOID, SCORE_SQRTSOFTPLUS = 0, 1, 2


def moe_route(logits: torch.Tensor, k: int, bias: Optional[torch.Tensor] = None, scoring: int = SCORE_SOFTMAX,
              route_scale: float = 1.0):
    """b200_moe_route.  logits [N,E] bf16 or f32 -> (indices i32 [N,k], weights f32 [N,k], counts i32 [E])."""
    n, e = logits.shape
    idx = torch.empty((n, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((n, k), dtype=torch.float32, device=logits.device)
    counts = torch.empty(e, dtype=torch.int32, device=logits.device)
    _lib.check(lib.b200_moe_route(_ptr(logits), int(logits.dtype == torch.float32), _ptr(bias), n, e, k, scoring,
                                  route_scale, _ptr(idx), _ptr(w), _ptr(counts), _stream()))
    return idx, w, counts


def moe_group(indices: torch.Tensor, counts: torch.Tensor, tile_rows: int = 128):
    """b200_moe_group -> (offsets [E+1], order [N*k], inv_order [N*k], items [cap,4], n_items [1])."""
    n, k = indices.shape
    e = counts.shape[0]
    dev_ = indices.device
    offsets = torch.empty(e + 1, dtype=torch.int32, device=dev_)
    order = torch.empty(n * k, dtype=torch.int32, device=dev_)
    inv = torch.empty(n * k, dtype=torch.int32, device=dev_)
    cap = e + (n * k + tile_rows - 1) // tile_rows
    items = torch.zeros((cap, 4), dtype=torch.int32, device=dev_)
    n_items = torch.zeros(1, dtype=torch.int32, device=dev_)
    _lib.check(lib.b200_moe_group(_ptr(indices), _ptr(counts), n, k, e, tile_rows, _ptr(offsets), _ptr(order), _ptr(inv),
                                  _ptr(items), _ptr(n_items), _stream()))
    return offsets, order, inv, items, n_items


class MoELayer:
    """DSV4MoE.forward (src/models/deepseek_v4.zig:1010-1056) on borrowed weight handles."""

    def __init__(self, hidden: int, n_experts: int, inter: int, top_k: int, gate: QWeight, experts_gate_up: QWeight,
                 experts_down: QWeight, shared_gate_up: Optional[QWeight] = None, shared_down: Optional[QWeight] = None,
                 bias: Optional[np.ndarray] = None, scoring: int = SCORE_SOFTMAX, route_scale: float = 1.0,
                 swiglu_limit: float = 10.0, shared_swiglu_limit: float = 0.0, tile_rows: int = 112,
                 max_tokens: int = 4096):
        self.cfg = _lib.MoeConfig(hidden, n_experts, inter, top_k, scoring, tile_rows, max_tokens, route_scale,
                                  swiglu_limit, shared_swiglu_limit)
        self._keep = (gate, experts_gate_up, experts_down, shared_gate_up, shared_down)
        b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
        h = C.c_void_p()
        _lib.check(lib.b200_moe_create(C.byref(self.cfg), gate._h,
                                       b.ctypes.data_as(C.POINTER(C.c_float)) if b is not None else None,
                                       experts_gate_up._h, experts_down._h,
                                       shared_gate_up._h if shared_gate_up else None,
                                       shared_down._h if shared_down else None, C.byref(h)))
        self._h = h.value

    def close(self):
        if getattr(self, "_h", None):
            lib.b200_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = out if out is not None else torch.empty_like(x)
        _lib.check(lib.b200_moe_forward(self._h, _ptr(x), x.shape[0], _ptr(out), _stream()))
        return out

    def last_routing(self, n_tokens: int):
        k, e = self.cfg.top_k, self.cfg.n_experts
        idx = np.zeros((n_tokens, k), np.uint32)
        w = np.zeros((n_tokens, k), np.float32)
        off = np.zeros(e + 1, np.int32)
        _lib.check(lib.b200_moe_last_routing(self._h, n_tokens, idx.ctypes.data, w.ctypes.data, off.ctypes.data))
        return idx, w, off


def moe_gather(x: torch.Tensor, order: torch.Tensor, weights: torch.Tensor, k: int):
    """b200_moe_gather -> (x_sorted [N*k, D] bf16, row_scales [N*k] f32)."""
    a, d = order.shape[0], x.shape[1]
    xs = torch.empty((a, d), dtype=torch.bfloat16, device=x.device)
    rs = torch.empty(a, dtype=torch.float32, device=x.device)
    _lib.check(lib.b200_moe_gather(_ptr(x), _ptr(order), _ptr(weights), a, k, d, _ptr(xs), _ptr(rs), _stream()))
    return xs, rs


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """b200_moe_gather_rows: dst[r] = src[idx[r]] (bf16 rows)."""
    out = torch.empty((idx.shape[0], src.shape[1]), dtype=torch.bfloat16, device=src.device)
    _lib.check(lib.b200_moe_gather_rows(_ptr(src), _ptr(idx), _ptr(out), idx.shape[0], src.shape[1], _stream()))
    return out


def moe_grouped_qmm(w: QWeight, x_sorted: torch.Tensor, items: torch.Tensor, n_items: torch.Tensor, tile_rows: int,
                    epilogue: int = EPI_NONE, row_scales: Optional[torch.Tensor] = None, swiglu_limit: float = 0.0):
    """b200_moe_grouped_qmm over work items {expert, first row, rows, 0}."""
    rows = x_sorted.shape[0]
    n_out = w.n // 2 if epilogue == EPI_SWIGLU else w.n
    out = torch.empty((rows, n_out), dtype=torch.bfloat16, device=x_sorted.device)
    _lib.check(lib.b200_moe_grouped_qmm(w._h, _ptr(x_sorted), rows, _ptr(out), epilogue, _ptr(row_scales), swiglu_limit,
                                        _ptr(items), _ptr(n_items), items.shape[0], tile_rows, _stream()))
    return out


def moe_combine(y_sorted: torch.Tensor, inv_order: torch.Tensor, n_tokens: int, k: int,
                shared_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    out = torch.empty((n_tokens, y_sorted.shape[1]), dtype=torch.bfloat16, device=y_sorted.device)
    _lib.check(lib.b200_moe_combine(_ptr(y_sorted), _ptr(inv_order), n_tokens, k, y_sorted.shape[1], _ptr(shared_out),
                                    _ptr(out), _stream()))
    return out


class Engine:
    """b200_engine_*: scheduler + device page pool + model step in one loop."""

    def __init__(self, model: LlamaModel, kv: PagedKVCache, max_prefill_tokens: int = 512):
        self._h = lib.b200_engine_create(model._h, kv._h, max_prefill_tokens)
        if not self._h:
            raise _lib.B200Error(_lib.ERR_CUDA)
        self._keep = (model, kv)

    def close(self):
        if getattr(self, "_h", None):
            lib.b200_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def submit(self, rid: int, prompt: Sequence[int], max_tokens: int, stop_tokens: Sequence[int] = ()):
        p = (C.c_uint32 * max(len(prompt), 1))(*[int(t) for t in prompt])
        s = (C.c_uint32 * max(len(stop_tokens), 1))(*[int(t) for t in stop_tokens])
        _lib.check(lib.b200_engine_submit(self._h, rid, p, len(prompt), max_tokens, s, len(stop_tokens)))

    def step(self, cap: int = 4096):
        out = (_lib.TokenOutput * cap)()
        n = C.c_uint64()
        _lib.check(lib.b200_engine_step(self._h, out, cap, C.byref(n), _stream()))
        return [(int(out[i].request_id), int(out[i].token)) for i in range(n.value)]

    def active_count(self) -> int:
        return int(lib.b200_engine_active_count(self._h))

    def result(self, rid: int, cap: int = 8192):
        out = (C.c_uint32 * cap)()
        n, done = C.c_uint64(), C.c_int32()
        _lib.check(lib.b200_engine_result(self._h, rid, out, cap, C.byref(n), C.byref(done)))
        return [int(out[i]) for i in range(min(n.value, cap))], bool(done.value)

    def free_pages(self) -> int:
        return int(lib.b200_engine_free_pages(self._h))

    def set_sampler(self, rid: int, temperature: float, top_k: int = 50, top_p: float = 1.0, seed: int = 0):
        _lib.check(lib.b200_engine_set_sampler(self._h, rid, temperature, top_k, top_p, seed))

    def park_slot(self) -> int:
        out = C.c_int32()
        _lib.check(lib.b200_engine_park_slot(self._h, C.byref(out)))
        return out.value

    def publish_prefix(self, slot: int, token_ids: Sequence[int]):
        arr = (C.c_uint32 * max(len(token_ids), 1))(*[int(t) for t in token_ids])
        _lib.check(lib.b200_engine_publish_prefix(self._h, slot, arr, len(token_ids)))

    def drop_prefix(self, slot: int):
        _lib.check(lib.b200_engine_drop_prefix(self._h, slot))

    def request_slot(self, rid: int) -> int:
        return int(lib.b200_engine_request_slot(self._h, rid))

    def set_prefix_sharing(self, on: bool = True):
        lib.b200_engine_set_prefix_sharing(self._h, int(on))

    def set_max_step_tokens(self, n: int):
        lib.b200_engine_set_max_step_tokens(self._h, int(n))

    def shared_tokens(self, rid: int) -> int:
        return int(lib.b200_engine_shared_tokens(self._h, rid))

    def cancel(self, rid: int):
        _lib.check(lib.b200_engine_cancel(self._h, rid))

    def request_status(self, rid: int) -> int:
        out = C.c_int32()
        _lib.check(lib.b200_engine_request_status(self._h, rid, C.byref(out)))
        return out.value

    def pressure_stats(self):
        """(deferred request-steps, preemptions, requests failed on their own)."""
        d, p, f = C.c_uint64(), C.c_uint64(), C.c_uint64()
        lib.b200_engine_pressure_stats(self._h, C.byref(d), C.byref(p), C.byref(f))
        return int(d.value), int(p.value), int(f.value)

    def forget(self, rid: int):
        lib.b200_engine_forget(self._h, rid)

    def last_batch(self, cap: int = 4096):
        """Request ids of the last step's batch, in the row order of the model's last logits."""
        ids = (C.c_uint64 * cap)()
        n = int(lib.b200_engine_last_batch(self._h, ids, cap))
        return [int(ids[i]) for i in range(min(n, cap))]
