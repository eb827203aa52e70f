"""ctypes binding of libdmlx_b200.so — the same C header a Zig host binds with @cImport.

The library is the product: importing this module fails loudly when it has not been built
(`python -m dmlx_b200.build`); there is no Python or CPU fallback behind it.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdmlx_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m dmlx_b200.build` "
        "(there is no fallback implementation)"
    )

lib = C.CDLL(LIB_PATH)

u64, u32, i32, f32 = C.c_uint64, C.c_uint32, C.c_int32, C.c_float
vp = C.c_void_p
P = C.POINTER


class PackDesc(C.Structure):
    _fields_ = [("seq_slot", i32), ("count", i32), ("base_pos", i32), ("src_offset", i32)]


class TokenOutput(C.Structure):
    _fields_ = [("request_id", u64), ("token", u32), ("_pad", u32)]


class SampleParams(C.Structure):
    _fields_ = [("temperature", f32), ("top_p", f32), ("repetition_penalty", f32), ("uniform", f32), ("top_k", i32),
                ("_pad", i32)]


class KvConfig(C.Structure):
    _fields_ = [(n, i32) for n in (
        "n_layers", "n_kv_heads", "head_dim", "page_size", "n_pages", "max_seqs", "max_pages_per_seq",
        "kv_dtype", "max_rows", "n_q_heads", "attn_scratch_chunks")]


# status codes (include/dmlx_b200.h)
OK = 0
ERR_INSUFFICIENT_BLOCKS = 1
ERR_INVALID_BLOCK_ID = 2
ERR_PAGE_POOL_EXHAUSTED = 3
ERR_INVALID_QUANT_BITS = 4
ERR_INVALID_BATCH_INDEX = 5
ERR_INVALID_ARGUMENT = 6
ERR_CUDA = 7
ERR_NO_DEVICE = 8
ERR_UNSUPPORTED = 9
ERR_CAPACITY = 10
ERR_DEVICE_FLAGGED = 11
ERR_CANCELLED = 12


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


_sig("b200_status_name", C.c_char_p, i32)
_sig("b200_last_error", C.c_char_p)
_sig("b200_version", i32)
_sig("b200_device_available", i32)

# block manager
_sig("b200_bm_create", vp, u64)
_sig("b200_bm_destroy", None, vp)
_sig("b200_bm_can_allocate", i32, vp, u64)
_sig("b200_bm_allocate_blocks", i32, vp, u64, u64, P(u64))
_sig("b200_bm_free_blocks", None, vp, u64)
_sig("b200_bm_copy_on_write", i32, vp, u64, P(u64))
_sig("b200_bm_free_count", u64, vp)
_sig("b200_bm_used_count", u64, vp)
_sig("b200_bm_total_blocks", u64, vp)
_sig("b200_hash_block", u64, u64, P(u32), u64)
_sig("b200_bm_find_cached_prefix", i32, vp, P(u32), u64, u64, P(u64), u64, P(u64))
_sig("b200_bm_register_block_hash", i32, vp, u64, u64)
_sig("b200_bm_get_ref", u64, vp, u64)
_sig("b200_bm_set_ref", None, vp, u64, u64)
_sig("b200_bm_is_used", i32, vp, u64)
_sig("b200_bm_get_tokens_used", u64, vp, u64)
_sig("b200_bm_set_tokens_used", None, vp, u64, u64)
_sig("b200_bm_share", None, vp, u64, u64)
_sig("b200_bm_blocks_of", u64, vp, u64, P(u64), u64)

# request
_sig("b200_request_create", vp, u64, P(u32), u64, u64, P(u32), u64)
_sig("b200_request_destroy", None, vp)
_sig("b200_request_id", u64, vp)
_sig("b200_request_state", i32, vp)
_sig("b200_request_prefill_offset", u64, vp)
_sig("b200_request_prompt_len", u64, vp)
_sig("b200_request_seq_len", u64, vp)
_sig("b200_request_is_stop_token", i32, vp, u32)
_sig("b200_request_has_pending_prefill", i32, vp)
_sig("b200_request_current_prefill_chunk_len", u64, vp, u64)
_sig("b200_request_generated", u64, vp, P(u32), u64)
_sig("b200_request_block_ids", u64, vp, P(u64), u64)
_sig("b200_request_force_state", None, vp, i32, u64, P(u32), u64)
_sig("b200_request_kv_slot", i32, vp)

# scheduler-side block manager + scheduler
_sig("b200_sched_bm_create", vp, u64)
_sig("b200_sched_bm_create_with_real", vp, vp)
_sig("b200_sched_bm_create_with_kv", vp, vp)
_sig("b200_sched_bm_destroy", None, vp)
_sig("b200_sched_bm_can_allocate", i32, vp, u64)
_sig("b200_sched_bm_free_count", u64, vp)
_sig("b200_sched_bm_total_blocks", u64, vp)
_sig("b200_sched_bm_used_blocks", u64, vp)
_sig("b200_scheduler_create", vp, vp, u64)
_sig("b200_scheduler_destroy", None, vp)
_sig("b200_scheduler_add_request", i32, vp, vp)
_sig("b200_scheduler_schedule", i32, vp, P(vp), P(u64), P(vp), P(u64), u64, P(u64))
_sig("b200_scheduler_postprocess", i32, vp, P(TokenOutput), u64)
_sig("b200_scheduler_active_count", u64, vp)
_sig("b200_scheduler_waiting_count", u64, vp)
_sig("b200_scheduler_running_count", u64, vp)

# batch builder
_sig("b200_batch_build", i32, P(vp), u64, P(vp), u64, i32, u64, P(u32), P(i32), P(i32), u64, P(i32), P(u64), P(u64))
_sig("b200_is_attending", i32, P(i32), u64, u64, u64)
_sig("b200_batch_mask", i32, P(i32), u64, P(f32), u64)
_sig("b200_greedy_host", u32, P(f32), u64)

# device layer
_sig("b200_pack_batch", i32, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp)
_sig("b200_kv_create", i32, P(KvConfig), P(vp))
_sig("b200_kv_destroy", None, vp)
_sig("b200_kv_dims", i32, vp, P(i32), P(i32))
_sig("b200_kv_reset", i32, vp)
_sig("b200_kv_set_free_order", i32, vp, P(i32), i32)
_sig("b200_kv_free_count", i32, vp, P(i32))
_sig("b200_kv_alloc", i32, vp, i32, i32, P(i32))
_sig("b200_kv_release", i32, vp, P(i32), i32)
_sig("b200_kv_fork", i32, vp, i32, i32, i32)
_sig("b200_kv_extend", i32, vp, i32, vp, i32)
_sig("b200_kv_rollback", i32, vp, i32, i32)
_sig("b200_kv_filter", i32, vp, P(i32), i32)
_sig("b200_kv_reserve", i32, vp, vp, i32, vp)
_sig("b200_kv_append", i32, vp, i32, vp, vp, i32, vp)
_sig("b200_kv_rope_append", i32, vp, i32, vp, vp, vp, vp, vp, i32, i32, f32, vp)
_sig("b200_kv_seq_len", i32, vp, i32, P(i32))
_sig("b200_kv_current_len", i32, vp, P(i32))
_sig("b200_kv_block_table", i32, vp, i32, P(i32), i32, P(i32))
_sig("b200_kv_ref_counts", i32, vp, P(i32), i32)
_sig("b200_kv_error_word", i32, vp, P(i32))
_sig("b200_kv_gather", i32, vp, i32, i32, vp, vp, i32, vp)
_sig("b200_kv_page_raw", i32, vp, i32, i32, vp, vp, P(f32), P(f32))
_sig("b200_kv_page_load", i32, vp, i32, i32, vp, vp, P(f32), P(f32))
_sig("b200_kv_set_len", i32, vp, i32, i32)
_sig("b200_paged_attn_decode", i32, vp, i32, vp, vp, vp, i32, vp, vp)
_sig("b200_paged_attn_prefill", i32, vp, i32, vp, vp, vp, i32, vp, vp)
_sig("b200_set_attn_pages_per_chunk", None, i32)
_sig("b200_set_attn_prefill_direct", None, i32)
_sig("b200_set_attn_path", None, i32)
_sig("b200_rmsnorm", i32, vp, vp, vp, i32, i32, f32, vp)
_sig("b200_rope", i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp)
_sig("b200_embed_gather", i32, vp, vp, vp, i32, i32, vp)
_sig("b200_argmax", i32, vp, i32, i32, vp, vp)
_sig("b200_sample_rows", i32, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp)
_sig("b200_prng_seed", None, u64, P(u64))
_sig("b200_prng_next_u64", u64, P(u64))
_sig("b200_prng_next_f32", f32, P(u64))
_sig("b200_qweight_create", i32, i32, i32, i32, i32, vp, vp, vp, P(vp))
_sig("b200_qweight_random", i32, i32, i32, i32, i32, u32, P(vp))
_sig("b200_qweight_destroy", None, vp)
_sig("b200_qweight_export", i32, vp, i32, vp, vp, vp)
_sig("b200_qmm", i32, vp, vp, i32, vp, i32, vp, f32, i32, vp)
_sig("b200_qmm_residual_norm", i32, vp, vp, i32, vp, vp, vp, f32, vp, vp)


class LlamaConfig(C.Structure):
    _fields_ = [(n, i32) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "max_rows",
                                   "max_reqs", "max_seqs")] + [("rms_eps", f32), ("rope_theta", f32)]


_sig("b200_qmm_error_word", i32, P(i32))
_sig("b200_qmm_static_scratch", i32, vp, vp, i32, vp, i32, vp, f32, vp)
_sig("b200_llama_create", i32, P(LlamaConfig), P(vp))
_sig("b200_llama_destroy", None, vp)
_sig("b200_llama_set_linear", i32, vp, i32, i32, i32, vp, vp, vp)
_sig("b200_llama_set_embedding", i32, vp, vp)
_sig("b200_llama_set_norm", i32, vp, i32, i32, vp)
_sig("b200_llama_finalize", i32, vp)
_sig("b200_llama_random_init", i32, vp, i32, u32)
_sig("b200_llama_step", i32, vp, vp, vp, i32, vp, i32, vp, P(i32), vp)
_sig("b200_llama_forward", i32, vp, vp, vp, i32, i32, vp, vp)
_sig("b200_llama_device_buffers", None, vp, P(vp), P(vp), P(vp))
_sig("b200_llama_last_logits", i32, vp, vp, i32)
_sig("b200_llama_set_samplers", i32, vp, P(SampleParams), i32)
_sig("b200_llama_last_logprobs", i32, vp, P(f32), i32)
_sig("b200_llama_launch_count", C.c_int64, vp)
_sig("b200_launch_count", C.c_int64)
_sig("b200_set_qmm_grouped_tmem_a", None, i32)
_sig("b200_set_qmm_grouped_block_scaled", None, i32)
_sig("b200_set_qmm_mx_persistent", None, i32)
_sig("b200_llama_profile_enable", None, vp, i32)
_sig("b200_llama_enable_graphs", None, vp, i32)
_sig("b200_llama_profile_collect", i32, vp, P(C.c_double), P(C.c_int64))


class QmmPartials(C.Structure):
    _fields_ = [("d_ws", vp)] + [(n, i32) for n in ("splits", "tn", "tts", "nt", "rows", "n", "pending")]


_sig("b200_qmm_deferred", i32, vp, vp, i32, vp, i32, vp, P(QmmPartials))
_sig("b200_kv_rope_append_partials", i32, vp, i32, P(QmmPartials), vp, i32, vp, vp, i32, i32, f32, vp)
_sig("b200_llama_set_fused_qkv_rope", None, vp, i32)


class MoeConfig(C.Structure):
    _fields_ = [(n, i32) for n in ("hidden", "n_experts", "inter", "top_k", "scoring", "tile_rows", "max_tokens")] + \
               [("route_scale", f32), ("swiglu_limit", f32), ("shared_swiglu_limit", f32), ("ep_rank", i32), ("ep_world", i32)]


EP_UNIQUE_ID_BYTES = 128


class EpWatchOps(C.Structure):
    _fields_ = [("done", C.CFUNCTYPE(C.c_int, vp)), ("async_error", C.CFUNCTYPE(C.c_int, vp)), ("abort", C.CFUNCTYPE(None, vp)),
                ("ctx", vp)]


_sig("b200_moe_route", i32, vp, i32, vp, i32, i32, i32, i32, f32, vp, vp, vp, vp)
_sig("b200_moe_group", i32, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp)
_sig("b200_moe_gather", i32, vp, vp, vp, i32, i32, i32, vp, vp, vp)
_sig("b200_moe_grouped_qmm", i32, vp, vp, i32, vp, i32, vp, f32, vp, vp, i32, i32, vp)
_sig("b200_moe_gather_rows", i32, vp, vp, vp, i32, i32, vp)
_sig("b200_moe_combine", i32, vp, vp, i32, i32, i32, vp, vp, vp)
_sig("b200_moe_create", i32, P(MoeConfig), vp, P(f32), vp, vp, vp, vp, P(vp))
_sig("b200_moe_destroy", None, vp)
_sig("b200_moe_forward", i32, vp, vp, i32, vp, vp)
_sig("b200_moe_last_routing", i32, vp, i32, vp, vp, vp)
_sig("b200_ep_unique_id", i32, P(C.c_uint8))
_sig("b200_ep_create", i32, i32, i32, P(C.c_uint8), P(vp))
_sig("b200_ep_destroy", None, vp)
_sig("b200_ep_rank", i32, vp)
_sig("b200_ep_world", i32, vp)
_sig("b200_ep_nccl_version", i32)
_sig("b200_ep_dispatch", i32, vp, vp, vp, i32, i32, vp)
_sig("b200_ep_plan", i32, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp)
_sig("b200_ep_combine", i32, vp, vp, vp, i32, i32, vp)
_sig("b200_moe_forward_ep", i32, vp, vp, vp, i32, vp, vp)
_sig("b200_ep_wait", i32, vp, vp, i32)
_sig("b200_ep_abort", i32, vp)
_sig("b200_ep_watch", i32, P(EpWatchOps), i32, i32)


_sig("b200_request_prompt", u64, vp, P(u32), u64)
_sig("b200_engine_create", vp, vp, vp, u64)
_sig("b200_engine_destroy", None, vp)
_sig("b200_engine_submit", i32, vp, u64, P(u32), u64, u64, P(u32), u64)
_sig("b200_engine_step", i32, vp, P(TokenOutput), u64, P(u64), vp)
_sig("b200_engine_active_count", u64, vp)
_sig("b200_engine_result", i32, vp, u64, P(u32), u64, P(u64), P(i32))
_sig("b200_engine_forget", None, vp, u64)
_sig("b200_engine_free_pages", i32, vp)
_sig("b200_engine_set_prefix_sharing", None, vp, i32)
_sig("b200_engine_park_slot", i32, vp, P(i32))
_sig("b200_engine_publish_prefix", i32, vp, i32, P(u32), u64)
_sig("b200_engine_drop_prefix", i32, vp, i32)
_sig("b200_engine_request_slot", i32, vp, u64)
_sig("b200_sched_bm_park_slot", i32, vp, P(i32))
_sig("b200_sched_bm_unpark_slot", i32, vp, i32)
_sig("b200_sched_bm_sync", i32, vp)
_sig("b200_engine_set_sampler", i32, vp, u64, f32, i32, f32, u64)
_sig("b200_engine_set_max_step_tokens", None, vp, u64)
_sig("b200_engine_shared_tokens", u64, vp, u64)
_sig("b200_engine_last_batch", u64, vp, P(u64), u64)
_sig("b200_engine_cancel", i32, vp, u64)
_sig("b200_engine_request_status", i32, vp, u64, P(i32))
_sig("b200_engine_pressure_stats", None, vp, P(u64), P(u64), P(u64))
_sig("b200_request_error", i32, vp)
_sig("b200_sched_bm_note_free", None, vp, u64)
_sig("b200_scheduler_remove", i32, vp, vp, i32)
_sig("b200_scheduler_preempt", i32, vp, vp)
_sig("b200_scheduler_hold_admission", None, vp, i32)
_sig("b200_scheduler_set_admission_budget", None, vp, u64)
_sig("b200_scheduler_running", u64, vp, P(vp), u64)
_sig("b200_kv_limits", i32, vp, P(i32), P(i32))
_sig("b200_qmm_debug_set_error_word", i32, i32, i32)
_sig("b200_qmm_debug_wait_runs_out", i32, i32, vp)


class B200Error(RuntimeError):
    def __init__(self, status: int):
        self.status = status
        name = lib.b200_status_name(status).decode()
        msg = lib.b200_last_error().decode()
        super().__init__(f"{name}: {msg}")


class InsufficientBlocks(B200Error):
    pass


class InvalidBlockId(B200Error):
    pass


class InvalidBatchIndex(B200Error):
    pass


_ERR_CLASS = {ERR_INSUFFICIENT_BLOCKS: InsufficientBlocks, ERR_INVALID_BLOCK_ID: InvalidBlockId,
              ERR_INVALID_BATCH_INDEX: InvalidBatchIndex}


def check(status: int) -> None:
    if status != OK:
        raise _ERR_CLASS.get(status, B200Error)(status)
