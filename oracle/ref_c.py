"""ctypes access to the C twin of the oracle (oracle/ref_kernels.c).  TEST / BENCH INFRASTRUCTURE."""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB if os.path.exists(_build.LIB) else _build.build()
        _lib = C.CDLL(path)
        _lib.ref_paged_attention_decode.restype = C.c_int
        _lib.ref_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return int(lib().ref_num_threads())


def use_all_cores() -> int:
    """Run the C twin on every core this process may use, whatever OMP_NUM_THREADS says."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().ref_set_threads(C.c_int(n))
    return num_threads()


def paged_attention_decode(k_pool_bf16: np.ndarray, v_pool_bf16: np.ndarray, block_table: np.ndarray, ctx: np.ndarray,
                           hq: int, hkv: int, d: int, q: np.ndarray) -> np.ndarray:
    """k/v pool: uint16 [pages, hkv, 32, d]; block_table int32 [n_seq, max_pages]; q f32 [n_seq, hq, d]."""
    n_seq = len(ctx)
    out = np.zeros((n_seq, hq, d), np.float32)
    bt = np.ascontiguousarray(block_table, np.int32)
    cx = np.ascontiguousarray(ctx, np.int32)
    qq = np.ascontiguousarray(q, np.float32)
    rc = lib().ref_paged_attention_decode(_p(k_pool_bf16), _p(v_pool_bf16), _p(bt), C.c_int32(bt.shape[1]), _p(cx),
                                          C.c_int32(n_seq), C.c_int32(hq), C.c_int32(hkv), C.c_int32(d), _p(qq), _p(out))
    if rc != 0:
        raise MemoryError("ref_paged_attention_decode")
    return out


def qmm_affine4(packed: np.ndarray, scales: np.ndarray, biases: np.ndarray, x: np.ndarray) -> np.ndarray:
    n, k = packed.shape[0], packed.shape[1] * 8
    xx = np.ascontiguousarray(x, np.float32)
    y = np.zeros((xx.shape[0], n), np.float32)
    lib().ref_qmm_affine4(_p(np.ascontiguousarray(packed, np.uint32)), _p(np.ascontiguousarray(scales, np.float32)),
                          _p(np.ascontiguousarray(biases, np.float32)), C.c_int32(n), C.c_int32(k), _p(xx),
                          C.c_int32(xx.shape[0]), _p(y))
    return y


def qmm_mxfp4(packed: np.ndarray, scales: np.ndarray, x: np.ndarray) -> np.ndarray:
    n, k = packed.shape[0], packed.shape[1] * 2
    xx = np.ascontiguousarray(x, np.float32)
    y = np.zeros((xx.shape[0], n), np.float32)
    lib().ref_qmm_mxfp4(_p(np.ascontiguousarray(packed, np.uint8)), _p(np.ascontiguousarray(scales, np.uint8)),
                        C.c_int32(n), C.c_int32(k), _p(xx), C.c_int32(xx.shape[0]), _p(y))
    return y
