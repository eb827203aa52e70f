"""The allocation-free matmul entry point (b200_qmm_static_scratch) against the regular one.

Some embedders of this library may not allocate device memory once serving has started — the page
pool owns the rest of HBM, or the step is being recorded into a CUDA graph where cudaMalloc is not
allowed.  For them the split-K scratch is a fixed array inside the library.  This file is collected
last on purpose: if it fails, a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import ref_math

pytestmark = pytest.mark.gpu


def _bits(a):
    return (ref_math.bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def _static(dev, lib, w, x, epilogue=0, residual=None, limit=0.0):
    n_out = w.n // 2 if epilogue == dev.EPI_SWIGLU else w.n
    out = torch.empty((x.shape[0], n_out), dtype=torch.bfloat16, device="cuda")
    st = lib.lib.b200_qmm_static_scratch(w._h, x.data_ptr(), x.shape[0], out.data_ptr(), epilogue,
                                         residual.data_ptr() if residual is not None else None, limit,
                                         torch.cuda.current_stream().cuda_stream)
    return st, out


def test_static_scratch_matches_regular_entry_point_and_oracle_twice():
    from dmlx_b200 import _lib as lib
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(2024)
    n, k = 768, 2048
    wf = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    packed, s, b = ref_math.quantize_affine4(wf)
    w = dev.QWeight(dev.Q_AFFINE4_G64, packed, _bits(s), _bits(b), n, k)
    wd = ref_math.dequantize_affine4(packed, s, b)
    # calls in a row with different shapes and epilogues: a later one must not see an earlier one's
    # leftovers.  24 and 5 rows write their output from the kernel; 200 rows (one token tile of 208)
    # and 300 rows (two tiles of 256) go through the K split, the array and the finish pass.
    cases = ((24, dev.EPI_NONE), (5, dev.EPI_SWIGLU), (200, dev.EPI_RESIDUAL), (300, dev.EPI_NONE), (24, dev.EPI_NONE))
    for rows, epi in cases:
        xf = ref_math.bf16_round(rng.normal(0, 1, (rows, k)))
        x = torch.tensor(xf, device="cuda").bfloat16()
        resf = ref_math.bf16_round(rng.normal(0, 1, (rows, n))) if epi == dev.EPI_RESIDUAL else None
        res = torch.tensor(resf, device="cuda").bfloat16() if resf is not None else None
        regular = dev.qmm(w, x, epi, residual=res, path=dev.QMM_TCGEN05)
        st, got = _static(dev, lib, w, x, epi, residual=res)
        assert st == 0, lib.lib.b200_last_error()
        torch.cuda.synchronize()
        assert dev.qmm_error_word() == 0  # reads the word of this entry point's kernels too
        y = ref_math.qmm(xf, wd)
        if epi == dev.EPI_RESIDUAL:
            y = y + resf
        elif epi == dev.EPI_SWIGLU:
            g_, u_ = y[:, 0::2], y[:, 1::2]
            y = g_ / (1.0 + np.exp(-g_)) * u_
        g, r = got.float().cpu().numpy(), regular.float().cpu().numpy()
        # the tolerance of the matmul tests, against the other entry point and against the CPU oracle
        assert np.abs(g - r).max() <= 2e-2 * np.abs(r).max(), (rows, epi)
        assert np.abs(g - y).max() <= 2e-2 * np.abs(y).max(), (rows, epi)


def test_static_scratch_error_word_is_read_and_cleared():
    """A bounded wait that runs out inside this entry point's kernels is reported through
    b200_qmm_error_word like any other matmul's: write the word by hand (no kernel is made to time
    out) and check that the reader sees and clears it."""
    from dmlx_b200 import _lib as lib
    from dmlx_b200 import device as dev

    w = dev.QWeight.random(dev.Q_AFFINE4_G64, 256, 256, seed=5)
    x = torch.zeros((8, 256), dtype=torch.bfloat16, device="cuda")
    st, _ = _static(dev, lib, w, x)   # first use on this device resolves the word's address
    assert st == 0
    torch.cuda.synchronize()
    assert dev.qmm_error_word() == 0
    lib.check(lib.lib.b200_qmm_debug_set_error_word(lib.ERR_DEVICE_FLAGGED, 1))
    assert dev.qmm_error_word() == lib.ERR_DEVICE_FLAGGED
    assert dev.qmm_error_word() == 0


def test_static_scratch_rejects_oversized_problems():
    from dmlx_b200 import _lib as lib
    from dmlx_b200 import device as dev

    h = C.c_void_p()
    lib.check(lib.lib.b200_qweight_random(dev.Q_AFFINE4_G64, 1, 128 * 512, 256, 1, C.byref(h)))
    w = dev.QWeight.__new__(dev.QWeight)
    w._h, w.mode, w.n, w.k, w.n_experts = h.value, dev.Q_AFFINE4_G64, 128 * 512, 256, 1
    x = torch.zeros((256, 256), dtype=torch.bfloat16, device="cuda")  # 256 x 65536 x 4 B = 64 MiB of scratch
    st, _ = _static(dev, lib, w, x)
    assert st == lib.ERR_CAPACITY
    assert b"built-in array" in lib.lib.b200_last_error()
    # rows are charged by whole token tiles: 120 rows (one tile of 128) fit the 32 MiB array exactly,
    # 257 rows count as two tiles of 256
    st, _ = _static(dev, lib, w, x[:120])
    assert st == 0, lib.lib.b200_last_error()
    torch.cuda.synchronize()
    x2 = torch.zeros((257, 256), dtype=torch.bfloat16, device="cuda")
    st, _ = _static(dev, lib, w, x2)
    assert st == lib.ERR_CAPACITY
