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


def test_static_scratch_matches_regular_entry_point_twice():
    from dmlx_b200 import _lib as lib
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(2024)
    n, k = 768, 2048
    wf = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    packed, s, b = ref_math.quantize_affine4(wf)
    w = dev.QWeight(dev.Q_AFFINE4_G64, packed, _bits(s), _bits(b), n, k)
    # two calls in a row with different shapes and epilogues: the second must not see the first's leftovers
    for rows, epi in ((24, dev.EPI_NONE), (5, dev.EPI_SWIGLU)):
        x = torch.tensor(ref_math.bf16_round(rng.normal(0, 1, (rows, k))), device="cuda").bfloat16()
        want = dev.qmm(w, x, epi, path=dev.QMM_TCGEN05)
        st, got = _static(dev, lib, w, x, epi)
        assert st == 0, lib.lib.b200_last_error()
        torch.cuda.synchronize()
        g, r = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.abs(g - r).max() <= 2e-2 * np.abs(r).max()  # the tolerance of the matmul tests; in practice identical
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
