"""Expert-parallel MoE on 2 GPUs (b200_moe_forward_ep: all-gather dispatch, reduce-scatter combine over
NCCL) equals the single-GPU layer with all experts local.  Skipped when fewer than 2 GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

E, K, D, INTER, N = 8, 2, 256, 128, 48


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _make(rng, n_e, rows, cols):
    packed = rng.integers(0, 256, (n_e, rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(118, 122, (n_e, rows, cols // 32), dtype=np.uint8)
    return packed, scales


def _data():
    rng = np.random.default_rng(31)
    wg = (rng.normal(0, 0.3, (E, D)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    return dict(wg=wg, gu=_make(rng, E, 2 * INTER, D), dn=_make(rng, E, D, INTER), sgu=_make(rng, 1, 2 * INTER, D),
                sdn=_make(rng, 1, D, INTER), bias=rng.normal(0, 0.01, E).astype(np.float32),
                x=[rng.normal(0, 1, (N, D)).astype(np.float32) for _ in range(2)])


def _qw(dev, pk, sc, lo, hi):
    p, s = pk[lo:hi], sc[lo:hi]
    n_e, rows, half = p.shape
    return dev.QWeight(dev.Q_MXFP4_G32, p.reshape(n_e * rows, half), s.reshape(n_e * rows, -1), None, rows, half * 2, n_experts=n_e)


def _worker(rank, port, out_dir):
    import torch.distributed as dist

    from dmlx_b200 import device as dev
    from dmlx_b200 import expert_parallel as ep

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=2)  # carries the communicator id only
    d = _data()
    el = E // 2
    gate = dev.QWeight(dev.Q_BF16, d["wg"], np.zeros(1, np.uint8), None, E, D)
    comm = ep.Communicator(rank, 2)
    layer = ep.ExpertParallelMoE(comm, D, E, INTER, K, gate, _qw(dev, *d["gu"], rank * el, (rank + 1) * el),
                                 _qw(dev, *d["dn"], rank * el, (rank + 1) * el), _qw(dev, *d["sgu"], 0, 1),
                                 _qw(dev, *d["sdn"], 0, 1), bias=d["bias"], route_scale=1.5, tile_rows=32, max_tokens=64)
    x = torch.tensor(d["x"][rank], device="cuda").bfloat16()
    for _ in range(3):  # several steps back to back: no host synchronisation between them
        out = layer.forward(x)
    comm.wait(timeout_ms=20000)
    np.save(os.path.join(out_dir, f"ep{rank}.npy"), out.float().cpu().numpy())
    assert dev.qmm_error_word() == 0
    layer.close()
    comm.close()
    dist.destroy_process_group()


def test_two_gpu_expert_parallel_matches_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    from dmlx_b200 import device as dev

    mp.spawn(_worker, args=(_free_port(), str(tmp_path)), nprocs=2, join=True)
    d = _data()
    gate = dev.QWeight(dev.Q_BF16, d["wg"], np.zeros(1, np.uint8), None, E, D)
    single = dev.MoELayer(D, E, INTER, K, gate, _qw(dev, *d["gu"], 0, E), _qw(dev, *d["dn"], 0, E), _qw(dev, *d["sgu"], 0, 1),
                          _qw(dev, *d["sdn"], 0, 1), bias=d["bias"], route_scale=1.5, tile_rows=32, max_tokens=64)
    for rank in range(2):
        want = single.forward(torch.tensor(d["x"][rank], device="cuda").bfloat16()).float().cpu().numpy()
        got = np.load(tmp_path / f"ep{rank}.npy")
        # same kernels and rows; the sum over k runs in f32 across the ranks and is rounded once
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max(), rank
