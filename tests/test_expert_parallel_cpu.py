"""Expert-parallel dispatch/combine bookkeeping on CPU: two gloo ranks exchange counts and rows with
the product's planning code (dmlx_b200.expert_parallel); the expert arithmetic in between is the
oracle's (there is no CPU compute path in the product).  The result must equal the single-process
oracle layer (src/models/deepseek_v4.zig:721-848) for every token."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref_math


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


E, K, D, INTER, N_PER_RANK, WORLD = 8, 2, 16, 8, 11, 2


def _weights():
    rng = np.random.default_rng(5)
    return (rng.normal(0, 0.3, (E, INTER, D)).astype(np.float32), rng.normal(0, 0.3, (E, INTER, D)).astype(np.float32),
            rng.normal(0, 0.3, (E, D, INTER)).astype(np.float32))


def _inputs(rank):
    rng = np.random.default_rng(100 + rank)
    x = rng.normal(0, 1, (N_PER_RANK, D)).astype(np.float32)
    logits = rng.normal(0, 1, (N_PER_RANK, E)).astype(np.float32)
    return x, logits


def _worker(rank, port, out_dir):
    from dmlx_b200 import expert_parallel as ep

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    wg, wu, wd = _weights()
    x, logits = _inputs(rank)
    wts, idx = ref_math.gate_forward(logits, None, K, route_scale=1.5)
    order, inv, tok, offsets = ref_math.group_by_expert(idx, E)
    counts = torch.tensor(np.diff(offsets), dtype=torch.int32)
    x_sorted = torch.tensor(x[tok])
    scales = torch.tensor(wts.reshape(-1)[order])
    # ---- product planning + exchange ----
    recv_counts = ep.exchange_counts(counts, WORLD)
    send = ep.send_splits(counts, WORLD)
    recv = recv_counts.sum(1).tolist()
    rows = ep.all_to_all_rows(x_sorted, send, recv)
    rscales = ep.all_to_all_rows(scales, send, recv)
    index, loc_off = ep.regroup_index(recv_counts)
    items = ep.work_items(loc_off, 4)
    assert int(items[:, 2].sum()) == rows.shape[0] == int(loc_off[-1])
    xe, se = rows[index.long()], rscales[index.long()]
    # ---- expert arithmetic (oracle): local expert e = global expert rank * E/W + e ----
    el = E // WORLD
    ye = torch.zeros((xe.shape[0], D))
    for e in range(el):
        ge = rank * el + e
        seg = slice(int(loc_off[e]), int(loc_off[e + 1]))
        xs = xe[seg].numpy().astype(np.float64)
        a = ref_math.limited_swiglu(xs @ wg[ge].T.astype(np.float64), xs @ wu[ge].T.astype(np.float64), 10.0)
        a = a * se[seg].numpy()[:, None]
        ye[seg] = torch.tensor((a @ wd[ge].T.astype(np.float64)).astype(np.float32))
    inverse = torch.empty_like(index)
    inverse[index.long()] = torch.arange(index.shape[0], dtype=torch.int32)
    y_sorted = ep.all_to_all_rows(ye[inverse.long()], recv, send)
    out = y_sorted[torch.tensor(inv).long()].view(N_PER_RANK, K, D).sum(1).numpy()
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out)
    dist.destroy_process_group()


def test_two_rank_dispatch_combine_matches_single_process(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    wg, wu, wd = _weights()
    for rank in range(WORLD):
        x, logits = _inputs(rank)
        wts, idx = ref_math.gate_forward(logits, None, K, route_scale=1.5)
        want = ref_math.switch_glu(x, idx, wts, wg, wu, wd, limit=10.0)
        got = np.load(tmp_path / f"out{rank}.npy")
        assert np.allclose(got, want, rtol=1e-4, atol=1e-5), rank


def test_regroup_index_and_items():
    from dmlx_b200 import expert_parallel as ep

    rc = torch.tensor([[2, 0, 1], [1, 3, 0]], dtype=torch.int32)  # 2 sources, 3 local experts
    index, off = ep.regroup_index(rc)
    # receive buffer: s0:[e0,e0,e2] s1:[e0,e1,e1,e1]; expert-major: e0: 0,1,3  e1: 4,5,6  e2: 2
    assert index.tolist() == [0, 1, 3, 4, 5, 6, 2] and off.tolist() == [0, 3, 6, 7]
    assert ep.work_items(off, 2).tolist() == [[0, 0, 2, 0], [0, 2, 1, 0], [1, 3, 2, 0], [1, 5, 1, 0], [2, 6, 1, 0]]
    assert ep.send_splits(torch.tensor([1, 2, 3, 4]), 2) == [3, 7]
