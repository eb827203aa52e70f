"""Expert parallelism on the CPU: what can be checked without a GPU.

* The decomposition the library uses — all-gather of the token rows, replicated routing, every rank
  evaluating its own experts for the tokens of all ranks, an f32 reduce-scatter of the per-rank sums —
  is run by two gloo ranks with the oracle's arithmetic in place of the kernels and must equal the
  single-process oracle layer (src/models/deepseek_v4.zig:721-848) for every token.
* The watchdog loop behind b200_ep_wait (b200_ep_watch) is driven with fake operations: work that
  finishes, a communicator that reports an error, work that never finishes.
* StepGuard, the host-side arrival check between steps: a rank that leaves after a step is noticed by
  the other before it queues anything for the next one.
"""
import ctypes as C
import os
import socket
import time

import numpy as np
import pytest
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
            rng.normal(0, 0.3, (E, D, INTER)).astype(np.float32), rng.normal(0, 0.5, (E, D)).astype(np.float32))


def _inputs(rank):
    return np.random.default_rng(100 + rank).normal(0, 1, (N_PER_RANK, D)).astype(np.float32)


def _layer_worker(rank, port, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    wg, wu, wd, wr = _weights()
    x = torch.tensor(_inputs(rank))
    # dispatch: every rank's rows to every rank, rank-major
    parts = [torch.empty_like(x) for _ in range(WORLD)]
    dist.all_gather(parts, x)
    x_all = torch.cat(parts).numpy()
    # replicated routing over the tokens of all ranks
    wts, idx = ref_math.gate_forward(x_all @ wr.T, None, K, route_scale=1.5)
    # plan: the assignments that fall on this rank's experts, grouped by local expert (stable)
    el = E // WORLD
    partial = np.zeros((WORLD * N_PER_RANK, D), np.float64)
    for e in range(el):
        ge = rank * el + e
        for t, j in zip(*np.nonzero(idx == ge)):
            xs = x_all[t].astype(np.float64)
            a = ref_math.limited_swiglu(wg[ge].astype(np.float64) @ xs, wu[ge].astype(np.float64) @ xs, 10.0) * float(wts[t, j])
            partial[t] += wd[ge].astype(np.float64) @ a
    # combine: sum over ranks, every rank keeps its own tokens (reduce-scatter; gloo: all-reduce + slice)
    total = torch.tensor(partial.astype(np.float32))
    dist.all_reduce(total)
    mine = total[rank * N_PER_RANK:(rank + 1) * N_PER_RANK].numpy()
    np.save(os.path.join(out_dir, f"out{rank}.npy"), mine)
    dist.destroy_process_group()


def test_two_rank_all_gather_route_reduce_scatter_matches_single_process(tmp_path):
    mp.spawn(_layer_worker, args=(_free_port(), str(tmp_path)), nprocs=WORLD, join=True)
    wg, wu, wd, wr = _weights()
    for rank in range(WORLD):
        x = _inputs(rank)
        wts, idx = ref_math.gate_forward(x @ wr.T, None, K, route_scale=1.5)
        want = ref_math.switch_glu(x, idx, wts, wg, wu, wd, limit=10.0)
        got = np.load(tmp_path / f"out{rank}.npy")
        assert np.allclose(got, want, rtol=1e-4, atol=1e-5), rank


def _watch(done_after=None, error_after=None, timeout_ms=200):
    from dmlx_b200 import _lib

    state = {"polls": 0, "aborted": 0}

    def done(_ctx):
        state["polls"] += 1
        return int(done_after is not None and state["polls"] > done_after)

    def err(_ctx):
        return int(error_after is not None and state["polls"] > error_after)

    def abort(_ctx):
        state["aborted"] += 1

    ops = _lib.EpWatchOps(_lib.EpWatchOps._fields_[0][1](done), _lib.EpWatchOps._fields_[1][1](err),
                          _lib.EpWatchOps._fields_[2][1](abort), None)
    t0 = time.monotonic()
    r = _lib.lib.b200_ep_watch(C.byref(ops), timeout_ms, 200)
    return r, state, time.monotonic() - t0


def test_watchdog_returns_when_the_work_finishes():
    r, st, _ = _watch(done_after=5)
    assert r == 0 and st["aborted"] == 0 and st["polls"] == 6


def test_watchdog_aborts_on_an_asynchronous_error():
    r, st, _ = _watch(error_after=3)
    assert r == 1 and st["aborted"] == 1


def test_watchdog_aborts_when_the_time_is_up():
    r, st, dt = _watch(timeout_ms=150)
    assert r == 2 and st["aborted"] == 1 and 0.14 <= dt < 2.0


def _guard_worker(rank, port, out_dir):
    from dmlx_b200 import expert_parallel as ep

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=2)
    store = dist.distributed_c10d._get_default_store()
    guard = ep.StepGuard(store, rank, 2, timeout_s=1.0)
    guard.arrive(1)        # both ranks are here
    result = "step 1 ok"
    if rank == 1:
        # leaves between steps, with nothing in flight (no collective was queued after the arrival)
        open(os.path.join(out_dir, "r1.txt"), "w").write(result)
        os._exit(0)
    t0 = time.monotonic()
    try:
        guard.arrive(2)
        result = "step 2 ok"
    except ep.PeerLost as e:
        result = f"lost after {time.monotonic() - t0:.2f}s: {e}"
    open(os.path.join(out_dir, "r0.txt"), "w").write(result)
    os._exit(0)  # the group cannot be destroyed collectively any more


def test_step_guard_notices_a_rank_that_left_between_steps(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_guard_worker, args=(r, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert open(tmp_path / "r1.txt").read() == "step 1 ok"
    r0 = open(tmp_path / "r0.txt").read()
    assert r0.startswith("lost after") and "rank(s) [1] did not reach step 2" in r0, r0
