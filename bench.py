#!/usr/bin/env python
"""Benchmark of the continuous-batching decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Workloads (BASELINE.json `configs`, synthetic seeded inputs):
  paged_attn_bf16 / paged_attn_fp8 : config 2, the paged-attention decode microbench — 64
      sequences, contexts log-uniform 128..32768, 32 query / 8 KV heads, head_dim 128, 32-token
      pages scattered by a random permutation over a pool of 1.25x the pages in use.
      One step = one decode of all 64 sequences through one attention layer.
Multi-GPU (torchrun, one rank per GPU): independent replicas of the workload, no collective in the
step (requests never interact); `value` = tokens of all ranks / max-over-ranks time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D, PAGE = 32, 8, 128, 32


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def c2_contexts(seed: int, n_seq: int = 64) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return np.rint(np.exp(rng.uniform(np.log(128), np.log(32768), n_seq))).astype(np.int64)


def algorithmic_bytes(ctxs: np.ndarray, kv_bytes: int) -> float:
    """Per call: K and V of every cached token once, q and out once, one page id per page,
    plus one f32 scale per (page, kv head, K|V) for FP8 pools."""
    pages = -(-ctxs // PAGE)
    b = (2 * HKV * D * kv_bytes * ctxs).sum() + len(ctxs) * 2 * HQ * D * 2 + 4 * pages.sum()
    if kv_bytes == 1:
        b += 2 * 4 * HKV * pages.sum()
    return float(b)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_c2(dev, torch, seed: int, fp8: bool, n_seq: int = 64):
    """Fills a scattered page pool with the config-2 contexts; returns the pool and the step inputs."""
    ctxs = c2_contexts(seed, n_seq)
    rng = np.random.default_rng(seed + 1)
    pages = int((-(-ctxs // PAGE)).sum())
    n_pages = int(np.ceil(pages * 1.25))
    kv = dev.PagedKVCache(1, HKV, D, n_pages, len(ctxs), int(-(-ctxs.max() // PAGE)), HQ, max_rows=int(ctxs.sum()),
                          kv_dtype=dev.KV_FP8_E4M3 if fp8 else dev.KV_BF16)
    kv.set_free_order(rng.permutation(n_pages).tolist())
    kv.reserve(dev.pack_desc_array([(s, int(c), 0, -1) for s, c in enumerate(ctxs)]).cuda())
    g = torch.Generator(device="cuda").manual_seed(seed)
    total = int(ctxs.sum())
    k = torch.randn((total, HKV, D), generator=g, device="cuda", dtype=torch.float32).bfloat16()
    v = torch.randn((total, HKV, D), generator=g, device="cuda", dtype=torch.float32).bfloat16()
    kv.append(0, k, v)
    torch.cuda.synchronize()
    assert kv.error_word() == 0
    q = (torch.randn((len(ctxs), HQ, D), generator=g, device="cuda") / np.sqrt(D)).bfloat16()
    return kv, ctxs, q, (k, v)


def cpu_baseline_c2(ctxs, kv, k_rows, v_rows, q, sample: int = 8, min_time: float = 3.0, warm: bool = True):
    """The reference's algorithm (gather pages -> repeat heads -> dense attention) in C/OpenMP on
    the host, on the first `sample` sequences of the same workload."""
    import torch

    from oracle import ref_c

    idx = np.arange(min(sample, len(ctxs)))
    # a compact pool holding just the sampled sequences, pages in order
    off = np.concatenate([[0], np.cumsum(ctxs)])
    tables, pools_k, pools_v, nxt = [], [], [], 0
    max_pages = int(-(-ctxs[idx].max() // PAGE))
    for s in idx:
        c = int(ctxs[s])
        np_s = -(-c // PAGE)
        ks = k_rows[off[s]:off[s] + c].view(torch.int16).cpu().numpy().view(np.uint16)
        vs = v_rows[off[s]:off[s] + c].view(torch.int16).cpu().numpy().view(np.uint16)
        pad = np_s * PAGE - c
        ks = np.concatenate([ks, np.zeros((pad, HKV, D), np.uint16)]).reshape(np_s, PAGE, HKV, D).transpose(0, 2, 1, 3)
        vs = np.concatenate([vs, np.zeros((pad, HKV, D), np.uint16)]).reshape(np_s, PAGE, HKV, D).transpose(0, 2, 1, 3)
        pools_k.append(np.ascontiguousarray(ks))
        pools_v.append(np.ascontiguousarray(vs))
        t = np.zeros(max_pages, np.int32)
        t[:np_s] = np.arange(nxt, nxt + np_s)
        nxt += np_s
        tables.append(t)
    kp, vp = np.concatenate(pools_k), np.concatenate(pools_v)
    qq = q[idx].float().cpu().numpy()
    if warm:
        ref_c.paged_attention_decode(kp, vp, np.stack(tables), ctxs[idx].astype(np.int32), HQ, HKV, D, qq)
    reps, t0 = 0, time.perf_counter()
    while True:
        ref_c.paged_attention_decode(kp, vp, np.stack(tables), ctxs[idx].astype(np.int32), HQ, HKV, D, qq)
        reps += 1
        if time.perf_counter() - t0 > min_time or reps >= 20:
            break
    dt = (time.perf_counter() - t0) / reps
    tok_s = len(idx) / dt
    return {"value": tok_s, "unit": "decode tokens/s", "cores": ref_c.num_threads(), "kind": "port",
            "sample": f"first {len(idx)} of {len(ctxs)} sequences ({int(ctxs[idx].sum())} cached tokens), "
                      f"{reps} repetitions; gather+repeat+dense attention as the reference does per step"}, dt


def run_reference(args, rank: int):
    """--impl reference: the reference's own algorithm for the path on the host cores.  The
    reference itself (Zig + MLX) cannot be built here, so the timed code is the oracle's C twin."""
    if rank != 0:
        return
    import torch

    seed = 1234
    ctxs = c2_contexts(seed)
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn((len(ctxs), HQ, D), generator=g) / np.sqrt(D)).bfloat16()
    # Calibrate on the first sequence, then take as many leading sequences as fit ~120 s overall.
    c0 = int(ctxs[0])
    k0 = torch.randn((c0, HKV, D), generator=g).bfloat16()
    _, dt0 = cpu_baseline_c2(ctxs, None, k0, k0, q, 1, min_time=0.0, warm=True)
    per_token = dt0 / c0
    budget_tokens = 120.0 / max(args.steps + args.warmup, 1) / per_token
    sample = int(np.searchsorted(np.cumsum(ctxs), budget_tokens, side="right"))
    sample = max(1, min(sample, 8))
    total = int(ctxs[:sample].sum())
    k = torch.randn((total, HKV, D), generator=g).bfloat16()
    v = torch.randn((total, HKV, D), generator=g).bfloat16()
    cb, dt = None, None
    times = []
    for i in range(args.warmup + args.steps):
        cb, dt = cpu_baseline_c2(ctxs, None, k, v, q, sample, min_time=0.0, warm=False)
        if i >= args.warmup:
            times.append(dt)
    ms = float(np.mean(times) * 1e3)
    val = sample / (ms / 1e3)
    cb["value"] = val
    print(json.dumps({
        "impl": "reference", "metric": "decode tokens/sec (ragged continuous batch)", "value": val,
        "unit": "decode tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": args.workload, "note": f"bounded sample: first {sample} of 64 sequences per step"},
        "cpu_baseline": cb, "e2e": {"value": val, "unit": "decode tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="paged_attn_bf16")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--seqs", type=int, default=64, help="sequences per GPU (64 = the configuration; fewer for profiling)")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = 10 if args.impl == "reference" else 500
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    from dmlx_b200 import device as dev  # raises if the CUDA library is missing: no fallback

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    fp8 = args.workload.endswith("fp8")
    kv, ctxs, q, (k_rows, v_rows) = build_c2(dev, torch, 1234 + rank, fp8, args.seqs)
    n_seq = len(ctxs)
    row_seq = torch.arange(n_seq, dtype=torch.int32, device="cuda")
    row_ctx = torch.tensor(ctxs, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    W = max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: one step = one attention decode over all sequences ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: it samples from warm-up to the end of the run
    for _ in range(W):
        kv.attention(0, q, row_seq, row_ctx, out)
    barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    t_all0 = torch.cuda.Event(enable_timing=True)
    t_all1 = torch.cuda.Event(enable_timing=True)
    t_all0.record()
    for a, b in evs:
        a.record()
        kv.attention(0, q, row_seq, row_ctx, out)
        b.record()
    t_all1.record()
    barrier()
    total_ms = t_all0.elapsed_time(t_all1)
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in evs]))
    assert kv.error_word() == 0

    # ---- end to end through the C-ABI with host buffers: q from pinned host memory every step,
    #      result read back to the host every step ----
    q_host = q.cpu().pin_memory()
    out_host = torch.empty_like(q_host).pin_memory()
    desc_host = torch.stack([row_seq.cpu(), row_ctx.cpu()]).pin_memory()
    d_desc = torch.empty_like(desc_host, device="cuda")
    for _ in range(W):
        q.copy_(q_host, non_blocking=True)
        d_desc.copy_(desc_host, non_blocking=True)
        kv.attention(0, q, d_desc[0], d_desc[1], out)
        out_host.copy_(out, non_blocking=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        q.copy_(q_host, non_blocking=True)
        d_desc.copy_(desc_host, non_blocking=True)
        kv.attention(0, q, d_desc[0], d_desc[1], out)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller consumes the result before the next step
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    if world > 1:
        t = torch.tensor([total_ms, e2e_ms, kern_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms, kern_ms = t.tolist()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    tokens_per_step = n_seq * world
    peak, peak_kind = load_peaks()
    kv_bytes = 1 if fp8 else 2
    alg = algorithmic_bytes(ctxs, kv_bytes)
    achieved = alg / (kern_ms * 1e-3) / 1e9
    result = {
        "metric": "decode tokens/sec (ragged continuous batch)",
        "value": tokens_per_step / (ms_per_step * 1e-3),
        "unit": "decode tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": W, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if not fp8 else "fp8_e4m3 KV, bf16 q/out, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": args.workload, "sequences_per_gpu": n_seq, "contexts": "log-uniform 128..32768 (seeded)",
                   "cached_tokens_per_gpu": int(ctxs.sum()), "q_heads": HQ, "kv_heads": HKV, "head_dim": D,
                   "page_tokens": PAGE, "pool": "random permutation over 1.25x pages in use",
                   "l2": f"inputs larger than L2 ({alg / 1e6:.0f} MB of KV per step)", "parallelism": f"dp{world}"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "traffic": None, "kernel": "paged_attn_kernel (+plan, +combine)",
                     "algorithmic_bytes_per_launch": alg, "kernel_ms": kern_ms, "frac_of_8TBs": achieved / 8000.0},
        "e2e": {"value": tokens_per_step / (e2e_ms / args.steps * 1e-3), "unit": "decode tokens/s",
                "h2d_bytes_per_step": int(q_host.numel() * 2 + desc_host.numel() * 4),
                "d2h_bytes_per_step": int(out_host.numel() * 2)},
        "gpu_launches": 3 * args.steps,
        "clocks": clocks,
    }
    traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(traffic_file):
        result["roofline"]["traffic"] = json.load(open(traffic_file)).get(args.workload)
    if not args.no_cpu_baseline:
        cb, _ = cpu_baseline_c2(ctxs, kv, k_rows, v_rows, q)
        result["cpu_baseline"] = cb
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
