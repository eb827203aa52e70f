#!/usr/bin/env python
"""Benchmark of the continuous-batching decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Workloads (synthetic seeded inputs):
  llama8b_int4 (default) : config 3, the Llama-3-8B-shaped int4 continuous-batching decode step at a
      fixed live-batch snapshot — 256 requests in flight, each with its lognormal prompt
      (mean 1024, sigma 0.6, clipped 32..8192) plus a uniform share of its 128..1024 output tokens
      already generated; weights affine 4-bit group 64 (random codes), paged bf16 KV in 32-token
      pages.  One step = one decode token for each of the 256 requests through all 32 layers,
      lm_head and greedy argmax.
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


# DRAM traffic / algorithmic bytes of the attention kernels: dram__bytes_read.sum + dram__bytes_write.sum
# of one ncu capture of a 16-sequence case of the attention microbench (a case that a capture can hold),
# divided by that case's algorithmic bytes.  Traffic grows in proportion to the cached tokens (one pass
# over every page), so the ratio carries over to a full launch.
TRAFFIC_RATIO = {"bf16": 1.02, "fp8": 1.04}


def traffic_ratio(fp8: bool = False):
    return TRAFFIC_RATIO["fp8" if fp8 else "bf16"]


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

    ref_c.use_all_cores()
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



# ---------------------------------------------------------------------------------------------
# config 3: Llama-3-8B-shaped int4 decode step
# ---------------------------------------------------------------------------------------------
L8 = dict(n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, vocab=128256)


def c3_snapshot(seed: int, n_req: int = 256):
    """Context length of every live request: prompt + tokens generated so far."""
    rng = np.random.default_rng(seed)
    sigma = 0.6
    mu = np.log(1024.0) - sigma * sigma / 2  # lognormal with mean 1024
    prompt = np.clip(np.rint(rng.lognormal(mu, sigma, n_req)), 32, 8192).astype(np.int64)
    out_len = rng.integers(128, 1025, n_req)
    done = (rng.random(n_req) * out_len).astype(np.int64)
    return prompt + done


def llama_weight_bytes(c) -> float:
    qkv = (c["n_heads"] + 2 * c["n_kv_heads"]) * c["head_dim"]
    per_layer = c["hidden"] * (qkv + c["n_heads"] * c["head_dim"]) + 3 * c["hidden"] * c["ffn"]
    return 0.5625 * (c["n_layers"] * per_layer + c["vocab"] * c["hidden"])


def run_llama(args, rank, world, local):
    import torch
    import torch.distributed as dist

    from dmlx_b200 import device as dev

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # a stream of our own: decode steps are replayed as CUDA graphs, which the legacy default
    # stream cannot capture
    torch.cuda.set_stream(torch.cuda.Stream())
    c = dict(L8)
    if args.layers:
        c["n_layers"] = args.layers
    n_req = args.seqs if args.seqs != 64 else 256
    K, W = args.steps, max(args.warmup, 3)
    ctxs = c3_snapshot(4321 + rank, n_req)
    grow = 2 * (K + W) + 8
    n_pages = int((-(-(ctxs + grow) // PAGE)).sum() * 1.1) + 16
    kv = dev.PagedKVCache(c["n_layers"], c["n_kv_heads"], c["head_dim"], n_pages, n_req,
                          int(-(-(ctxs.max() + grow) // PAGE)), c["n_heads"], max_rows=max(n_req, 16))
    rng = np.random.default_rng(99 + rank)
    kv.set_free_order(rng.permutation(n_pages).tolist())
    do_arrivals = not args.no_arrivals and n_req == 256
    model = dev.LlamaModel(c["n_layers"], c["hidden"], c["n_heads"], c["n_kv_heads"], c["head_dim"], c["ffn"], c["vocab"],
                           max_rows=max(n_req, 16, (args.step_tokens + 256) if do_arrivals else 0), max_reqs=max(n_req, 256 if do_arrivals else 0),
                           max_seqs=max(n_req, 256 if do_arrivals else 0), rms_eps=1e-5, rope_theta=500000.0)
    model.random_init(dev.Q_AFFINE4_G64, seed=7 + rank)
    if getattr(args, "unfused_qkv_rope", False):
        model.set_fused_qkv_rope(False)
    # live-batch snapshot: every request already holds `ctx` cached tokens in every layer
    kv.reserve(dev.pack_desc_array([(s, int(n), 0, -1) for s, n in enumerate(ctxs)]).cuda())
    g = torch.Generator(device="cuda").manual_seed(5 + rank)
    total = int(ctxs.sum())
    krows = torch.randn((total, c["n_kv_heads"], c["head_dim"]), generator=g, device="cuda").bfloat16()
    vrows = torch.randn((total, c["n_kv_heads"], c["head_dim"]), generator=g, device="cuda").bfloat16()
    for layer in range(c["n_layers"]):
        kv.append(layer, krows, vrows)
    torch.cuda.synchronize()
    assert kv.error_word() == 0
    del krows, vrows

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    lens = ctxs.copy()

    def host_descs():
        return [(s, 1, int(lens[s]), -1) for s in range(n_req)]

    def device_descs(n_steps):
        a = np.zeros((n_steps, n_req, 4), np.int32)
        for i in range(n_steps):
            a[i, :, 0] = np.arange(n_req)
            a[i, :, 1] = 1
            a[i, :, 2] = lens + i
            a[i, :, 3] = -1
        return torch.tensor(a, device="cuda")

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- device-resident: descriptors already in HBM, no host copies in the timed region ----
    d = device_descs(W + K)
    cur = torch.empty_like(d[0])  # fixed address: decode steps of one shape replay one CUDA graph
    for i in range(W):
        cur.copy_(d[i])
        model.forward_device(kv, cur, n_req)
    barrier()
    launches0 = model.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(W, W + K):
        cur.copy_(d[i])
        model.forward_device(kv, cur, n_req)
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    launches = model.launch_count() - launches0
    lens += W + K
    assert kv.error_word() == 0 and dev.qmm_error_word() == 0
    # ---- the same steps with per-kernel CUDA events (roofline of the dominant kernel) ----
    P = min(K, 10)
    d = device_descs(P)
    model.profile_enable(True)
    for i in range(P):
        cur.copy_(d[i])
        model.forward_device(kv, cur, n_req)
    prof = model.profile_collect()
    model.profile_enable(False)
    live_tokens = float(lens.sum() + n_req * (P + 1) / 2.0)
    lens += P
    # ---- end to end: host descriptors in, host tokens out, every step ----
    for _ in range(2):
        model.step(kv, host_descs())
        lens += 1
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    E = min(K, 20)
    t0.record()
    for _ in range(E):
        toks, free = model.step(kv, host_descs())
        lens += 1
    t1.record()
    barrier()
    e2e_ms = t0.elapsed_time(t1) / E
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([total_ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = t.tolist()
    # the same model through the engine as an arrival process (all ranks take part: 256 requests in total)
    arrivals = None
    # (a failure in these two additions is reported under their key; it does not cost the run its headline line)
    if do_arrivals:
        launches_before = model.launch_count()
        kv.close()
        try:
            arrivals = run_arrivals(args, rank, world, local, model=model, c=c)
        except Exception as e:  # noqa: BLE001
            arrivals = {"error": f"{type(e).__name__}: {e}"}
    # on several GPUs: the one workload with an exchange step, the MoE layer stack under expert parallelism
    expert_parallel = None
    if world > 1 and not args.no_ep and not args.layers:
        try:
            model.close()
            torch.cuda.empty_cache()
            mc, m_total, m_e2e, mK, _, _, _, _ = moe_measure(args, rank, world, torch, dist, dev, steps=20)
            expert_parallel = moe_summary(mc, m_total, m_e2e, mK, world)
        except Exception as e:  # noqa: BLE001
            expert_parallel = {"error": f"{type(e).__name__}: {e}"}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_per_step = total_ms / K
    peak, peak_kind = load_peaks()
    attn_ms, attn_calls = prof["attention"]
    mm_ms, mm_calls = prof["matmul"]
    kv_bytes_per_call = 2 * c["n_kv_heads"] * c["head_dim"] * 2 * live_tokens + n_req * 2 * c["n_heads"] * c["head_dim"] * 2 \
        + 4 * float((-(-lens // PAGE)).sum())
    attn_launch_ms = attn_ms / max(attn_calls, 1)
    achieved = kv_bytes_per_call / (attn_launch_ms * 1e-3) / 1e9
    wbytes = llama_weight_bytes(c)
    result = {
        "metric": "decode tokens/sec (ragged continuous batch)",
        "value": n_req * world / (ms_per_step * 1e-3), "unit": "decode tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 affine g64 weights, bf16 activations and KV, f32 accumulate", "data": "synthetic",
        "config": {"workload": "llama8b_int4 decode step at a 256-request live-batch snapshot" if n_req == 256 and not args.layers
                   else f"llama8b_int4 reduced ({c['n_layers']} layers, {n_req} requests)",
                   "requests_per_gpu": n_req, "layers": c["n_layers"], "hidden": c["hidden"], "q_heads": c["n_heads"],
                   "kv_heads": c["n_kv_heads"], "head_dim": c["head_dim"], "ffn": c["ffn"], "vocab": c["vocab"],
                   "cached_tokens_per_gpu": int(lens.sum()), "prompt": "lognormal mean 1024 sigma 0.6 clip 32..8192",
                   "page_tokens": PAGE, "l2": f"inputs larger than L2 ({(wbytes + 32 * kv_bytes_per_call) / 1e9:.1f} GB read per step)",
                   "parallelism": f"dp{world}"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "traffic": None, "frac_of_8TBs": achieved / 8000.0,
                     "kernel": "paged_attn_mma_kernel (+plan, +combine), one launch per layer",
                     "algorithmic_bytes_per_launch": kv_bytes_per_call, "kernel_ms": attn_launch_ms,
                     "step_breakdown_ms": {k: v[0] / P for k, v in prof.items()},
                     "step_breakdown_sum_ms": sum(v[0] for v in prof.values()) / P,
                     "step_breakdown_note": "per-kernel CUDA events on eager launches outside graph replay: each figure "
                                            "includes the launch gap that follows the kernel, so the sum exceeds ms_per_step",
                     "matmul": {"ms_per_step": mm_ms / P, "weight_GBs": wbytes / (mm_ms / P * 1e-3) / 1e9,
                                "tflops": 2.0 * n_req * wbytes / 0.5625 / (mm_ms / P * 1e-3) / 1e12}},
        "e2e": {"value": n_req * world / (e2e_ms * 1e-3), "unit": "decode tokens/s",
                "h2d_bytes_per_step": 16 * n_req, "d2h_bytes_per_step": 4 * n_req + 36},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    result["roofline"]["traffic"] = traffic_ratio() * kv_bytes_per_call
    result["roofline"]["traffic_note"] = "dram bytes of an ncu capture of a 16-sequence case, scaled by cached tokens (ratio to algorithmic bytes 1.02)"
    if arrivals:
        result["arrivals"] = arrivals
    if expert_parallel:
        result["expert_parallel"] = expert_parallel
    if not args.no_cpu_baseline and world == 1:
        result["cpu_baseline"] = cpu_baseline_c3(c, n_req)
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline_c3(c, n_req, sample_req: int = 32, layers: int = 3, min_time: float = 2.0, seed: int = 4321):
    """One decode step of the reference's structure on the host, bounded: `layers` layers (each with its
    own weights) for the first `sample_req` requests of the snapshot (per-step page gather + head repeat
    + dense attention, then the four int4 matmuls of the layer), repeated until `min_time` seconds have
    been measured, and extrapolated to the full stack + lm_head by parameter count and to the whole
    batch by request count."""
    from oracle import ref_c

    ref_c.use_all_cores()
    ctxs = c3_snapshot(seed, n_req)[:sample_req]
    rng = np.random.default_rng(0)
    hq, hkv, d, hid, ffn = c["n_heads"], c["n_kv_heads"], c["head_dim"], c["hidden"], c["ffn"]
    pages = -(-ctxs // PAGE)
    kp = rng.integers(0, 2 ** 16, (int(pages.sum()), hkv, PAGE, d), dtype=np.uint16) & 0xBF7F
    table = np.zeros((sample_req, int(pages.max())), np.int32)
    nxt = 0
    for s in range(sample_req):
        table[s, :pages[s]] = np.arange(nxt, nxt + pages[s])
        nxt += pages[s]
    q = rng.normal(0, 1, (sample_req, hq, d)).astype(np.float32)
    x = rng.normal(0, 1, (sample_req, hid)).astype(np.float32)
    xf = rng.normal(0, 1, (sample_req, ffn)).astype(np.float32)

    def qw(n, k):
        return (rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint32), np.full((n, k // 64), 0.005, np.float32),
                np.full((n, k // 64), -0.04, np.float32))

    weights = [(qw((hq + 2 * hkv) * d, hid), qw(hid, hq * d), qw(2 * ffn, hid), qw(hid, ffn)) for _ in range(layers)]
    measured, passes = 0.0, 0
    while measured < min_time or passes == 0:
        t0 = time.perf_counter()
        for wqkv, wo, wgu, wdn in weights:
            ref_c.qmm_affine4(*wqkv, x)
            ref_c.paged_attention_decode(kp, kp, table, ctxs.astype(np.int32), hq, hkv, d, q)
            ref_c.qmm_affine4(*wo, x)
            ref_c.qmm_affine4(*wgu, x)
            ref_c.qmm_affine4(*wdn, xf)
        measured += time.perf_counter() - t0
        passes += 1
    t_layer = measured / passes / layers
    per_layer_params = hid * ((hq + 2 * hkv) * d + hq * d) + 3 * hid * ffn
    t_step = t_layer * (c["n_layers"] + c["vocab"] * hid / per_layer_params * 0.5)
    return {"value": sample_req / t_step, "unit": "decode tokens/s", "cores": ref_c.num_threads(), "kind": "port",
            "measured_s": measured, "passes": passes, "sample_step_s": measured / passes,
            "sample": f"{layers} layers for the first {sample_req} of {n_req} requests ({int(ctxs.sum())} cached tokens), "
                      f"{passes} passes = {measured:.2f} s measured, extrapolated to {c['n_layers']} layers + lm_head"}


# ---------------------------------------------------------------------------------------------
# the Llama-3-8B-shaped int4 workload as an arrival process through the engine
# ---------------------------------------------------------------------------------------------
def c3_requests(seed: int, vocab: int, n_req: int = 256, rate: float = 20.0):
    """256 requests arriving Poisson at `rate` per second: prompt lengths lognormal (mean 1024, sigma 0.6,
    clipped 32..8192), output lengths uniform 128..1024, token ids uniform over the vocabulary."""
    rng = np.random.default_rng(seed)
    arrive = np.cumsum(rng.exponential(1.0 / rate, n_req)) if rate > 0 else np.zeros(n_req)
    sigma = 0.6
    mu = np.log(1024.0) - sigma * sigma / 2
    prompt = np.clip(np.rint(rng.lognormal(mu, sigma, n_req)), 32, 8192).astype(np.int64)
    out_len = rng.integers(128, 1025, n_req)
    prompts = [rng.integers(0, vocab, int(n)).astype(np.uint32) for n in prompt]
    return arrive, prompts, out_len


def route_requests(prompts, out_len, world: int):
    """Request -> replica.  Every rank computes the same table from the request list alone: each
    request goes to the replica with the fewest tokens assigned so far (a static stand-in for routing by
    least live KV pages, which would need the replicas' state on the router)."""
    load = np.zeros(world, np.int64)
    owner = np.zeros(len(prompts), np.int64)
    for i, (p, o) in enumerate(zip(prompts, out_len)):
        r = int(np.argmin(load))
        owner[i] = r
        load[r] += len(p) + int(o)
    return owner


def run_arrival_scenario(dev, torch, model, c, rank, world, barrier, rate: float, pool_pages: int, chunk: int,
                         step_tokens: int, n_req: int = 256, seed: int = 2025, time_limit: float = 150.0):
    """One pass of the arrival process through b200_engine_step (host buffers in and out every step):
    submissions at their arrival times, chunked prefill interleaved with decode, requests finishing and
    returning their pages, admission waiting on the page pool.  Returns this rank's raw measurements."""
    arrive, prompts, out_len = c3_requests(seed, c["vocab"], n_req, rate)
    owner = route_requests(prompts, out_len, world)
    mine = [i for i in range(n_req) if owner[i] == rank]
    max_pages_per_seq = int(-(-(8192 + 1024 + 1) // PAGE))
    # split-K partial slots of the attention kernels: a prefill chunk is served in groups of 4 rows (16 MMA
    # rows / GQA group of 4), each group walking its whole context in chunks of 8 pages
    scratch_chunks = (step_tokens // 4 + n_req) * (max_pages_per_seq // 8 + 1)
    kv = dev.PagedKVCache(c["n_layers"], c["n_kv_heads"], c["head_dim"], pool_pages, max(len(mine), 1), max_pages_per_seq,
                          c["n_heads"], max_rows=step_tokens + n_req, attn_scratch_chunks=scratch_chunks)
    eng = dev.Engine(model, kv, max_prefill_tokens=chunk)
    eng.set_max_step_tokens(step_tokens)
    first_t, last_t, count = {}, {}, {}
    ttft, itl, batch_sizes, step_ms = [], [], [], []
    nxt, done, steps, out_tokens = 0, 0, 0, 0
    barrier()
    t_start = time.perf_counter()
    busy = 0.0
    while done < len(mine):
        now = time.perf_counter() - t_start
        if now > time_limit:
            break
        while nxt < len(mine) and arrive[mine[nxt]] <= now:
            i = mine[nxt]
            eng.submit(i + 1, prompts[i], int(out_len[i]))
            nxt += 1
        if eng.active_count() == 0:
            if nxt < len(mine):
                time.sleep(max(0.0, min(0.002, arrive[mine[nxt]] - now)))
            continue
        t0 = time.perf_counter()
        outs = eng.step()
        t1 = time.perf_counter()
        busy += t1 - t0
        steps += 1
        step_ms.append((t1 - t0) * 1e3)
        batch_sizes.append(len(outs))
        t = t1 - t_start
        for rid, _tok in outs:
            if rid not in first_t:
                first_t[rid] = t
                ttft.append(t - arrive[rid - 1])
                count[rid] = 0
            else:
                itl.append(t - last_t[rid])
            last_t[rid] = t
            count[rid] += 1
            out_tokens += 1
            if count[rid] >= out_len[rid - 1]:
                done += 1
                eng.forget(rid)
    makespan = time.perf_counter() - t_start
    deferred, preempted, failed = eng.pressure_stats()
    free_end, err = eng.free_pages(), kv.error_word()
    eng.close()
    kv.close()
    return {"requests": len(mine), "finished": done, "out_tokens": out_tokens, "makespan": makespan, "busy": busy, "steps": steps,
            "ttft": ttft, "itl": itl, "batch": batch_sizes, "step_ms": step_ms, "deferred": deferred, "preempted": preempted,
            "failed": failed, "pages_back": free_end == pool_pages, "error_word": err,
            "prompt_tokens": int(sum(len(prompts[i]) for i in mine))}


def summarise_arrivals(parts, rate, pool_pages, chunk, step_tokens, world):
    """Whole-job figures from the per-rank measurements (latencies pooled over all requests)."""
    def pct(a, q):
        return float(np.percentile(a, q)) if len(a) else None

    ttft = np.concatenate([np.asarray(p["ttft"], np.float64) for p in parts])
    itl = np.concatenate([np.asarray(p["itl"], np.float64) for p in parts])
    batch = np.concatenate([np.asarray(p["batch"], np.float64) for p in parts])
    step_ms = np.concatenate([np.asarray(p["step_ms"], np.float64) for p in parts])
    makespan = max(p["makespan"] for p in parts)
    out_tokens = sum(p["out_tokens"] for p in parts)
    return {
        "workload": "256 requests, Poisson arrivals at %g req/s, prompts lognormal (mean 1024, sigma 0.6, clip 32..8192), outputs uniform 128..1024, greedy, through b200_engine_step with host buffers" % rate
                    if rate > 0 else "256 requests all present at t = 0 (saturation), same prompts and outputs, through b200_engine_step with host buffers",
        "replicas": world, "routing": "least assigned tokens" if world > 1 else None,
        "requests": sum(p["requests"] for p in parts), "finished": sum(p["finished"] for p in parts),
        "prompt_tokens": sum(p["prompt_tokens"] for p in parts), "output_tokens": out_tokens,
        "makespan_s": makespan, "decode_tokens_per_s": out_tokens / makespan,
        "total_tokens_per_s": (out_tokens + sum(p["prompt_tokens"] for p in parts)) / makespan,
        "gpu_busy_fraction": float(np.mean([p["busy"] / p["makespan"] for p in parts])),
        "ttft_ms": {"p50": pct(ttft, 50) * 1e3, "p90": pct(ttft, 90) * 1e3, "p99": pct(ttft, 99) * 1e3} if len(ttft) else None,
        "itl_ms": {"p50": pct(itl, 50) * 1e3, "p90": pct(itl, 90) * 1e3, "p99": pct(itl, 99) * 1e3} if len(itl) else None,
        "engine_steps": sum(p["steps"] for p in parts), "step_ms": {"p50": pct(step_ms, 50), "p99": pct(step_ms, 99)},
        "tokens_joined_per_step_mean": float(batch.mean()) if len(batch) else None,
        "pool_pages_per_replica": pool_pages, "prefill_chunk": chunk, "step_token_budget": step_tokens,
        "request_steps_deferred_for_pages": sum(p["deferred"] for p in parts),
        "preemptions": sum(p["preempted"] for p in parts), "requests_failed": sum(p["failed"] for p in parts),
        "every_page_returned": all(p["pages_back"] for p in parts), "error_words_clear": all(p["error_word"] == 0 for p in parts),
    }


def run_arrivals(args, rank, world, local, model=None, c=None, quiet=False):
    """--workload llama8b_int4_arrivals: the arrival process on its own (also called by the default
    workload, which reports it beside the snapshot step)."""
    import torch
    import torch.distributed as dist

    from dmlx_b200 import device as dev

    own = model is None
    if own:
        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        torch.cuda.set_stream(torch.cuda.Stream())
        c = dict(L8)
        if args.layers:
            c["n_layers"] = args.layers
        model = dev.LlamaModel(c["n_layers"], c["hidden"], c["n_heads"], c["n_kv_heads"], c["head_dim"], c["ffn"], c["vocab"],
                               max_rows=args.step_tokens + 256, max_reqs=256, max_seqs=256, rms_eps=1e-5, rope_theta=500000.0)
        model.random_init(dev.Q_AFFINE4_G64, seed=7 + rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = {}
    # the two scenarios on a pool small enough that admission has to wait (--pool-pages), and the saturated one
    # again on a pool that holds all 256 requests at once (4 MiB per page over 32 layers: 64 GiB)
    for name, rate, pool in (("poisson_20rps", 20.0, args.pool_pages), ("saturation", 0.0, args.pool_pages),
                             ("saturation_large_pool", 0.0, 16384)):
        if args.arrival_scenarios != "both" and args.arrival_scenarios != name:
            continue
        part = run_arrival_scenario(dev, torch, model, c, rank, world, barrier, rate, pool, args.prefill_chunk, args.step_tokens)
        if world > 1:
            parts = [None] * world
            dist.all_gather_object(parts, part)
        else:
            parts = [part]
        out[name] = summarise_arrivals(parts, rate, pool, args.prefill_chunk, args.step_tokens, world)
    if own:
        if rank == 0 and not quiet:
            sat = out.get("saturation") or next(iter(out.values()))
            print(json.dumps({
                "metric": "decode tokens/sec (ragged continuous batch)", "value": sat["decode_tokens_per_s"], "unit": "decode tokens/s",
                "n_gpus": world, "steps": sat["engine_steps"], "warmup": 0, "ms_per_step": sat["step_ms"]["p50"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int4 affine g64 weights, bf16 activations and KV, f32 accumulate", "data": "synthetic",
                "config": {"workload": "llama8b_int4_arrivals: " + sat["workload"], "layers": c["n_layers"],
                           "l2": "inputs larger than L2 (4.2 GB of weights per step)", "parallelism": f"dp{world}, 256 requests in total"},
                "arrivals": out, "e2e": {"value": sat["decode_tokens_per_s"], "unit": "decode tokens/s",
                                         "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                                         "note": "every engine step copies its descriptors and prefill tokens in and its tokens out"},
                "roofline": None, "gpu_launches": int(model.launch_count()), "clocks": None}))
        if world > 1:
            dist.destroy_process_group()
    return out


# ---------------------------------------------------------------------------------------------
# config 4: MXFP4 MoE layer stack (expert parallel across ranks)
# ---------------------------------------------------------------------------------------------
MOE = dict(hidden=4096, n_experts=256, inter=2048, top_k=6, layers=4, tokens=4096)


def moe_measure(args, rank, world, torch, dist, dev, steps=None):
    """The MoE layer stack on `world` ranks (experts sharded over the ranks when world > 1): device-timed
    and end-to-end times of a step, max over ranks.  Returns (config, total_ms, e2e_ms, K, W, launches, clocks, bytes)."""
    from dmlx_b200 import expert_parallel as ep

    c = dict(MOE)
    if args.layers:
        c["layers"] = args.layers
    if args.moe_tmem_a >= 0:
        dev.set_qmm_grouped_tmem_a(bool(args.moe_tmem_a))
    if args.moe_block_scaled >= 0:
        dev.set_qmm_grouped_block_scaled(bool(args.moe_block_scaled))
    K, W = steps or args.steps, max(args.warmup, 3)
    n_tok = c["tokens"] // world  # the step decodes 4096 tokens in total: strong scaling
    el = c["n_experts"] // world
    rng = np.random.default_rng(77)
    bias = rng.normal(0, 0.004, c["n_experts"]).astype(np.float32)  # skewed load
    comm = ep.Communicator(rank, world) if world > 1 else None
    layers = []
    for l in range(c["layers"]):
        gate = dev.QWeight.random(dev.Q_BF16, c["n_experts"], c["hidden"], 1, seed=1000 + l)
        gu = dev.QWeight.random(dev.Q_MXFP4_G32, 2 * c["inter"], c["hidden"], el, seed=2000 + 97 * l + rank)
        dn = dev.QWeight.random(dev.Q_MXFP4_G32, c["hidden"], c["inter"], el, seed=3000 + 97 * l + rank)
        sgu = dev.QWeight.random(dev.Q_MXFP4_G32, 2 * c["inter"], c["hidden"], 1, seed=4000 + l)
        sdn = dev.QWeight.random(dev.Q_MXFP4_G32, c["hidden"], c["inter"], 1, seed=5000 + l)
        if world == 1:
            layers.append(dev.MoELayer(c["hidden"], c["n_experts"], c["inter"], c["top_k"], gate, gu, dn, sgu, sdn,
                                       bias=bias, route_scale=1.5, tile_rows=args.moe_tile, max_tokens=n_tok))
        else:
            layers.append(ep.ExpertParallelMoE(comm, c["hidden"], c["n_experts"], c["inter"], c["top_k"], gate, gu, dn, sgu, sdn,
                                               bias=bias, route_scale=1.5, tile_rows=args.moe_tile, max_tokens=n_tok))
    x_host = torch.randn((n_tok, c["hidden"]), generator=torch.Generator().manual_seed(11 + rank)).bfloat16().pin_memory()
    x = x_host.cuda()
    bufs = [torch.empty_like(x) for _ in range(2)]

    def step(inp):
        h = inp
        for i, layer in enumerate(layers):
            h = layer.forward(h, bufs[i & 1])
        return h

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    for _ in range(W):
        step(x)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = dev.launch_count()
    e0.record()
    for _ in range(K):
        step(x)
    e1.record()
    barrier()
    launches = dev.launch_count() - launches0
    total_ms = e0.elapsed_time(e1)
    out_host = torch.empty_like(x_host).pin_memory()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(K):
        x.copy_(x_host, non_blocking=True)
        out_host.copy_(step(x), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    t1.record()
    barrier()
    e2e_ms = t0.elapsed_time(t1)
    clocks = sampler.stop() if rank == 0 else None
    assert dev.qmm_error_word() == 0
    if comm is not None:
        comm.wait(timeout_ms=20000)
    if world > 1:
        t = torch.tensor([total_ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = t.tolist()
    for layer in layers:
        layer.close()
    if comm is not None:
        comm.close()
    return c, total_ms, e2e_ms, K, W, int(launches), clocks, int(x_host.numel() * 2 * world)


def moe_summary(c, total_ms, e2e_ms, K, world):
    """Short form of the MoE measurement (the default workload reports it when it runs on several GPUs)."""
    ms = total_ms / K
    per_expert_params = 3 * c["inter"] * c["hidden"]
    flops = c["layers"] * c["tokens"] * (c["top_k"] + 1) * 2.0 * per_expert_params
    return {"workload": f"moe_mxfp4 layer stack: {c['layers']} layers, hidden {c['hidden']}, {c['n_experts']} routed experts of "
                        f"{c['inter']} + 1 shared, top-{c['top_k']}, {c['tokens']} tokens per step in total",
            "parallelism": f"ep{world}: experts sharded over the ranks, all-gather dispatch + f32 reduce-scatter combine (NCCL)",
            "scaling": "strong", "ms_per_step": ms, "tokens_per_s": c["tokens"] / (ms * 1e-3),
            "e2e_tokens_per_s": c["tokens"] / (e2e_ms / K * 1e-3), "tflops_bf16_equivalent": flops / (ms * 1e-3) / 1e12}


def run_moe(args, rank, world, local):
    import torch
    import torch.distributed as dist

    from dmlx_b200 import device as dev

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    c, total_ms, e2e_ms, K, W, launches, clocks, io_bytes = moe_measure(args, rank, world, torch, dist, dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms = total_ms / K
    per_expert_params = 3 * c["inter"] * c["hidden"]
    flops = c["layers"] * c["tokens"] * (c["top_k"] + 1) * 2.0 * per_expert_params
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0)) * world
    achieved = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "decode tokens/sec (ragged continuous batch)", "value": c["tokens"] / (ms * 1e-3), "unit": "decode tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "mxfp4 weights (E2M1 + E8M0/32), bf16 activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": "moe_mxfp4 layer stack", "layers": c["layers"], "hidden": c["hidden"], "experts": c["n_experts"],
                   "expert_inter": c["inter"], "shared_experts": 1, "top_k": c["top_k"], "tokens_per_step": c["tokens"],
                   "routing": "softmax + seeded per-expert bias (skewed load)",
                   "l2": f"inputs larger than L2 ({c['layers'] * 257 * per_expert_params * 0.53125 / 1e9:.1f} GB of expert weights)",
                   "parallelism": f"ep{world}" if world > 1 else "single GPU, all experts local"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_kind": "of measured (sustained cuBLAS bf16)" if peaks else "of fallback", "traffic": None,
                     "kernel": "qmm_mx_kernel grouped (gate/up + down, tcgen05 kind::mxf8f6f4 block-scaled) and dense (shared expert)",
                     "algorithmic_flops_per_step": flops},
        "e2e": {"value": c["tokens"] / (e2e_ms / K * 1e-3), "unit": "decode tokens/s",
                "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes},
        "gpu_launches": int(launches), "clocks": clocks,
    }))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# quantised matmul microbench: the Llama-3-8B layer shapes at a given number of packed rows
# ---------------------------------------------------------------------------------------------
QMM_SHAPES = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336),
              "lm_head": (128256, 4096)}


def run_qmm(args, local):
    """One step = every selected shape once (weights rotated so that nothing is served from L2).
    Up to 16 rows the path is a weight stream (HBM roofline on the weight bytes); from 64 rows it is
    a dense contraction (tensor roofline)."""
    import torch

    from dmlx_b200 import device as dev

    torch.cuda.set_device(local)
    mxfp4 = args.workload.endswith("mxfp4")
    mode = dev.Q_MXFP4_G32 if mxfp4 else dev.Q_AFFINE4_G64
    bytes_per_weight = 0.53125 if mxfp4 else 0.5625
    rows = args.rows
    names = list(QMM_SHAPES) if args.shape == "all" else [args.shape]
    stream = torch.cuda.Stream()
    per_shape, launches = {}, 0
    sampler = ClockSampler(local)
    sampler.start()
    with torch.cuda.stream(stream):
        for name in names:
            n, k = QMM_SHAPES[name]
            copies = 2 if n > 100000 else 8  # more weight bytes than the 126 MB L2 between reuses
            ws = [dev.QWeight.random(mode, n, k, 1, seed=17 + i) for i in range(copies)]
            x = torch.randn((rows, k), device="cuda").bfloat16()
            epi = dev.EPI_SWIGLU if name == "gate_up" else dev.EPI_NONE
            out = torch.empty((rows, n // 2 if epi else n), device="cuda", dtype=torch.bfloat16)
            for _ in range(max(args.warmup, 3)):
                for w in ws:
                    dev.qmm(w, x, epi, out=out, path=args.path)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for w in ws:
                    dev.qmm(w, x, epi, out=out, path=args.path)
            g.replay()
            stream.synchronize()
            l0 = dev.launch_count()
            for w in ws:  # counted outside the graph: launches per pass over the copies
                dev.qmm(w, x, epi, out=out, path=args.path)
            per_call = (dev.launch_count() - l0) / copies
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
            us = e0.elapsed_time(e1) / args.steps / copies * 1e3
            launches += per_call * args.steps * copies
            per_shape[name] = {"us": us, "weight_GBs": bytes_per_weight * n * k / us / 1e3,
                               "tflops": 2.0 * rows * n * k / us / 1e6, "kernels_per_call": per_call}
            del ws, g
    clocks = sampler.stop()
    assert dev.qmm_error_word() == 0
    hbm_peak, peak_kind = load_peaks()
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    total_us = sum(v["us"] for v in per_shape.values())
    total_w = sum(bytes_per_weight * QMM_SHAPES[nm][0] * QMM_SHAPES[nm][1] for nm in names)
    top = max(names, key=lambda nm: QMM_SHAPES[nm][0] * QMM_SHAPES[nm][1])
    if rows <= 58:  # below the ridge (208 flop/B over 3.56 flop/B per row): weight streaming
        roof = {"bound": "hbm", "achieved": per_shape[top]["weight_GBs"], "peak": hbm_peak, "unit": "GB/s",
                "frac": per_shape[top]["weight_GBs"] / hbm_peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                "frac_of_8TBs": per_shape[top]["weight_GBs"] / 8000.0}
    else:
        tpeak = float(peaks.get("bf16_tflops", 1590.0))
        roof = {"bound": "tensor", "achieved": per_shape[top]["tflops"], "peak": tpeak, "unit": "TFLOP/s",
                "frac": per_shape[top]["tflops"] / tpeak, "peak_kind": "of measured (burst cuBLAS bf16)" if peaks else "of fallback",
                "traffic": None}
    roof["kernel"] = f"{top}: " + ("qmm_mma_kernel" if rows <= 16 and args.path in (0, 3) else "automatic choice between qmm_tca_kernel and qmm_tc2_kernel" if args.path == 0 else f"path {args.path}")
    print(json.dumps({
        "metric": "quantised matmul weight bytes per second", "value": total_w / total_us / 1e3, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_us / 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": ("mxfp4" if mxfp4 else "int4 affine g64") + " weights, bf16 activations, f32 accumulate",
        "data": "synthetic", "config": {"workload": args.workload, "rows": rows, "shapes": {nm: QMM_SHAPES[nm] for nm in names},
                                        "path": args.path, "l2": "weights rotated over more than L2 between reuses"},
        "roofline": roof, "per_shape": per_shape, "e2e": None, "gpu_launches": int(launches), "clocks": clocks,
    }))


# ---------------------------------------------------------------------------------------------
# config 5: chunked prefill + decode with a shared prompt prefix (copy-on-write pages), FP8 KV
# ---------------------------------------------------------------------------------------------
C5 = dict(prefix=2048, suffix_lo=64, suffix_hi=1024, chunk=512, requests=512, new_tokens=32, step_tokens=8192)


def run_prefix_prefill(args, rank, world, local):
    """The per-GPU share of config 5 (512 requests over 8 GPUs = 64 per GPU unless --seqs says
    otherwise) through the engine step: the first request prefills the 2048-token prefix, the others
    take its pages over by reference count when they start, prefill only their own suffix in
    512-token chunks (a step carries at most 8192 tokens) interleaved with the decode of the
    requests that are already generating.  Host descriptors in, host tokens out, every step."""
    import torch
    import torch.distributed as dist

    from dmlx_b200 import device as dev

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    c, w = dict(L8), dict(C5)
    if args.layers:
        c["layers"] = c["n_layers"] = args.layers
    n_req = args.seqs if args.seqs != 64 else w["requests"] // 8
    rows_cap = w["step_tokens"] + n_req
    rng = np.random.default_rng(515 + rank)
    prefix = rng.integers(0, c["vocab"], w["prefix"]).tolist()
    suffixes = [rng.integers(0, c["vocab"], int(rng.integers(w["suffix_lo"], w["suffix_hi"] + 1))).tolist() for _ in range(n_req)]
    per_req_pages = -(-(w["suffix_hi"] + w["new_tokens"]) // PAGE) + 2
    n_pages = w["prefix"] // PAGE + n_req * per_req_pages + 64
    kv = dev.PagedKVCache(c["n_layers"], c["n_kv_heads"], c["head_dim"], n_pages, n_req,
                          -(-(w["prefix"] + w["suffix_hi"] + w["new_tokens"]) // PAGE) + 2, c["n_heads"], max_rows=rows_cap,
                          kv_dtype=dev.KV_FP8_E4M3, attn_scratch_chunks=4 * rows_cap + 1024)
    model = dev.LlamaModel(c["n_layers"], c["hidden"], c["n_heads"], c["n_kv_heads"], c["head_dim"], c["ffn"], c["vocab"],
                           max_rows=rows_cap, max_reqs=n_req, max_seqs=n_req, rms_eps=1e-5, rope_theta=500000.0)
    model.random_init(dev.Q_AFFINE4_G64, seed=7 + rank)

    def scenario(n):
        kv.reset()
        eng = dev.Engine(model, kv, max_prefill_tokens=w["chunk"])
        eng.set_prefix_sharing(True)
        eng.set_max_step_tokens(w["step_tokens"])
        eng.submit(1, prefix + suffixes[0], w["new_tokens"])
        steps = 0
        for _ in range(w["prefix"] // w["chunk"]):  # the prefix is in the pool before the others arrive
            eng.step()
            steps += 1
        for i in range(1, n):
            eng.submit(i + 1, prefix + suffixes[i], w["new_tokens"])
        while eng.active_count() > 0 and steps < 100000:
            eng.step()
            steps += 1
        shared = sum(eng.shared_tokens(i + 1) for i in range(n))
        gen = sum(len(eng.result(i + 1)[0]) for i in range(n))
        free = eng.free_pages()
        eng.close()
        return steps, shared, gen, free

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(1, min(args.warmup, 2))):
        scenario(min(n_req, 6))  # warm-up: lazy set-up, scratch growth
    K = max(1, min(args.steps, 3))
    barrier()
    l0 = dev.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        steps, shared, gen, free = scenario(n_req)
    e1.record()
    barrier()
    launches = dev.launch_count() - l0
    total_ms = e0.elapsed_time(e1)
    assert kv.error_word() == 0 and dev.qmm_error_word() == 0
    assert gen == n_req * w["new_tokens"] and free == n_pages, (gen, free)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms = total_ms / K
    prompt_tokens = sum(w["prefix"] + len(sfx) for sfx in suffixes)
    computed = prompt_tokens - shared + gen - n_req  # every generated token but each request's first comes from a decode row
    params = llama_weight_bytes(c) / 0.5625
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    tpeak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    tflops = 2.0 * params * computed / (ms * 1e-3) / 1e12
    val = gen * world / (ms * 1e-3)
    print(json.dumps({
        "metric": "decode tokens/sec (ragged continuous batch)", "value": val, "unit": "decode tokens/s", "n_gpus": world,
        "steps": K, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4 affine g64 weights, bf16 activations, FP8-E4M3 KV, f32 accumulate", "data": "synthetic",
        "config": {"workload": "prefix_prefill: chunked prefill + decode with a shared prompt prefix", "requests_per_gpu": n_req,
                   "layers": c["n_layers"], "prefix_tokens": w["prefix"], "suffix_tokens": [w["suffix_lo"], w["suffix_hi"]],
                   "prefill_chunk": w["chunk"], "step_token_budget": w["step_tokens"], "new_tokens_per_request": w["new_tokens"],
                   "engine_steps": steps, "prompt_tokens": prompt_tokens, "prompt_tokens_shared": shared,
                   "tokens_computed": computed, "a_step_is": "one whole scenario (all requests prefilled and decoded)",
                   "l2": "weights (4.5 GB) are read every engine step", "parallelism": f"dp{world}"},
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": tpeak, "unit": "TFLOP/s", "frac": tflops / tpeak,
                     "peak_kind": "of measured (sustained cuBLAS bf16)" if peaks else "of fallback", "traffic": None,
                     "kernel": "whole scenario: dense flops of the tokens computed over its duration"},
        "e2e": {"value": val, "unit": "decode tokens/s", "h2d_bytes_per_step": int(4 * (prompt_tokens - shared) + 16 * steps * n_req),
                "d2h_bytes_per_step": int(4 * gen)},
        "gpu_launches": int(launches), "clocks": clocks,
    }))
    if world > 1:
        dist.destroy_process_group()


def run_reference(args, rank: int):
    """--impl reference: the reference's own algorithm for the path on the host cores.  The
    reference itself (Zig + MLX) cannot be built here, so the timed code is the oracle's C twin."""
    if rank != 0:
        return
    from oracle import ref_c

    ref_c.use_all_cores()  # torchrun exports OMP_NUM_THREADS=1
    if args.workload.startswith("llama"):
        # one step = one bounded sample (3 layers for 32 of the 256 requests); `value` extrapolates it to
        # the full stack, `ms_per_step` is the time the sample itself took
        times, cb = [], None
        for i in range(args.warmup + args.steps):
            cb = cpu_baseline_c3(dict(L8), 256, min_time=0.0)
            if i >= args.warmup:
                times.append((cb["sample_step_s"], 32 / cb["value"]))
            if sum(t for t, _ in times) > 150.0:
                break
        ms = float(np.mean([t for t, _ in times]) * 1e3)
        full_ms = float(np.mean([f for _, f in times]) * 1e3)
        val = 32 / (full_ms / 1e3)
        cb["value"] = val
        cb["sample"] = f"3 layers for the first 32 of 256 requests per step, {len(times)} steps, extrapolated to 32 layers + lm_head"
        print(json.dumps({
            "impl": "reference", "metric": "decode tokens/sec (ragged continuous batch)", "value": val,
            "unit": "decode tokens/s", "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "llama8b_int4 decode step at a 256-request live-batch snapshot",
                       "note": "ms_per_step is the measured time of one bounded sample (3 layers, 32 of 256 requests); value "
                               "extrapolates it to the full stack: 32 requests / extrapolated_full_step_ms",
                       "extrapolated_full_step_ms": full_ms},
            "cpu_baseline": cb,
            "e2e": {"value": val, "unit": "decode tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return
    if args.workload.startswith(("qmm", "moe")):
        # dequantise + matmul in the C twin on a bounded sample of weight rows, extrapolated linearly
        mxfp4 = args.workload.endswith("mxfp4")
        rng = np.random.default_rng(0)
        if args.workload.startswith("qmm"):
            names = list(QMM_SHAPES) if args.shape == "all" else [args.shape]
            shapes, rows, scale_to = [QMM_SHAPES[nm] for nm in names], args.rows, 1.0
        else:  # one expert's gate/up and down matmuls at the mean rows per expert, times 257 experts and the layers
            shapes = [(2 * MOE["inter"], MOE["hidden"]), (MOE["hidden"], MOE["inter"])]
            rows = MOE["tokens"] * MOE["top_k"] // MOE["n_experts"]
            scale_to = float((MOE["n_experts"] + MOE["tokens"] / rows) * MOE["layers"])
        times = []
        for i in range(args.warmup + args.steps):
            t_step = 0.0
            for n, k in shapes:
                ns = min(n, 4096)
                x = rng.normal(0, 1, (rows, k)).astype(np.float32)
                if mxfp4:
                    w = (rng.integers(0, 256, (ns, k // 2), dtype=np.uint8), rng.integers(118, 124, (ns, k // 32), dtype=np.uint8))
                    t0 = time.perf_counter()
                    ref_c.qmm_mxfp4(w[0], w[1], x)
                else:
                    w = (rng.integers(0, 2 ** 32, (ns, k // 8), dtype=np.uint32), np.full((ns, k // 64), 0.005, np.float32),
                         np.full((ns, k // 64), -0.04, np.float32))
                    t0 = time.perf_counter()
                    ref_c.qmm_affine4(w[0], w[1], w[2], x)
                t_step += (time.perf_counter() - t0) * n / ns
            if i >= args.warmup:
                times.append(t_step * scale_to)
        ms = float(np.mean(times) * 1e3)
        bpw = 0.53125 if mxfp4 else 0.5625
        if args.workload.startswith("qmm"):
            metric, unit, val = "quantised matmul weight bytes per second", "GB/s", sum(bpw * n * k for n, k in shapes) / (ms * 1e-3) / 1e9
        else:
            metric, unit, val = "decode tokens/sec (ragged continuous batch)", "decode tokens/s", MOE["tokens"] / (ms * 1e-3)
        cb = {"value": val, "unit": unit, "cores": ref_c.num_threads(), "kind": "port",
              "sample": f"first 4096 weight rows of every matrix at {rows} rows, extrapolated linearly"}
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": args.workload, "rows": rows}, "cpu_baseline": cb,
            "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
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
    ap.add_argument("--workload", default="llama8b_int4")
    ap.add_argument("--moe-tile", type=int, default=112,
                    help="moe_mxfp4 only: token tile of the grouped matmul (up to 112 rows the block-scaled kernel keeps two accumulator sets)")
    ap.add_argument("--moe-block-scaled", type=int, default=-1, help="moe_mxfp4 only: 1 runs the grouped matmuls on tcgen05.mma kind::mxf8f6f4 (hardware block scaling), 0 on the dequantising kernels (default: library choice)")
    ap.add_argument("--moe-tmem-a", type=int, default=-1, help="moe_mxfp4 only: 0/1 forces the grouped matmul kernel (default: library choice)")
    ap.add_argument("--layers", type=int, default=0, help="llama8b_int4 only: fewer layers (profiling / smoke runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--rows", type=int, default=1, help="qmm_* only: packed rows")
    ap.add_argument("--shape", default="all", help="qmm_* only: qkv | o | gate_up | down | lm_head | all")
    ap.add_argument("--path", type=int, default=0, help="qmm_* only: kernel path (0 = automatic)")
    ap.add_argument("--seqs", type=int, default=64, help="sequences per GPU (64 = the configuration; fewer for profiling)")
    ap.add_argument("--mx-persistent", type=int, default=-1, help="block-scaled MXFP4 path: 1 persistent CTAs over work items, 0 one CTA per item (default: library choice)")
    ap.add_argument("--no-arrivals", action="store_true", help="llama8b_int4 only: skip the arrival-process scenarios")
    ap.add_argument("--attn-pages-per-chunk", type=int, default=0,
                    help="tuning: pages per split-K chunk of the decode attention (0 = the library's default)")
    ap.add_argument("--unfused-qkv-rope", action="store_true",
                    help="llama8b_int4 snapshot step only: keep the q/k/v projection's own finish pass (A/B of the fused RoPE + append)")
    ap.add_argument("--no-ep", action="store_true", help="llama8b_int4 on several GPUs only: skip the expert-parallel MoE measurement")
    ap.add_argument("--arrival-scenarios", default="both", help="poisson_20rps | saturation | saturation_large_pool | both (= all three)")
    ap.add_argument("--pool-pages", type=int, default=3072, help="arrival scenarios: KV pages per replica (32 tokens x 32 layers x 4 KiB each)")
    ap.add_argument("--prefill-chunk", type=int, default=512, help="arrival scenarios: prefill chunk (tokens)")
    ap.add_argument("--step-tokens", type=int, default=2048, help="arrival scenarios: token budget of one engine step")
    args = ap.parse_args()
    if args.attn_pages_per_chunk > 0:
        from dmlx_b200 import device as _dev
        _dev.set_attn_pages_per_chunk(args.attn_pages_per_chunk)
    if args.steps is None:
        args.steps = 10 if args.impl == "reference" else (150 if args.workload.startswith("llama") else (20 if args.workload.startswith(("moe", "qmm")) else (2 if args.workload.startswith("prefix") else 500)))
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
    if args.mx_persistent >= 0:
        from dmlx_b200 import _lib
        _lib.lib.b200_set_qmm_mx_persistent(args.mx_persistent)
    if args.workload == "llama8b_int4_arrivals":
        run_arrivals(args, rank, world, local)
        return
    if args.workload.startswith("llama"):
        run_llama(args, rank, world, local)
        return
    if args.workload.startswith("moe"):
        run_moe(args, rank, world, local)
        return
    if args.workload.startswith("qmm"):
        if rank == 0:
            run_qmm(args, local)
        return
    if args.workload.startswith("prefix"):
        run_prefix_prefill(args, rank, world, local)
        return
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
                     "peak_kind": f"of {peak_kind}", "traffic": None, "kernel": ("paged_attn_mma_fp8_kernel" if fp8 else "paged_attn_mma_kernel") + " (+plan, +combine)",
                     "algorithmic_bytes_per_launch": alg, "kernel_ms": kern_ms, "frac_of_8TBs": achieved / 8000.0},
        "e2e": {"value": tokens_per_step / (e2e_ms / args.steps * 1e-3), "unit": "decode tokens/s",
                "h2d_bytes_per_step": int(q_host.numel() * 2 + desc_host.numel() * 4),
                "d2h_bytes_per_step": int(out_host.numel() * 2)},
        "gpu_launches": 3 * args.steps,
        "clocks": clocks,
    }
    result["roofline"]["traffic"] = traffic_ratio(fp8) * alg
    result["roofline"]["traffic_note"] = "dram bytes of an ncu capture of a 16-sequence case, scaled by cached tokens"
    if not args.no_cpu_baseline and world == 1:
        cb, _ = cpu_baseline_c2(ctxs, kv, k_rows, v_rows, q)
        result["cpu_baseline"] = cb
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
