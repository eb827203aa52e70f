"""CPU (numpy, fp32/fp64) restatement of the reference's floating-point math on the decode path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``dmlx_b200/`` may import this module.

Pinning status
--------------
* rms_norm / rope / sdpa / embedding are pinned against the reference's own golden vectors
  (src/tests/golden/{rmsnorm,rope,sdpa,embedding}_*.bin, recipe tests/generate_golden.py:62-112),
  to the reference's thresholds (cosine >= 0.9999 and |diff| <= 1e-4,
  src/tests/golden_test.zig:35-48,298-300) in tests/test_oracle_math.py.
* PARITY UNPINNED: affine 4-bit ``quantized_matmul`` bit layout and rounding, ``gather_qmm``
  (MXFP4) outputs, argsort tie order, multi-step greedy ids.  That arithmetic lives in MLX /
  mlx_z v0.0.2 (build.zig.zon:7-10), which is not vendored in the reference tree; the formats
  below are self-consistent definitions following the layout facts the reference states
  (src/kvcache/paged.zig:358,1199-1208; src/models/llama_loader.zig:262-279;
  src/models/deepseek_v4_loader.zig:839-920).
* FP8-E4M3 KV pages with per-(page, kv-head) scales have no counterpart in the reference's Paged
  strategy (it offers affine 4/8-bit pages, src/kvcache/paged.zig:352-356); the definition here is
  this project's own and parity for it is measured against the bf16 path.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import ml_dtypes
import numpy as np

BF16 = ml_dtypes.bfloat16
E4M3 = ml_dtypes.float8_e4m3fn
E4M3_MAX = 448.0


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bfloat16, returned as float32."""
    return np.asarray(x, np.float32).astype(BF16).astype(np.float32)


# ---------------------------------------------------------------------------
# KAT-pinned primitives
# ---------------------------------------------------------------------------


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    """x * rsqrt(mean(x^2) + eps) * weight over the last axis (src/models/llama.zig:462,473,592)."""
    x = np.asarray(x, np.float32)
    ms = np.mean(x.astype(np.float64) ** 2, axis=-1, keepdims=True)
    return (x * (1.0 / np.sqrt(ms + eps)).astype(np.float32) * weight).astype(np.float32)


def rope(x: np.ndarray, positions: np.ndarray, theta: float = 10000.0) -> np.ndarray:
    """Non-traditional (half-split) rotary embedding (tests/generate_golden.py:79).

    x: [..., S, D]; positions: [S] (per-row absolute positions).  Pair (i, i + D/2) is rotated by
    positions * theta^(-2i/D).  At B=1 a per-row position equals the reference's scalar offset +
    row index (src/models/llama.zig:213-215).
    """
    x = np.asarray(x, np.float32)
    d = x.shape[-1]
    half = d // 2
    inv = theta ** (-np.arange(half, dtype=np.float64) * 2.0 / d)
    ang = np.asarray(positions, np.float64)[:, None] * inv[None, :]
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    x1, x2 = x[..., :half], x[..., half:]
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1)


def sdpa(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, mask: Optional[np.ndarray] = None) -> np.ndarray:
    """softmax(q k^T * scale + mask) v (src/models/llama.zig:249-270)."""
    s = np.einsum("...qd,...kd->...qk", q.astype(np.float64), k.astype(np.float64)) * scale
    if mask is not None:
        s = s + mask
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("...qk,...kd->...qd", p, v.astype(np.float64)).astype(np.float32)


def embedding(weight: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """Row gather (src/models/llama.zig:566)."""
    return weight[np.asarray(ids, np.int64)]


def silu(x):
    return x / (1.0 + np.exp(-x))


# ---------------------------------------------------------------------------
# Weight formats
# ---------------------------------------------------------------------------


def quantize_affine4(w: np.ndarray, group: int = 64) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Affine 4-bit quantisation along K in groups of ``group``.

    Returns (packed uint32 [N, K/8], scales bf16-valued f32 [N, K/group], biases same).
    Element j of each run of 8 sits in bits 4j..4j+3 (el_per_int = 32/bits,
    src/kvcache/paged.zig:358; scales/biases [out, in/group], src/models/llama_loader.zig:270).
    """
    w = np.asarray(w, np.float32)
    n, k = w.shape
    g = w.reshape(n, k // group, group)
    wmin, wmax = g.min(-1), g.max(-1)
    scale = bf16_round((wmax - wmin) / 15.0)
    scale = np.where(scale == 0, np.float32(1.0), scale)
    bias = bf16_round(wmin)
    q = np.clip(np.rint((g - bias[..., None]) / scale[..., None]), 0, 15).astype(np.uint32)
    q = q.reshape(n, k // 8, 8)
    packed = np.zeros((n, k // 8), np.uint32)
    for j in range(8):
        packed |= q[:, :, j] << np.uint32(4 * j)
    return packed, scale, bias


def dequantize_affine4(packed: np.ndarray, scales: np.ndarray, biases: np.ndarray, group: int = 64) -> np.ndarray:
    """w = q * scale + bias (MLX "affine" mode as used by src/kvcache/quantized.zig:339-362)."""
    n, k8 = packed.shape
    q = np.stack([(packed >> np.uint32(4 * j)) & np.uint32(15) for j in range(8)], axis=-1)
    q = q.reshape(n, k8 * 8).astype(np.float32)
    return q * np.repeat(scales, group, axis=1) + np.repeat(biases, group, axis=1)


E2M1_TABLE = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                       0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)  # deepseek_v4_loader.zig:862


_E2M1_PAIRS = np.stack([E2M1_TABLE[np.arange(256) & 0x0F], E2M1_TABLE[np.arange(256) >> 4]], axis=-1)  # byte -> two values


def dequantize_mxfp4(packed: np.ndarray, scales_e8m0: np.ndarray, block: int = 32) -> np.ndarray:
    """src/models/deepseek_v4_loader.zig:858-920: each byte packs two E2M1 codes, low nibble = even
    element; one E8M0 scale 2^(s-127) per ``block`` elements (:839-856)."""
    n, k = packed.shape[0], packed.shape[1] * 2
    w = _E2M1_PAIRS[packed].reshape(n, k // block, block)  # one gather: byte -> (even element, odd element)
    sc = np.exp2(scales_e8m0.astype(np.float32) - 127.0)
    return (w * sc[:, :, None]).reshape(n, k)


def qmm(x: np.ndarray, w_deq: np.ndarray) -> np.ndarray:
    """y = x @ dequant(W)^T with fp64 accumulation (call sites src/models/llama.zig:127,367,596)."""
    return (x.astype(np.float64) @ w_deq.astype(np.float64).T).astype(np.float32)


# ---------------------------------------------------------------------------
# FP8-E4M3 KV pages with one scale per (page, kv head)  [project-defined, see module docstring]
# ---------------------------------------------------------------------------


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Saturating round-to-nearest-even float32 -> E4M3 bytes."""
    return np.clip(np.asarray(x, np.float32), -E4M3_MAX, E4M3_MAX).astype(E4M3).view(np.uint8)


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return np.asarray(b, np.uint8).view(E4M3).astype(np.float32)


def fp8_page_append(page_q: np.ndarray, scale: float, n_old: int, new_rows: np.ndarray) -> Tuple[np.ndarray, float]:
    """Append rows to one (page, head) tile of E4M3 codes.

    page_q: [page_size, D] uint8 holding n_old valid rows at scale ``scale`` (ignored if n_old=0).
    new scale = max(old scale, amax(new rows)/448) (amax floor 1e-12); when the scale grows the
    old rows are re-encoded as e4m3(decode(q) * old/new); new rows are e4m3(x / new_scale).
    """
    new_rows = np.asarray(new_rows, np.float32)
    amax = np.float32(max(float(np.abs(new_rows).max()), 1e-12))
    s_new = np.float32(amax / np.float32(E4M3_MAX))
    out = page_q.copy()
    if n_old > 0:
        s_old = np.float32(scale)
        if s_new > s_old:
            ratio = np.float32(s_old / s_new)
            out[:n_old] = e4m3_encode(e4m3_decode(out[:n_old]) * ratio)
        else:
            s_new = s_old
    inv = np.float32(1.0) / s_new
    out[n_old : n_old + len(new_rows)] = e4m3_encode(new_rows * inv)
    return out, float(s_new)


# ---------------------------------------------------------------------------
# Attention over a request's own cached rows (the B=1 oracle)
# ---------------------------------------------------------------------------


def gqa_attention_decode(q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """One query row against a request's cached K/V.

    q: [Hq, D]; k, v: [ctx, Hkv, D].  Each group of Hq/Hkv query heads reads one KV head — the
    effect of repeatHeads (src/models/llama.zig:240-241,303-323) followed by
    softmax(q k^T / sqrt(D)) v (:249-270).
    """
    hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    out = np.zeros((hq, d), np.float32)
    scale = 1.0 / np.sqrt(d)
    for h in range(hq):
        kk, vv = k[:, h // g, :], v[:, h // g, :]
        out[h] = sdpa(q[h][None, :], kk, vv, scale)[0]
    return out


# ---------------------------------------------------------------------------
# LLaMA forward at B=1 (src/models/llama.zig:138-299, 372-438, 460-481, 556-609)
# ---------------------------------------------------------------------------


@dataclass
class LlamaConfig:
    n_layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    eps: float = 1e-5
    theta: float = 10000.0


def random_llama_weights(cfg: LlamaConfig, seed: int, std: float = 0.02) -> Dict[str, np.ndarray]:
    """N(0, std) fp32 matrices, norm weights = 1 (as the reference's tiny test model,
    src/tests/e2e_tests.zig:30-80).  Values are rounded to bf16 so every implementation starts
    from identical numbers."""
    rng = np.random.default_rng(seed)
    w: Dict[str, np.ndarray] = {}

    def mat(n, k):
        return bf16_round(rng.normal(0.0, std, size=(n, k)).astype(np.float32))

    w["embed"] = mat(cfg.vocab, cfg.hidden)
    for l in range(cfg.n_layers):
        w[f"l{l}.attn_norm"] = np.ones(cfg.hidden, np.float32)
        w[f"l{l}.wq"] = mat(cfg.n_heads * cfg.head_dim, cfg.hidden)
        w[f"l{l}.wk"] = mat(cfg.n_kv_heads * cfg.head_dim, cfg.hidden)
        w[f"l{l}.wv"] = mat(cfg.n_kv_heads * cfg.head_dim, cfg.hidden)
        w[f"l{l}.wo"] = mat(cfg.hidden, cfg.n_heads * cfg.head_dim)
        w[f"l{l}.ffn_norm"] = np.ones(cfg.hidden, np.float32)
        w[f"l{l}.gate"] = mat(cfg.ffn, cfg.hidden)
        w[f"l{l}.up"] = mat(cfg.ffn, cfg.hidden)
        w[f"l{l}.down"] = mat(cfg.hidden, cfg.ffn)
    w["final_norm"] = np.ones(cfg.hidden, np.float32)
    w["lm_head"] = mat(cfg.vocab, cfg.hidden)
    return w


class LlamaB1:
    """A single request evaluated alone: the only setting in which the reference's arithmetic is
    exact and unpadded (RoPE offset is one scalar per forward, src/models/llama.zig:213; the paged
    cache concatenates per-sequence gathers along axis 0, src/kvcache/paged.zig:814-833)."""

    def __init__(self, cfg: LlamaConfig, weights: Dict[str, np.ndarray]):
        self.cfg, self.w = cfg, weights
        self.k: List[np.ndarray] = [np.zeros((0, cfg.n_kv_heads, cfg.head_dim), np.float32) for _ in range(cfg.n_layers)]
        self.v: List[np.ndarray] = [np.zeros((0, cfg.n_kv_heads, cfg.head_dim), np.float32) for _ in range(cfg.n_layers)]

    def forward(self, tokens: Sequence[int]) -> np.ndarray:
        """Append ``tokens`` (a prefill chunk or one decode token); returns last-row logits [V]."""
        c, w = self.cfg, self.w
        s = len(tokens)
        off = self.k[0].shape[0]
        pos = np.arange(off, off + s)
        x = embedding(w["embed"], np.asarray(tokens))
        for l in range(c.n_layers):
            h = rms_norm(x, w[f"l{l}.attn_norm"], c.eps)
            q = (h @ w[f"l{l}.wq"].T).reshape(s, c.n_heads, c.head_dim)
            k = (h @ w[f"l{l}.wk"].T).reshape(s, c.n_kv_heads, c.head_dim)
            v = (h @ w[f"l{l}.wv"].T).reshape(s, c.n_kv_heads, c.head_dim)
            q = rope(q.transpose(1, 0, 2), pos, c.theta).transpose(1, 0, 2)
            k = rope(k.transpose(1, 0, 2), pos, c.theta).transpose(1, 0, 2)
            self.k[l] = np.concatenate([self.k[l], k], 0)
            self.v[l] = np.concatenate([self.v[l], v], 0)
            attn = np.zeros((s, c.n_heads, c.head_dim), np.float32)
            for r in range(s):  # causal within the chunk (src/models/llama.zig:570-585)
                n_ctx = off + r + 1
                attn[r] = gqa_attention_decode(q[r], self.k[l][:n_ctx], self.v[l][:n_ctx])
            x = x + attn.reshape(s, -1) @ w[f"l{l}.wo"].T
            h = rms_norm(x, w[f"l{l}.ffn_norm"], c.eps)
            gate, up = h @ w[f"l{l}.gate"].T, h @ w[f"l{l}.up"].T
            x = x + (silu(gate) * up) @ w[f"l{l}.down"].T  # src/models/llama.zig:396-415
        h = rms_norm(x[-1:], w["final_norm"], c.eps)
        return (h @ w["lm_head"].T)[0].astype(np.float32)  # last position only (generation.zig:124-138)


# ---------------------------------------------------------------------------
# MoE (src/moe_router.zig:55-164; src/models/deepseek_v4.zig:546-681, 721-848, 947-966, 1010-1056)
# ---------------------------------------------------------------------------


def topk_route(scores_for_choice: np.ndarray, k: int) -> np.ndarray:
    """Ascending argsort, last k columns (src/moe_router.zig:59-73; deepseek_v4.zig:383-396).
    The sort is taken to be stable (MLX's tie order is not pinned by any reference test), so among
    equal scores the larger expert index wins and the output is in ascending-score order."""
    order = np.argsort(scores_for_choice, axis=-1, kind="stable")
    return order[:, -k:].astype(np.uint32)


def gate_forward(logits: np.ndarray, bias: Optional[np.ndarray], k: int, route_scale: float = 1.0,
                 scoring: str = "softmax") -> Tuple[np.ndarray, np.ndarray]:
    """DSV4Gate.forward without hash routing (deepseek_v4.zig:555-681).  logits: [N, E] f32.
    Returns (weights [N,k] f32, indices [N,k] u32)."""
    lg = logits.astype(np.float32)
    if scoring == "softmax":
        m = lg.max(-1, keepdims=True)
        e = np.exp(lg - m)
        scores = (e / e.sum(-1, keepdims=True, dtype=np.float32)).astype(np.float32)
    elif scoring == "sigmoid":
        scores = (1.0 / (1.0 + np.exp(-lg))).astype(np.float32)
    else:  # sqrtsoftplus (:566-576)
        scores = np.sqrt(np.log1p(np.exp(lg))).astype(np.float32)
    choice = scores + bias[None, :].astype(np.float32) if bias is not None else scores
    idx = topk_route(choice, k)
    wts = np.take_along_axis(scores, idx.astype(np.int64), axis=1)
    if scoring != "softmax":
        wts = wts / (wts.sum(-1, keepdims=True) + np.float32(1e-20))
    return (wts * np.float32(route_scale)).astype(np.float32), idx


def group_by_expert(indices: np.ndarray, n_experts: int):
    """deepseek_v4.zig:747-784: order = argsort(flat idx) (stable), inv = argsort(order),
    token = order // k.  Also the per-expert offsets a ragged grouped GEMM consumes."""
    flat = indices.reshape(-1).astype(np.int64)
    k = indices.shape[1]
    order = np.argsort(flat, kind="stable")
    inv = np.argsort(order, kind="stable")
    counts = np.bincount(flat, minlength=n_experts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return order.astype(np.int32), inv.astype(np.int32), (order // k).astype(np.int32), offsets


def limited_swiglu(gate: np.ndarray, up: np.ndarray, limit: float) -> np.ndarray:
    """deepseek_v4.zig:947-966: silu(min(g, L)) * clip(u, -L, L) when L > 0."""
    if limit > 0:
        g = np.minimum(gate, limit)
        u = np.clip(up, -limit, limit)
        return silu(g) * u
    return silu(gate) * up


def switch_glu(x: np.ndarray, indices: np.ndarray, scores: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray,
               w_down: np.ndarray, limit: float = 10.0) -> np.ndarray:
    """DSV4SwitchGLU.forward (deepseek_v4.zig:721-848).  w_*: dequantised [E, out, in] f32.
    The routing score multiplies the activation before the down projection (:796-805)."""
    n, k = indices.shape
    out = np.zeros((n, w_down.shape[1]), np.float64)
    for t in range(n):
        for j in range(k):
            e = int(indices[t, j])
            g = w_gate[e].astype(np.float64) @ x[t].astype(np.float64)
            u = w_up[e].astype(np.float64) @ x[t].astype(np.float64)
            a = limited_swiglu(g, u, limit) * float(scores[t, j])
            out[t] += w_down[e].astype(np.float64) @ a
    return out.astype(np.float32)


def expert_forward(x: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray, limit: float = 0.0) -> np.ndarray:
    """Shared expert (DSV4Expert.forward, deepseek_v4.zig:489-517)."""
    g = x.astype(np.float64) @ w_gate.astype(np.float64).T
    u = x.astype(np.float64) @ w_up.astype(np.float64).T
    return (limited_swiglu(g, u, limit) @ w_down.astype(np.float64).T).astype(np.float32)


def expand_tokens(x: np.ndarray, k: int) -> np.ndarray:
    """src/moe_router.zig:111-132: [N,D] -> [N*k,D]."""
    return np.repeat(x, k, axis=0)


def reduce_experts(expert_outs: np.ndarray, weights: np.ndarray) -> np.ndarray:
    """src/moe_router.zig:139-164: weighted sum over k."""
    n, k = weights.shape
    return (expert_outs.reshape(n, k, -1) * weights[:, :, None]).sum(1)
