"""CPU oracle (test infrastructure only) for the samplers of src/sampling.zig, in f32 like the reference.

Every running sum is numpy's float32 cumsum, which adds left to right exactly as the reference's
loops do.  exp() is numpy's float32 exp; Zig's @exp may differ from it in the last bit, so each
function also returns a *margin*: how close the uniform variate (or top_p) came to the cumulative
value that decided the outcome.  A checker accepts a different token only when that margin is
within rounding.

Parity: the reference holds no golden vectors for its samplers (its tests use temperature 0 or
check shapes only), so this restatement is pinned on hand-computed cases in tests/test_sampling.py
and is otherwise unpinned.  The PRNG below restates two published algorithms of the Zig 0.16 standard
library the reference builds against (std.Random.DefaultPrng = xoshiro256++ seeded by SplitMix64,
and Random.float(f32)); the standard library is not part of the reference tree, and no Zig toolchain
exists here to run it: pinned on the xoshiro256++ / SplitMix64 known-answer vectors only.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np

F = np.float32
M64 = (1 << 64) - 1


def greedy(logits: np.ndarray) -> int:
    """First strict maximum (src/sampling.zig:22-39)."""
    return int(np.argmax(logits))  # numpy returns the first maximum too


def sample_from_probs(probs: np.ndarray, r: float) -> Tuple[int, float]:
    """src/sampling.zig:258-268: first i with r < cumsum(probs)[i], else n - 1."""
    cum = np.cumsum(probs.astype(F), dtype=F)
    hit = np.nonzero(F(r) < cum)[0]
    idx = int(hit[0]) if len(hit) else len(probs) - 1
    near = cum[max(idx - 1, 0) : idx + 1]
    return idx, float(np.abs(near.astype(np.float64) - float(F(r))).min())


def temperature_sample(logits: np.ndarray, temperature: float, r: float) -> Tuple[int, float]:
    """src/sampling.zig:42-72."""
    if temperature <= 0.0:
        return greedy(logits), 1.0
    x = logits.astype(F)
    e = np.exp((x - x.max()) / F(temperature)).astype(F)
    total = np.cumsum(e, dtype=F)[-1]
    return sample_from_probs(e / total, r)


def top_k_top_p(logits: np.ndarray, temperature: float, k: int, p: float, r: float) -> Tuple[int, float]:
    """src/sampling.zig:175-242.  k <= 0 stands for the whole vocabulary."""
    if temperature <= 0.0:
        return greedy(logits), 1.0
    x = logits.astype(F)
    scores = x / F(temperature)
    order = np.argsort(-scores, kind="stable")  # the reference's insertion sort is stable (:197)
    k_actual = len(x) if k <= 0 else min(k, len(x))
    top = scores[order[:k_actual]]
    e = np.exp(top - top[0]).astype(F)
    probs = e / np.cumsum(e, dtype=F)[-1]
    cum = np.cumsum(probs, dtype=F)
    over = np.nonzero(cum > F(p))[0]
    cutoff = int(over[0]) + 1 if len(over) else k_actual
    near = cum[max(cutoff - 2, 0) : cutoff]
    margin_p = float(np.abs(near.astype(np.float64) - float(F(p))).min()) if cutoff < k_actual or len(over) else 1.0
    nucleus = probs[:cutoff] / cum[cutoff - 1]  # the reference re-adds the same terms in the same order
    idx, margin_r = sample_from_probs(nucleus, r)
    return int(order[idx]), min(margin_p, margin_r)


def apply_repetition_penalty(logits: np.ndarray, context: Sequence[int], penalty: float) -> np.ndarray:
    """src/sampling.zig:328-354: once per occurrence."""
    out = logits.astype(F).copy()
    for t in context:
        if t < len(out):
            out[t] = out[t] / F(penalty) if out[t] > 0 else out[t] * F(penalty)
    return out


def logprob(logits: np.ndarray, token: int) -> float:
    """src/sampling.zig:355-375."""
    x = logits.astype(F)
    m = x.max()
    s = np.cumsum(np.exp(x - m).astype(F), dtype=F)[-1]
    return float(x[token] - (m + np.log(s)))


def sampler_config_sample(logits: np.ndarray, temperature: float, top_k: int, top_p: float, r: float,
                          repetition_penalty: float = 1.0, context: Optional[Sequence[int]] = None):
    """SamplerConfig.sample (src/sampling.zig:298-322) -> (token, logprob, margin)."""
    x = logits.astype(F)
    if repetition_penalty > 1.0 and context is not None and len(context) > 0:
        x = apply_repetition_penalty(x, context, repetition_penalty)
    if temperature <= 0.0:
        tok, margin = greedy(x), 1.0
    elif top_p >= 1.0 and (top_k <= 0 or top_k >= len(x)):
        tok, margin = temperature_sample(x, temperature, r)
    else:
        tok, margin = top_k_top_p(x, temperature, top_k, top_p, r)
    return tok, logprob(x, tok), margin


class Xoshiro256:
    """xoshiro256++ seeded through SplitMix64, as std.Random.DefaultPrng.init(seed) does."""

    def __init__(self, seed: int):
        sm = seed & M64
        self.s = []
        for _ in range(4):
            sm = (sm + 0x9E3779B97F4A7C15) & M64
            z = sm
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
            self.s.append(z ^ (z >> 31))

    @staticmethod
    def _rotl(x: int, k: int) -> int:
        return ((x << k) | (x >> (64 - k))) & M64

    def next_u64(self) -> int:
        s = self.s
        r = (self._rotl((s[0] + s[3]) & M64, 23) + s[0]) & M64
        t = (s[1] << 17) & M64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return r

    def next_f32(self) -> float:
        """Random.float(f32): 23 mantissa bits, exponent lowered by the leading-zero count."""
        def clz(x: int, bits: int) -> int:
            return bits - x.bit_length()

        r = self.next_u64()
        lz = clz(r, 64)
        if lz >= 41:
            lz = 41 + clz(self.next_u64(), 64)
            if lz == 41 + 64:
                lz += clz((self.next_u64() & 0xFFFFFFFF) | 0x7FF, 32)
        bits = ((126 - lz) << 23) | (r & 0x7FFFFF)
        return float(np.array([bits], np.uint32).view(np.float32)[0])


def acceptable_tokens(logits: np.ndarray, temperature: float, top_k: int, top_p: float, r: float, tol: float,
                      repetition_penalty: float = 1.0, context: Optional[Sequence[int]] = None) -> set:
    """Tokens SamplerConfig.sample could return if every cumulative sum were perturbed by at most
    `tol`: the exact answer, plus a neighbour when r (or top_p) lies within tol of the cumulative value
    that separates them.  With tol = 0 this is {the oracle's token}."""
    x = logits.astype(F)
    if repetition_penalty > 1.0 and context is not None and len(context) > 0:
        x = apply_repetition_penalty(x, context, repetition_penalty)
    if temperature <= 0.0:
        return {greedy(x)}
    r = float(F(r))

    def owners(cum: np.ndarray, order: np.ndarray) -> set:
        c = cum.astype(np.float64)
        lo = np.concatenate([[-np.inf], c[:-1]])
        hi = c.copy()
        hi[-1] = np.inf  # the last candidate takes everything above (:267)
        ok = (r >= lo - tol) & (r < hi + tol)
        return {int(t) for t in order[np.nonzero(ok)[0]]}

    if top_p >= 1.0 and (top_k <= 0 or top_k >= len(x)):
        e = np.exp((x - x.max()) / F(temperature)).astype(F)
        probs = e / np.cumsum(e, dtype=F)[-1]
        return owners(np.cumsum(probs, dtype=F), np.arange(len(x)))
    scores = x / F(temperature)
    order = np.argsort(-scores, kind="stable")
    k_actual = len(x) if top_k <= 0 else min(top_k, len(x))
    top = scores[order[:k_actual]]
    e = np.exp(top - top[0]).astype(F)
    probs = e / np.cumsum(e, dtype=F)[-1]
    cum = np.cumsum(probs, dtype=F)
    c64 = cum.astype(np.float64)
    cutoffs = {int(i) + 1 for i in np.nonzero(np.abs(c64 - float(F(top_p))) <= tol)[0]}
    cutoffs |= {min(c + 1, k_actual) for c in list(cutoffs)}
    over = np.nonzero(cum > F(top_p))[0]
    cutoffs.add(int(over[0]) + 1 if len(over) else k_actual)
    out = set()
    for c in cutoffs:
        nucleus = probs[:c] / cum[c - 1]
        out |= owners(np.cumsum(nucleus, dtype=F), order[:c])
    return out
