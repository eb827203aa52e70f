"""Pins the floating-point oracle against the reference's own golden vectors
(src/tests/golden/*.bin, produced by tests/generate_golden.py with Python MLX) to the
reference's thresholds: cosine >= 0.9999 and |diff| <= 1e-4 (src/tests/golden_test.zig:35-48,
298-300).  Also self-consistency checks for the formats no reference test pins."""
import json
import os

import numpy as np

from oracle import ref_math as M

G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    meta = json.load(open(os.path.join(G, name + ".bin.json")))
    dt = {"float32": "<f4", "int32": "<i4"}[meta["dtype"]]
    return np.fromfile(os.path.join(G, name + ".bin"), dtype=dt).reshape(meta["shape"])


def close(a, b):
    a, b = a.reshape(-1).astype(np.float64), b.reshape(-1).astype(np.float64)
    cos = a @ b / (np.linalg.norm(a) * np.linalg.norm(b))
    return cos >= 0.9999 and np.abs(a - b).max() <= 1e-4


def test_rmsnorm_golden():  # generate_golden.py:62-72
    x = load("rmsnorm_input")
    assert close(M.rms_norm(x, np.ones(x.shape[-1], np.float32), 1e-5), load("rmsnorm_output"))


def test_rope_golden():  # generate_golden.py:75-83: dims=8, traditional=False, base 1e4, offset 0
    x = load("rope_input")  # (1,2,4,8): positions run along axis -2
    assert close(M.rope(x, np.arange(x.shape[-2]), 10000.0), load("rope_output"))


def test_sdpa_golden():  # generate_golden.py:86-99
    q, k, v = load("sdpa_q"), load("sdpa_k"), load("sdpa_v")
    assert close(M.sdpa(q, k, v, 1.0 / np.sqrt(8.0)), load("sdpa_output"))


def test_embedding_golden():  # generate_golden.py:102-112
    assert np.array_equal(M.embedding(load("embedding_weight"), load("embedding_indices")), load("embedding_output"))


def test_gqa_decode_equals_sdpa_on_golden():
    """The per-request decode attention used as the paged-attention oracle reduces to the pinned
    sdpa when there is one head: last query row against all keys."""
    q, k, v = load("sdpa_q")[0, 0], load("sdpa_k")[0, 0], load("sdpa_v")[0, 0]
    full = M.sdpa(q, k, v, 1.0 / np.sqrt(8.0))
    for r in range(4):
        got = M.gqa_attention_decode(q[r][None, :], k[:, None, :], v[:, None, :])
        assert np.allclose(got[0], full[r], atol=1e-6)


def test_affine4_roundtrip():  # kvcache_tests.zig:1681-1741 (Property 10): 4-bit cosine >= 0.95
    rng = np.random.default_rng(10)
    for _ in range(20):
        w = rng.normal(0, 1, (8, 128)).astype(np.float32)
        p, s, b = M.quantize_affine4(w)
        assert p.dtype == np.uint32 and p.shape == (8, 16) and s.shape == (8, 2)
        d = M.dequantize_affine4(p, s, b)
        cos = (w.reshape(-1) @ d.reshape(-1)) / (np.linalg.norm(w) * np.linalg.norm(d))
        assert cos >= 0.95
        assert np.abs(w - d).max() <= 0.6 * s.max()


def test_mxfp4_table_and_scale():  # deepseek_v4_loader.zig:839-920
    packed = np.array([[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE] + [0] * 8], np.uint8)  # 32 elems
    sc = np.array([[128]], np.uint8)  # 2^(128-127) = 2
    w = M.dequantize_mxfp4(packed, sc)
    assert w[0, :16].tolist() == [0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12]


def test_fp8_page_append_monotone_scale():
    rng = np.random.default_rng(5)
    page = np.zeros((32, 16), np.uint8)
    rows = rng.normal(0, 1, (32, 16)).astype(np.float32)
    rows[20] *= 8.0  # forces a rescale mid-page
    scale, n = 0.0, 0
    for r in range(32):
        page, s2 = M.fp8_page_append(page, scale, n, rows[r : r + 1])
        assert s2 >= scale
        scale, n = s2, n + 1
    deq = M.e4m3_decode(page) * scale
    assert np.abs(deq - rows).max() <= 0.07 * np.abs(rows).max()


def test_topk_and_grouping():  # moe_router.zig:169-439 (set/weights properties); deepseek_v4.zig:747-784
    rng = np.random.default_rng(18)
    logits = rng.normal(0, 1, (64, 16)).astype(np.float32)
    bias = rng.normal(0, 0.1, 16).astype(np.float32)
    w, idx = M.gate_forward(logits, bias, 4, route_scale=2.0)
    assert idx.shape == (64, 4) and w.shape == (64, 4)
    sm = np.exp(logits - logits.max(-1, keepdims=True))
    sm /= sm.sum(-1, keepdims=True)
    for t in range(64):
        chosen = set(idx[t].tolist())
        assert len(chosen) == 4
        ranked = np.argsort(sm[t] + bias, kind="stable")[-4:]
        assert idx[t].tolist() == ranked.tolist()
        assert np.allclose(w[t], 2.0 * sm[t][idx[t]], rtol=1e-5)
    order, inv, tok, offs = M.group_by_expert(idx, 16)
    flat = idx.reshape(-1)
    assert np.all(np.diff(flat[order].astype(np.int64)) >= 0) and np.array_equal(order[inv], np.arange(256))
    assert offs[-1] == 256 and np.array_equal(tok, order // 4)
    # ties: the larger index wins and comes last (stable ascending sort, last k)
    assert M.topk_route(np.zeros((1, 8), np.float32), 3).tolist() == [[5, 6, 7]]


def test_reduce_experts_matches_switch_glu_sum():  # moe_router.zig:111-164
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, (5, 8)).astype(np.float32)
    assert M.expand_tokens(x, 3).shape == (15, 8)
    outs = rng.normal(0, 1, (15, 8)).astype(np.float32)
    w = rng.random((5, 3)).astype(np.float32)
    r = M.reduce_experts(outs, w)
    assert np.allclose(r[2], sum(w[2, j] * outs[6 + j] for j in range(3)), atol=1e-6)


def test_llama_b1_chunked_equals_whole():
    """Prefilling in chunks gives the same logits as prefilling at once (the property chunked
    prefill relies on, src/scheduler.zig:262-266)."""
    cfg = M.LlamaConfig(2, 32, 4, 2, 8, 64, 50)
    w = M.random_llama_weights(cfg, 1)
    toks = [3, 7, 11, 2, 9, 30, 1]
    a = M.LlamaB1(cfg, w).forward(toks)
    m = M.LlamaB1(cfg, w)
    m.forward(toks[:3])
    m.forward(toks[3:5])
    b = m.forward(toks[5:])
    assert np.allclose(a, b, atol=1e-5)
