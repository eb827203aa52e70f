"""GPU parity: split-K GQA paged-attention decode against the per-request oracle
(softmax(q k^T / sqrt(D)) v over the request's own cached rows, src/models/llama.zig:231-270).

Tolerance (bf16 outputs): max |diff| / max |ref| <= 2e-2 and cosine >= 0.9995."""
import numpy as np
import pytest
import torch

from oracle import ref_math

pytestmark = pytest.mark.gpu

REL_TOL, COS_TOL = 2e-2, 0.9995


def _close(got, want):
    g, w = got.astype(np.float64).reshape(-1), want.astype(np.float64).reshape(-1)
    rel = np.abs(g - w).max() / max(np.abs(w).max(), 1e-30)
    cos = g @ w / (np.linalg.norm(g) * np.linalg.norm(w) + 1e-30)
    return rel, cos


def _run_case(ctxs, hq, hkv, d, kv_dtype, seed, scatter=True, pages_per_chunk=0, path=0):
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(seed)
    n = len(ctxs)
    pages = sum(-(-c // 32) for c in ctxs)
    n_pages = int(pages * 1.25) + 2
    kv = dev.PagedKVCache(1, hkv, d, n_pages, n, max(-(-max(ctxs) // 32), 1), hq, max_rows=max(sum(ctxs), n, 1),
                          kv_dtype=kv_dtype)
    dev.set_attn_pages_per_chunk(pages_per_chunk)
    dev.set_attn_path(path)
    if scatter:
        kv.set_free_order(rng.permutation(n_pages).tolist())
    k = ref_math.bf16_round(rng.normal(0, 1, (sum(ctxs), hkv, d)).astype(np.float32))
    v = ref_math.bf16_round(rng.normal(0, 1, (sum(ctxs), hkv, d)).astype(np.float32))
    q = ref_math.bf16_round((rng.normal(0, 1, (n, hq, d)) / np.sqrt(d)).astype(np.float32) * np.sqrt(d))
    desc = dev.pack_desc_array([(s, c, 0, -1) for s, c in enumerate(ctxs)]).cuda()
    kv.reserve(desc)
    kv.append(0, torch.tensor(k, device="cuda").bfloat16(), torch.tensor(v, device="cuda").bfloat16())
    row_seq = torch.arange(n, dtype=torch.int32, device="cuda")
    row_ctx = torch.tensor(ctxs, dtype=torch.int32, device="cuda")
    out = kv.attention(0, torch.tensor(q, device="cuda").bfloat16(), row_seq, row_ctx)
    torch.cuda.synchronize()
    assert kv.error_word() == 0
    got = out.float().cpu().numpy()
    if kv_dtype == dev.KV_FP8_E4M3:
        # the oracle for FP8 pools reads what the pool holds: decode(codes) * scale
        kk, vv = [], []
        for s in range(n):
            a, b = kv.gather(0, s)
            kk.append(a.float().cpu().numpy())
            vv.append(b.float().cpu().numpy())
        k_eff, v_eff = np.concatenate(kk) if sum(ctxs) else k, np.concatenate(vv) if sum(ctxs) else v
    else:
        k_eff, v_eff = k, v
    off = 0
    want = np.zeros_like(got)
    for s, c in enumerate(ctxs):
        if c > 0:
            want[s] = ref_math.gqa_attention_decode(q[s], k_eff[off : off + c], v_eff[off : off + c])
        off += c
    kv.close()
    dev.set_attn_path(0)
    dev.set_attn_pages_per_chunk(0)   # back to the automatic choice
    return got, want, (k, v, q)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("kv_dtype,path", [(0, 0), (0, 1), (1, 0), (1, 1)])  # bf16 tensor-core, bf16 CUDA-core, FP8 tensor-core (head_dim 128), FP8 CUDA-core
def test_ragged_contexts(d, kv_dtype, path):
    ctxs = [1, 31, 32, 33, 64, 65, 200, 257, 700, 5, 1023, 96]
    hq, hkv = (8, 2) if d == 64 else (32, 8)
    got, want, _ = _run_case(ctxs, hq, hkv, d, kv_dtype, seed=7 + d + kv_dtype, path=path)
    rel, cos = _close(got, want)
    assert rel <= REL_TOL and cos >= COS_TOL, (rel, cos)
    for s in range(len(ctxs)):  # every row on its own, so a short context cannot hide behind a long one
        r, c = _close(got[s], want[s])
        assert r <= REL_TOL and c >= COS_TOL, (s, ctxs[s], r, c)


def test_fp8_close_to_bf16_oracle():
    """FP8 pools against the bf16 (unquantised) oracle: the quantisation error itself stays inside
    the tolerance the north-star states for bf16 outputs."""
    from dmlx_b200 import device as dev

    ctxs = [300, 1024, 77]
    got, _, (k, v, q) = _run_case(ctxs, 32, 8, 128, dev.KV_FP8_E4M3, seed=99)
    off = 0
    for s, c in enumerate(ctxs):
        want = ref_math.gqa_attention_decode(q[s], k[off : off + c], v[off : off + c])
        rel, cos = _close(got[s], want)
        assert rel <= 6e-2 and cos >= 0.998, (s, rel, cos)  # E4M3 carries 3 mantissa bits
        off += c


@pytest.mark.parametrize("ppc", [4, 8, 32])
@pytest.mark.parametrize("path", [0, 1])
def test_split_sizes_agree(ppc, path):
    got, want, _ = _run_case([2000, 40, 513], 32, 8, 128, 0, seed=5, pages_per_chunk=ppc, path=path)
    rel, cos = _close(got, want)
    assert rel <= REL_TOL and cos >= COS_TOL


def test_gqa_group_sizes_tensor_core_path():
    """The tensor-core kernel takes the group's query heads as MMA rows: groups of 1, 2 and 8."""
    for hq, hkv in ((2, 2), (4, 2), (16, 2)):
        got, want, _ = _run_case([130, 31, 64], hq, hkv, 128, 0, seed=hq)
        rel, cos = _close(got, want)
        assert rel <= REL_TOL and cos >= COS_TOL, (hq, hkv, rel, cos)


def test_empty_context_row_is_zero():
    got, want, _ = _run_case([0, 40], 8, 2, 64, 0, seed=3)
    assert np.all(got[0] == 0)
    rel, cos = _close(got[1], want[1])
    assert rel <= REL_TOL and cos >= COS_TOL


def test_prefill_rows_as_causal_decode_rows():
    """A prefill chunk is served by giving each row its causal context (position + 1): row r of a
    request sees only its first r+1 tokens — the block-diagonal causal mask of
    src/batch_builder.zig:168-177 without materialising it."""
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(21)
    hq, hkv, d, n_tok = 8, 2, 64, 70
    kv = dev.PagedKVCache(1, hkv, d, 8, 1, 4, hq, max_rows=128, attn_scratch_chunks=256)
    k = ref_math.bf16_round(rng.normal(0, 1, (n_tok, hkv, d)).astype(np.float32))
    v = ref_math.bf16_round(rng.normal(0, 1, (n_tok, hkv, d)).astype(np.float32))
    q = ref_math.bf16_round(rng.normal(0, 1, (n_tok, hq, d)).astype(np.float32))
    kv.reserve(dev.pack_desc_array([(0, n_tok, 0, -1)]).cuda())
    kv.append(0, torch.tensor(k, device="cuda").bfloat16(), torch.tensor(v, device="cuda").bfloat16())
    row_seq = torch.zeros(n_tok, dtype=torch.int32, device="cuda")
    row_ctx = torch.arange(1, n_tok + 1, dtype=torch.int32, device="cuda")
    got = kv.attention(0, torch.tensor(q, device="cuda").bfloat16(), row_seq, row_ctx).float().cpu().numpy()
    assert kv.error_word() == 0
    for r in range(n_tok):
        want = ref_math.gqa_attention_decode(q[r], k[: r + 1], v[: r + 1])
        rel, cos = _close(got[r], want)
        assert rel <= REL_TOL and cos >= COS_TOL, (r, rel, cos)


@pytest.mark.parametrize("hq,hkv,d,kv_dtype", [(8, 2, 64, 0), (32, 8, 128, 0), (16, 2, 128, 0), (4, 4, 64, 0),
                                                (32, 8, 128, 1), (16, 2, 128, 1)])
def test_prefill_groups_match_oracle_and_row_kernel(hq, hkv, d, kv_dtype):
    """b200_paged_attn_prefill on a mixed batch: prefill chunks that start in the middle of a cached
    prefix (src/scheduler.zig:183-186 chunk cursor), chunks of 1..70 rows, and plain decode rows.
    Every row equals the oracle on its causal prefix, and the per-row kernel on the same inputs."""
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(5 + hq + d)
    # (cached tokens before the chunk, rows in the chunk)
    reqs = [(0, 70), (100, 33), (37, 1), (250, 5), (0, 1), (64, 16), (31, 2), (500, 1)]
    totals = [c + n for c, n in reqs]
    n_pages = sum(-(-t // 32) for t in totals) + 4
    n_rows = sum(n for _, n in reqs)
    kv = dev.PagedKVCache(1, hkv, d, n_pages, len(reqs), max(-(-max(totals) // 32), 1), hq, max_rows=max(totals) + n_rows,
                          attn_scratch_chunks=4096, kv_dtype=kv_dtype)
    kv.set_free_order(rng.permutation(n_pages).tolist())
    ks = [ref_math.bf16_round(rng.normal(0, 1, (t, hkv, d)).astype(np.float32)) for t in totals]
    vs = [ref_math.bf16_round(rng.normal(0, 1, (t, hkv, d)).astype(np.float32)) for t in totals]
    kv.reserve(dev.pack_desc_array([(s, t, 0, -1) for s, t in enumerate(totals)]).cuda())
    kv.append(0, torch.tensor(np.concatenate(ks), device="cuda").bfloat16(), torch.tensor(np.concatenate(vs), device="cuda").bfloat16())
    if kv_dtype != 0:  # the oracle for FP8 pools reads what the pool holds: decode(codes) * scale
        eff = [kv.gather(0, s) for s in range(len(reqs))]
        ks = [a.float().cpu().numpy() for a, _ in eff]
        vs = [b.float().cpu().numpy() for _, b in eff]
    q = ref_math.bf16_round(rng.normal(0, 1, (n_rows, hq, d)).astype(np.float32))
    row_seq = np.concatenate([np.full(n, s, np.int32) for s, (_, n) in enumerate(reqs)])
    row_ctx = np.concatenate([np.arange(c + 1, c + n + 1, dtype=np.int32) for c, n in reqs])
    qd, rs, rc = torch.tensor(q, device="cuda").bfloat16(), torch.tensor(row_seq, device="cuda"), torch.tensor(row_ctx, device="cuda")
    got = kv.attention(0, qd, rs, rc, prefill=True).float().cpu().numpy()
    per_row = kv.attention(0, qd, rs, rc).float().cpu().numpy()
    assert kv.error_word() == 0
    for r in range(n_rows):
        s, c = int(row_seq[r]), int(row_ctx[r])
        want = ref_math.gqa_attention_decode(q[r], ks[s][:c], vs[s][:c])
        rel, cos = _close(got[r], want)
        assert rel <= REL_TOL and cos >= COS_TOL, (r, s, c, rel, cos)
    assert np.abs(got - per_row).max() <= 2e-2 * np.abs(per_row).max()  # both kernels read the same pool
    kv.close()


@pytest.mark.parametrize("hq,hkv,d,kv_dtype", [(32, 8, 128, 0), (32, 8, 128, 1), (8, 2, 64, 0)])
def test_prefill_batches_of_1024_rows_and_more_write_their_rows_directly(hq, hkv, d, kv_dtype):
    """From 1024 rows on b200_paged_attn_prefill gives every group of rows one chunk as long as its context
    and the kernel normalises and writes the rows itself.  Chunks that start inside a cached prefix, contexts
    over more than 32 pages, plus decode rows in the same batch.  A sample of rows against the oracle, every
    row against the chunked path (partials + combine pass) on the same pool."""
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(91 + hq + d + kv_dtype)
    reqs = [(0, 520), (700, 333), (1500, 1), (64, 200), (2100, 1), (31, 47)]   # 1102 rows
    totals = [c + n for c, n in reqs]
    n_pages = sum(-(-t // 32) for t in totals) + 4
    n_rows = sum(n for _, n in reqs)
    assert n_rows >= 1024
    kv = dev.PagedKVCache(1, hkv, d, n_pages, len(reqs), -(-max(totals) // 32), hq, max_rows=max(totals) + n_rows,
                          attn_scratch_chunks=8192, kv_dtype=kv_dtype)
    kv.set_free_order(rng.permutation(n_pages).tolist())
    ks = [ref_math.bf16_round(rng.normal(0, 1, (t, hkv, d)).astype(np.float32)) for t in totals]
    vs = [ref_math.bf16_round(rng.normal(0, 1, (t, hkv, d)).astype(np.float32)) for t in totals]
    kv.reserve(dev.pack_desc_array([(s, t, 0, -1) for s, t in enumerate(totals)]).cuda())
    kv.append(0, torch.tensor(np.concatenate(ks), device="cuda").bfloat16(), torch.tensor(np.concatenate(vs), device="cuda").bfloat16())
    if kv_dtype != 0:
        eff = [kv.gather(0, s) for s in range(len(reqs))]
        ks = [a.float().cpu().numpy() for a, _ in eff]
        vs = [b.float().cpu().numpy() for _, b in eff]
    q = ref_math.bf16_round(rng.normal(0, 1, (n_rows, hq, d)).astype(np.float32))
    row_seq = np.concatenate([np.full(n, s, np.int32) for s, (_, n) in enumerate(reqs)])
    row_ctx = np.concatenate([np.arange(c + 1, c + n + 1, dtype=np.int32) for c, n in reqs])
    qd, rs, rc = torch.tensor(q, device="cuda").bfloat16(), torch.tensor(row_seq, device="cuda"), torch.tensor(row_ctx, device="cuda")
    launches = dev.launch_count()
    got = kv.attention(0, qd, rs, rc, prefill=True).float().cpu().numpy()
    direct_launches = dev.launch_count() - launches
    assert kv.error_word() == 0
    try:
        dev.set_attn_prefill_direct(False)
        launches = dev.launch_count()
        chunked = kv.attention(0, qd, rs, rc, prefill=True).float().cpu().numpy()
        assert dev.launch_count() - launches == direct_launches + 1   # the combine pass
    finally:
        dev.set_attn_prefill_direct(True)
    assert kv.error_word() == 0
    assert np.abs(got - chunked).max() <= 1e-2 * np.abs(chunked).max()
    for r in list(range(0, n_rows, 37)) + [519, 520, 852, 853, 854, 1053, 1054, n_rows - 1]:
        s, c = int(row_seq[r]), int(row_ctx[r])
        want = ref_math.gqa_attention_decode(q[r], ks[s][:c], vs[s][:c])
        rel, cos = _close(got[r], want)
        assert rel <= REL_TOL and cos >= COS_TOL, (r, s, c, rel, cos)
    kv.close()


@pytest.mark.parametrize("ctxs,forced", [([300, 70, 1500, 33], 8), ([4100, 3900, 4200, 3500], 16), ([9000, 7000, 8100], 32)])
@pytest.mark.parametrize("kv_dtype", [0, 1])
def test_chunk_length_chosen_on_the_device_equals_the_forced_one(ctxs, forced, kv_dtype):
    """With the tuning hook at 0 the plan kernel picks 8, 16 or 32 pages per chunk from the batch's mean context
    (below 96 pages per row, below 192, above).  The outputs must be the bits of a run with that length forced,
    and match the oracle."""
    auto, want, _ = _run_case(ctxs, 32, 8, 128, kv_dtype, seed=7 + forced)
    same, _, _ = _run_case(ctxs, 32, 8, 128, kv_dtype, seed=7 + forced, pages_per_chunk=forced)
    assert np.array_equal(auto, same)
    other, _, _ = _run_case(ctxs, 32, 8, 128, kv_dtype, seed=7 + forced, pages_per_chunk=4)
    assert not np.array_equal(auto, other) or len(ctxs) == 0   # another split order rounds differently somewhere
    for s in range(len(ctxs)):
        r, c = _close(auto[s], want[s])
        assert r <= REL_TOL and c >= COS_TOL, (s, ctxs[s], r, c)


@pytest.mark.parametrize("kv_dtype", [0, 1])  # bf16 pool, FP8-E4M3 pool (tensor-core kernels, head_dim 128)
def test_long_contexts_of_the_attention_microbench(kv_dtype):
    """Three sequences drawn from the attention microbench's range (log-uniform 128..32768 tokens, 32
    query / 8 KV heads, head_dim 128), one of them at the maximum of 32768 tokens = 1024 pages = 128
    split-K chunks, pages scattered over a pool sized to the pages x 1.25.  Per row against the
    per-request oracle; for the FP8 pool the oracle reads what the pool holds (codes x scale)."""
    ctxs = [32768, 4127, 128]
    got, want, _ = _run_case(ctxs, 32, 8, 128, kv_dtype, seed=2048 + kv_dtype)
    for s in range(len(ctxs)):
        r, c = _close(got[s], want[s])
        assert r <= REL_TOL and c >= COS_TOL, (s, ctxs[s], r, c)
