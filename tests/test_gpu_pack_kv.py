"""GPU parity: ragged packing and the device page pool, bit-exact against the integer oracle.

All calls go through the C-ABI (dmlx_b200.device is a ctypes shim)."""
import numpy as np
import pytest
import torch

from oracle import ref_host, ref_math

pytestmark = pytest.mark.gpu


def _dev():
    from dmlx_b200 import device

    return device


def _desc(dev, rows):
    return dev.pack_desc_array(rows).cuda(non_blocking=True)


def test_pack_matches_batch_builder():
    """cu_seqlens / positions / tokens equal batch_builder.build on the same schedule
    (src/batch_builder.zig:90-214); 50 random mixed prefill+decode schedules."""
    dev = _dev()
    rng = np.random.default_rng(101)
    for _ in range(50):
        n_pre, n_dec = int(rng.integers(0, 5)), int(rng.integers(0, 9))
        if n_pre + n_dec == 0:
            n_dec = 1
        pre, dec, descs, flat = [], [], [], []
        last_token = np.zeros(64, np.uint32)
        slot = 0
        for i in range(n_pre):
            prompt = rng.integers(0, 32000, int(rng.integers(1, 40))).tolist()
            off = int(rng.integers(0, len(prompt)))
            r = ref_host.Request(i, prompt, 10)
            r.force_state(ref_host.PREFILLING, off, [])
            pre.append(r)
            descs.append((slot, len(prompt) - off, off, len(flat)))
            flat.extend(prompt[off:])
            slot += 1
        for i in range(n_dec):
            prompt = rng.integers(0, 32000, int(rng.integers(1, 40))).tolist()
            gen = rng.integers(0, 32000, int(rng.integers(1, 6))).tolist()
            r = ref_host.Request(100 + i, prompt, 10)
            r.force_state(ref_host.DECODING, len(prompt), gen)
            dec.append(r)
            last_token[slot] = gen[-1]
            descs.append((slot, 1, len(prompt) + len(gen) - 1, -1))
            slot += 1
        want = ref_host.build_batch(ref_host.ScheduleResult(pre, dec, 0), with_mask=False)
        d_flat = torch.tensor(np.array(flat + [0], np.int64).astype(np.int32), device="cuda")
        d_last = torch.tensor(last_token.astype(np.int32), device="cuda")
        got = dev.pack_batch(_desc(dev, descs), want.total_tokens, d_flat, d_last)
        t = want.total_tokens
        assert got.cu_seqlens.cpu().numpy().tolist() == want.cu_seqlens.tolist()
        assert got.token_ids[:t].cpu().numpy().astype(np.uint32).tolist() == want.batched_tokens.tolist()
        assert got.position_ids[:t].cpu().numpy().tolist() == want.position_ids.tolist()
        assert got.row_to_req[:t].cpu().numpy().tolist() == want.row_to_req.tolist()
        assert got.row_ctx[:t].cpu().numpy().tolist() == (want.position_ids + 1).tolist()
        assert got.last_row.cpu().numpy()[: len(descs)].tolist() == (want.cu_seqlens[1:] - 1).tolist()


def _check_tables(kv, ref, n_seqs):
    assert kv.free_count() == ref.free_count()
    for s in range(n_seqs):
        assert kv.block_table(s) == ref.tables[s], f"seq {s}"
        assert kv.seq_len(s) == ref.lens[s]
    assert kv.ref_counts().tolist() == ref.ref


def test_pool_random_workload_bit_exact():
    """Block tables, ref-counts and free count follow the LIFO allocator of paged.BlockManager
    (src/kvcache/paged.zig:61-73,116-118,142-162,167-206) through random multi-step workloads with
    growth, release, prefix fork + copy-on-write and rollback."""
    dev = _dev()
    rng = np.random.default_rng(202)
    for trial in range(6):
        n_pages, n_seqs = int(rng.integers(40, 200)), 12
        kv = dev.PagedKVCache(1, 2, 64, n_pages, n_seqs, 64, 8, max_rows=4096)
        ref = ref_host.PagedKVTables(n_pages, n_seqs)
        if trial % 2 == 1:  # scattered pool: random pop order
            order = rng.permutation(n_pages).tolist()
            kv.set_free_order(order)
            ref.free = order[::-1]
        live = set()
        for step in range(60):
            op = rng.random()
            if op < 0.55:
                seqs = [s for s in rng.permutation(n_seqs)[: int(rng.integers(1, 7))].tolist()]
                counts = [int(rng.integers(1, 70)) if s not in live else int(rng.integers(1, 4)) for s in seqs]
                counts = [min(c, 64 * 32 - ref.lens[s]) for s, c in zip(seqs, counts)]
                try:
                    ref.reserve(seqs, counts)
                    expect_err = 0
                except ref_host.InsufficientBlocks:
                    expect_err = 1
                kv.reserve(_desc(dev, [(s, c, 0, -1) for s, c in zip(seqs, counts)]))
                assert kv.error_word() == expect_err
                if not expect_err:
                    live.update(seqs)
            elif op < 0.7 and live:
                s = int(rng.choice(sorted(live)))
                ref.release(s)
                kv.release([s])
                live.discard(s)
            elif op < 0.85 and live:
                free_slots = [s for s in range(n_seqs) if s not in live and not ref.tables[s]]
                src = int(rng.choice(sorted(live)))
                if free_slots and ref.lens[src] > 0:
                    dst, nt = free_slots[0], int(rng.integers(1, ref.lens[src] + 1))
                    ref.fork(src, dst, nt)
                    kv.fork(src, dst, nt)
                    live.add(dst)
            elif live:
                s = int(rng.choice(sorted(live)))
                to = int(rng.integers(0, ref.lens[s] + 1))
                ref.rollback(s, to)
                kv.rollback(s, to)
            _check_tables(kv, ref, n_seqs)
        kv.close()


def test_cow_two_sharers_same_step():
    """Two sequences that share a partially filled page and both append in one step: the first
    (in batch order) takes a private copy, the second keeps the original (paged.zig:167-206)."""
    dev = _dev()
    kv = dev.PagedKVCache(2, 2, 64, 16, 4, 8, 8)
    ref = ref_host.PagedKVTables(16, 4)
    rows = torch.randn(40, 2, 64, device="cuda").bfloat16()
    for layer in range(2):
        pass
    kv.reserve(_desc(dev, [(0, 40, 0, -1)]))
    for layer in range(2):
        kv.append(layer, rows, rows * 2)
    ref.reserve([0], [40])
    kv.fork(0, 1, 40)
    ref.fork(0, 1, 40)
    new = torch.randn(2, 2, 64, device="cuda").bfloat16()
    kv.reserve(_desc(dev, [(0, 1, 40, -1), (1, 1, 40, -1)]))
    for layer in range(2):
        kv.append(layer, new, new)
    ref.reserve([0, 1], [1, 1])
    assert kv.error_word() == 0
    _check_tables(kv, ref, 4)
    assert ref.cow_log == [(1, 2)]
    for layer in range(2):
        k0, v0 = kv.gather(layer, 0)
        k1, v1 = kv.gather(layer, 1)
        assert torch.equal(k0[:40], rows) and torch.equal(k1[:40], rows)  # the copy carried the data
        assert torch.equal(v0[:40], rows * 2) and torch.equal(v1[:40], rows * 2)
        assert torch.equal(k0[40], new[0]) and torch.equal(k1[40], new[1])


def test_append_gather_roundtrip_bf16():
    """append then gather returns exactly the rows written, in order (updateAndFetch's contiguous
    view, src/kvcache/paged.zig:533-637,705-802), for ragged multi-request steps over a scattered pool."""
    dev = _dev()
    rng = np.random.default_rng(303)
    kv = dev.PagedKVCache(2, 2, 128, 64, 4, 16, 8)
    kv.set_free_order(rng.permutation(64).tolist())
    want = {s: [] for s in range(4)}
    for step in range(5):
        seqs = [0, 1, 2, 3][: int(rng.integers(1, 5))]
        counts = [int(rng.integers(1, 45)) for _ in seqs]
        total = sum(counts)
        base = [kv.seq_len(s) for s in seqs]
        kv.reserve(_desc(dev, [(s, c, b, -1) for s, c, b in zip(seqs, counts, base)]))
        k = torch.randn(total, 2, 128, device="cuda").bfloat16()
        v = torch.randn(total, 2, 128, device="cuda").bfloat16()
        for layer in range(2):
            kv.append(layer, k + layer, v - layer)
        off = 0
        for s, c in zip(seqs, counts):
            want[s].append((k[off : off + c], v[off : off + c]))
            off += c
    assert kv.error_word() == 0
    for s in range(4):
        if not want[s]:
            continue
        kw = torch.cat([a for a, _ in want[s]])
        vw = torch.cat([b for _, b in want[s]])
        for layer in range(2):
            kg, vg = kv.gather(layer, s)
            assert torch.equal(kg, (kw + layer).bfloat16()) and torch.equal(vg, (vw - layer).bfloat16())


def test_fp8_pages_bit_exact():
    """E4M3 codes and per-(page, head) scales equal the oracle's definition, including the
    re-encode when a later append raises the page scale."""
    dev = _dev()
    rng = np.random.default_rng(404)
    H, D = 2, 64
    kv = dev.PagedKVCache(1, H, D, 8, 1, 8, 8, kv_dtype=dev.KV_FP8_E4M3)
    pages_k = {}
    n = 0
    for step, cnt in enumerate([5, 1, 1, 30, 1, 20]):
        rows = rng.normal(0, 1, (cnt, H, D)).astype(np.float32)
        if step == 2:
            rows *= 6.0  # forces a rescale of the first page
        rows = ref_math.bf16_round(rows)
        kv.reserve(_desc(dev, [(0, cnt, n, -1)]))
        t = torch.tensor(rows, device="cuda").bfloat16()
        kv.append(0, t, t * 0.5)
        for i in range(cnt):
            p, slot = (n + i) // 32, (n + i) % 32
            for h in range(H):
                q, sc, filled = pages_k.get((p, h), (np.zeros((32, D), np.uint8), 0.0, 0))
                pages_k[(p, h)] = (q, sc, filled)
        # oracle: apply per page touched, as the kernel does (one touch = rows of this step in that page)
        pos = n
        while pos < n + cnt:
            p = pos // 32
            hi = min((p + 1) * 32, n + cnt)
            for h in range(H):
                q, sc, filled = pages_k[(p, h)]
                q2, sc2 = ref_math.fp8_page_append(q, sc, filled, rows[pos - n : hi - n, h, :])
                pages_k[(p, h)] = (q2, sc2, filled + hi - pos)
            pos = hi
        n += cnt
    table = kv.block_table(0)
    for (p, h), (q, sc, filled) in pages_k.items():
        k_raw, v_raw, ks, vs = kv.page_raw(0, table[p])
        assert np.float32(ks[h]) == np.float32(sc), (p, h)
        assert np.array_equal(k_raw[h][:filled], q[:filled]), (p, h)
    kg, _ = kv.gather(0, 0)
    assert kg.shape[0] == n


def test_pool_exhaustion_is_flagged_not_trapped():
    """InsufficientBlocks surfaces through the error word and leaves the pool untouched
    (error.InsufficientBlocks, src/kvcache/paged.zig:109)."""
    dev = _dev()
    kv = dev.PagedKVCache(1, 2, 64, 4, 2, 8, 8)
    kv.reserve(_desc(dev, [(0, 100, 0, -1)]))
    kv.reserve(_desc(dev, [(1, 64, 0, -1)]))
    assert kv.error_word() == 1
    assert kv.free_count() == 0 and kv.seq_len(1) == 0 and kv.block_table(1) == []
    with pytest.raises(Exception):
        kv.alloc(1, 1)
    kv.reserve(_desc(dev, [(7, 1, 0, -1)]))  # bad slot
    assert kv.error_word() == 5


@pytest.mark.parametrize("kv_dtype_name", ["KV_BF16", "KV_FP8_E4M3"])
def test_extend_copies_a_sequence_between_pools(kv_dtype_name):
    """VTable.extend (src/kvcache/paged.zig:947-1109): a sequence prefilled in its own pool joins a
    running pool as a new sequence with its own page copies: same gathered rows and raw page bytes
    in every layer, reference counts 1, pages drawn from the destination's free stack in order; the
    two pools stay independent afterwards.  Errors: occupied slot, other shape, pool too small."""
    dev = _dev()
    kv_dtype = getattr(dev, kv_dtype_name)
    rng = np.random.default_rng(404)
    src = dev.PagedKVCache(2, 2, 128, 16, 2, 8, 8, kv_dtype=kv_dtype)
    dst = dev.PagedKVCache(2, 2, 128, 32, 4, 8, 8, kv_dtype=kv_dtype)
    src.set_free_order(rng.permutation(16).tolist())
    order = rng.permutation(32).tolist()
    dst.set_free_order(order)
    n_tok = 32 * 3 + 7
    src.reserve(_desc(dev, [(1, n_tok, 0, -1)]))
    dst.reserve(_desc(dev, [(0, 40, 0, -1)]))  # the running pool already serves a sequence
    for layer in range(2):
        src.append(layer, torch.randn(n_tok, 2, 128, device="cuda").bfloat16() * (1 + layer),
                   torch.randn(n_tok, 2, 128, device="cuda").bfloat16())
        dst.append(layer, torch.randn(40, 2, 128, device="cuda").bfloat16(), torch.randn(40, 2, 128, device="cuda").bfloat16())
    torch.cuda.synchronize()
    held = dst.block_table(0)
    free_before = dst.free_count()
    dst.extend(2, src, 1)
    assert dst.seq_len(2) == n_tok and dst.free_count() == free_before - 4
    table = dst.block_table(2)
    assert len(table) == 4 and not set(table) & set(held)
    assert [dst.ref_counts()[p] for p in table] == [1, 1, 1, 1]
    for layer in range(2):
        ks, vs = src.gather(layer, 1)
        kd, vd = dst.gather(layer, 2)
        assert torch.equal(ks, kd) and torch.equal(vs, vd)
        for ps, pd in zip(src.block_table(1), table):
            for x, y in zip(src.page_raw(layer, ps), dst.page_raw(layer, pd)):
                assert np.array_equal(x, y)
    # the copy keeps living when the source goes away, and grows on its own
    src.release([1])
    dst.reserve(_desc(dev, [(2, 30, n_tok, -1)]))
    torch.cuda.synchronize()
    assert dst.seq_len(2) == n_tok + 30 and len(dst.block_table(2)) == 5 and dst.error_word() == 0
    with pytest.raises(Exception):
        dst.extend(0, dst, 2)  # slot 0 is in use
    other = dev.PagedKVCache(2, 2, 64, 16, 2, 8, 8, kv_dtype=kv_dtype)
    with pytest.raises(Exception):
        other.extend(0, dst, 2)
    small = dev.PagedKVCache(2, 2, 128, 3, 2, 8, 8, kv_dtype=kv_dtype)
    with pytest.raises(Exception):
        small.extend(0, dst, 2)  # 5 pages needed, 3 in the pool
    assert small.free_count() == 3
    for p in (src, dst, other, small):
        p.close()


def test_filter_current_len_and_reset_match_the_page_table_oracle():
    """Three members of the KVCacheStrategy vtable on the device pool: filter keeps the listed
    sequences and frees what only the others held (src/kvcache/paged.zig:879-945), currentLen is the
    longest sequence (:842-849), reset empties the pool (:851-862).  Tables, reference counts, free
    count and the order in which freed pages come back are compared with the oracle after every call,
    with shared (forked) pages in play; a slot outside the pool is InvalidBatchIndex (:904)."""
    from dmlx_b200 import _lib

    dev = _dev()
    rng = np.random.default_rng(404)
    n_pages, n_seqs = 96, 10
    kv = dev.PagedKVCache(1, 2, 64, n_pages, n_seqs, 16, 8, max_rows=4096)
    ref = ref_host.PagedKVTables(n_pages, n_seqs)
    assert kv.current_len() == ref.current_len() == 0
    for rnd in range(4):
        seqs = list(range(0, 6))
        counts = [int(rng.integers(1, 150)) for _ in seqs]
        ref.reserve(seqs, counts)
        kv.reserve(_desc(dev, [(s, c, 0, -1) for s, c in zip(seqs, counts)]))
        assert kv.error_word() == 0
        # slots 6..8 share prefixes of 0..2; a prefix of the whole source shares its partly filled last page too
        for dst, src in ((6, 0), (7, 1), (8, 2)):
            nt = ref.lens[src] if dst == 6 else int(rng.integers(1, ref.lens[src] + 1))
            ref.fork(src, dst, nt)
            kv.fork(src, dst, nt)
        _check_tables(kv, ref, n_seqs)
        assert kv.current_len() == ref.current_len() == max(ref.lens)
        keep = [[1, 6, 8, 3], [0, 7], [], [9, 2, 4]][rnd]   # a donor without its sharer, a sharer without its donor, nobody, an empty slot
        ref.filter(keep)
        kv.filter(keep)
        _check_tables(kv, ref, n_seqs)
        assert kv.current_len() == ref.current_len()
        # the pages that came back are handed out again in the same order
        grow = [s for s in range(n_seqs) if s not in keep][:3]
        ref.reserve(grow, [40, 33, 70][: len(grow)])
        kv.reserve(_desc(dev, [(s, c, 0, -1) for s, c in zip(grow, [40, 33, 70])]))
        assert kv.error_word() == 0
        _check_tables(kv, ref, n_seqs)
        ref.reset()
        kv.reset()
        _check_tables(kv, ref, n_seqs)
        assert kv.current_len() == 0 and kv.free_count() == n_pages and sum(kv.ref_counts().tolist()) == 0
    with pytest.raises(_lib.InvalidBatchIndex):
        kv.filter([0, n_seqs])
    with pytest.raises(ref_host.InvalidBatchIndex):
        ref.filter([0, n_seqs])
    kv.close()


def test_rope_append_in_one_call_matches_rope_then_append():
    """b200_kv_rope_append: q and k rotated in place with per-row positions (non-traditional RoPE,
    src/models/llama.zig:213-215) and the rotated K rows and V rows written to their pages, against the
    oracle's rope followed by the gathered view of the pool."""
    dev = _dev()
    rng = np.random.default_rng(17)
    hq, hkv, d = 8, 2, 64
    ctxs = [37, 5, 64]
    kv = dev.PagedKVCache(1, hkv, d, 16, 3, 4, hq, max_rows=256)
    desc = dev.pack_desc_array([(s, c, 0, -1) for s, c in enumerate(ctxs)]).cuda()
    kv.reserve(desc)
    t = sum(ctxs)
    q = ref_math.bf16_round(rng.normal(0, 1, (t, hq, d)))
    k = ref_math.bf16_round(rng.normal(0, 1, (t, hkv, d)))
    v = ref_math.bf16_round(rng.normal(0, 1, (t, hkv, d)))
    pos = np.concatenate([np.arange(c) for c in ctxs]).astype(np.int32)
    seq = np.concatenate([np.full(c, s) for s, c in enumerate(ctxs)]).astype(np.int32)
    qd, kd, vd = (torch.tensor(a, device="cuda").bfloat16() for a in (q, k, v))
    kv.rope_append(0, qd, kd, vd, torch.tensor(pos, device="cuda"), torch.tensor(seq, device="cuda"), theta=10000.0)
    torch.cuda.synchronize()
    assert kv.error_word() == 0
    off = 0
    for s, c in enumerate(ctxs):
        want_q = ref_math.rope(q[off:off + c].transpose(1, 0, 2), np.arange(c)).transpose(1, 0, 2)
        want_k = ref_math.rope(k[off:off + c].transpose(1, 0, 2), np.arange(c)).transpose(1, 0, 2)
        got_k, got_v = kv.gather(0, s)
        assert np.abs(qd[off:off + c].float().cpu().numpy() - want_q).max() <= 2e-2 * np.abs(want_q).max()
        assert np.abs(got_k.float().cpu().numpy() - want_k).max() <= 2e-2 * np.abs(want_k).max()
        assert np.array_equal(got_v.float().cpu().numpy(), v[off:off + c])
        off += c
    kv.close()


@pytest.mark.parametrize("rows_per_seq", [(5,), (1, 1, 1, 1, 1, 1, 1, 1), (40, 3), (200, 97, 3)])
def test_rope_append_from_the_projection_partial_sums_gives_the_same_bits(rows_per_seq):
    """b200_qmm_deferred + b200_kv_rope_append_partials against b200_qmm + b200_kv_rope_append on the same inputs:
    the q rows and the K and V pages must be bit-identical (the fused kernel sums the K splits in split order and
    rounds to bf16 where the finish pass would).  Row counts chosen to reach the small-batch kernel, the
    tensor-memory kernel and a launch with several token tiles."""
    dev = _dev()
    rng = np.random.default_rng(5 + sum(rows_per_seq))
    hq, hkv, d, k = 6, 2, 128, 1024
    n = (hq + 2 * hkv) * d
    w = dev.QWeight.random(dev.Q_AFFINE4_G64, n, k, seed=11)
    t = sum(rows_per_seq)
    x = torch.tensor(ref_math.bf16_round(rng.normal(0, 1, (t, k))), device="cuda").bfloat16()
    starts = [int(rng.integers(0, 60)) for _ in rows_per_seq]   # rows continue sequences that already hold tokens
    pos = np.concatenate([np.arange(s0, s0 + c) for s0, c in zip(starts, rows_per_seq)]).astype(np.int32)
    seq = np.concatenate([np.full(c, s) for s, c in enumerate(rows_per_seq)]).astype(np.int32)
    posd, seqd = torch.tensor(pos, device="cuda"), torch.tensor(seq, device="cuda")
    results = []
    for fused in (False, True):
        kv = dev.PagedKVCache(1, hkv, d, 32, len(rows_per_seq), 12, hq, max_rows=512)
        kv.set_free_order(list(range(32)))
        for s, s0 in enumerate(starts):
            if s0 > 0:
                kv.reserve(dev.pack_desc_array([(s, s0, 0, -1)]).cuda())
        kv.reserve(dev.pack_desc_array([(s, c, s0, -1) for s, (s0, c) in enumerate(zip(starts, rows_per_seq))]).cuda())
        qkv = torch.zeros((t, n), dtype=torch.bfloat16, device="cuda")
        if fused:
            parts = dev.qmm_deferred(w, x, qkv)
            assert parts.pending == 1, "this shape is expected to split K"
            assert parts.rows == t and parts.n == n and parts.nt * 128 == n
            kv.rope_append_partials(0, parts, qkv, n, posd, seqd, hq, theta=500000.0)
        else:
            parts = dev.qmm_deferred(w, x, qkv, defer=False)
            assert parts.pending == 0
            qc = qkv[:, : hq * d].contiguous().view(t, hq, d)
            kc = qkv[:, hq * d: (hq + hkv) * d].contiguous().view(t, hkv, d)
            vc = qkv[:, (hq + hkv) * d:].contiguous().view(t, hkv, d)
            kv.rope_append(0, qc, kc, vc, posd, seqd, theta=500000.0)
            qkv[:, : hq * d] = qc.view(t, hq * d)
        torch.cuda.synchronize()
        assert kv.error_word() == 0 and dev.qmm_error_word() == 0
        q = qkv[:, : hq * d].clone().view(torch.int16).cpu().numpy()
        pages = []
        for s, (s0, c) in enumerate(zip(starts, rows_per_seq)):
            gk, gv = kv.gather(0, s)
            pages.append((gk[s0:s0 + c].view(torch.int16).cpu().numpy(), gv[s0:s0 + c].view(torch.int16).cpu().numpy()))
        results.append((q, pages))
        kv.close()
    (q0, p0), (q1, p1) = results
    assert np.array_equal(q0, q1)
    for (k0, v0), (k1, v1) in zip(p0, p1):
        assert np.array_equal(k0, k1) and np.array_equal(v0, v1)
    assert np.abs(q0.astype(np.int32)).max() > 0

