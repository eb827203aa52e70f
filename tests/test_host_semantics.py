"""Known-answer and property tests for the host-side integer semantics.

Every case is a restatement of one of the reference's own tests (cited per test) and runs
against two implementations behind one API: the CPU oracle (``oracle.ref_host``) and the product's
C++ host layer through the C-ABI (``dmlx_b200.host``).  Passing on the oracle pins the oracle;
passing on the product is the parity gate for the scheduler / batch builder / block manager.
"""
import numpy as np
import pytest


def _drain(sched, H, outputs):
    sched.postprocess(outputs)


# ---- src/tests/scheduler_tests.zig ----------------------------------------------------------


def test_empty_schedule(H):  # scheduler_tests.zig:24-35
    s = H.Scheduler(H.SchedBlockManager(16), 512)
    r = s.schedule()
    assert r.is_empty() and r.blocks_needed == 0


def test_single_request_lifecycle(H):  # scheduler_tests.zig:37-70
    s = H.Scheduler(H.SchedBlockManager(16), 512)
    req = H.Request(1, [1, 2, 3], 5, [])
    s.add_request(req)
    assert req.state == H.WAITING
    r1 = s.schedule()
    assert len(r1.prefill_requests) == 1 and len(r1.decode_requests) == 0
    assert req.state == H.PREFILLING
    s.postprocess([(1, 100)])
    assert req.state == H.DECODING and list(req.generated_tokens) == [100]
    r2 = s.schedule()
    assert len(r2.prefill_requests) == 0 and len(r2.decode_requests) == 1


def test_stop_token_and_max_tokens(H):  # scheduler_tests.zig:72-118
    s = H.Scheduler(H.SchedBlockManager(16), 512)
    a = H.Request(1, [1, 2], 100, [99])
    b = H.Request(2, [1, 2], 2, [])
    s.add_request(a)
    s.add_request(b)
    s.schedule()
    s.postprocess([(1, 5), (2, 6)])
    s.schedule()
    s.postprocess([(1, 99), (2, 7)])
    assert a.state == H.DONE and b.state == H.DONE
    assert s.active_count() == 0


def test_decode_prioritised_over_prefill(H):  # scheduler_tests.zig:120-148
    s = H.Scheduler(H.SchedBlockManager(16), 512)
    r1 = H.Request(1, [1, 2], 10, [])
    s.add_request(r1)
    s.schedule()
    s.postprocess([(1, 50)])
    r2 = H.Request(2, [3, 4], 10, [])
    s.add_request(r2)
    res = s.schedule()
    assert [r.id for r in res.decode_requests] == [1]
    assert [r.id for r in res.prefill_requests] == [2]


def test_waiting_when_no_blocks(H):  # scheduler_tests.zig:150-171
    s = H.Scheduler(H.SchedBlockManager(0), 512)
    req = H.Request(1, [1, 2], 10, [])
    s.add_request(req)
    res = s.schedule()
    assert res.is_empty() and res.blocks_needed == 1
    assert req.state == H.WAITING and s.active_count() == 1


def test_blocks_freed_on_completion(H):  # scheduler_tests.zig:173-195
    bm = H.SchedBlockManager(4)
    s = H.Scheduler(bm, 512)
    req = H.Request(1, [1], 1, [])
    s.add_request(req)
    s.schedule()
    assert bm.free_count() == 3 and list(req.block_ids) == [0]
    s.postprocess([(1, 9)])
    assert bm.free_count() == 4 and req.state == H.DONE


def test_seq_len_tracks_progress(H):  # scheduler_tests.zig:248-264
    s = H.Scheduler(H.SchedBlockManager(4), 512)
    req = H.Request(1, [1, 2, 3], 10, [])
    assert req.seq_len() == 0
    s.add_request(req)
    s.schedule()
    s.postprocess([(1, 7)])
    assert req.seq_len() == 4
    s.schedule()
    s.postprocess([(1, 8)])
    assert req.seq_len() == 5


def test_chunked_prefill_progression(H):  # scheduler_tests.zig:538-597, 686-714
    s = H.Scheduler(H.SchedBlockManager(8), 3)
    req = H.Request(1, list(range(10, 17)), 4, [])  # 7 tokens -> chunks 3,3,1
    s.add_request(req)
    offs = []
    for _ in range(3):
        res = s.schedule()
        assert [r.id for r in res.prefill_requests] == [1]
        s.postprocess([(1, 42)])
        offs.append(req.prefill_offset)
    assert offs == [3, 6, 7]
    assert req.state == H.DECODING and list(req.generated_tokens) == [42]


def test_property_prioritisation(H):  # scheduler_tests.zig:280-406 (Property 7), 100 cases
    rng = np.random.default_rng(7)
    for _ in range(100):
        bm = H.SchedBlockManager(int(rng.integers(1, 12)))
        s = H.Scheduler(bm, 512)
        reqs = [H.Request(i + 1, [1, 2, 3], int(rng.integers(1, 5)), []) for i in range(int(rng.integers(1, 10)))]
        for r in reqs:
            s.add_request(r)
        for _step in range(6):
            res = s.schedule()
            dec, pre = [r.id for r in res.decode_requests], [r.id for r in res.prefill_requests]
            assert not (set(dec) & set(pre))
            for r in reqs:  # every running request is scheduled
                if r.state == H.DECODING:
                    assert r.id in dec
            s.postprocess([(i, 5) for i in pre + dec])
            assert bm.free_count() + sum(len(r.block_ids) for r in reqs) == bm.total_blocks


# ---- src/tests/batch_builder_tests.zig + integration_tests.zig ------------------------------


def _sched_result(H, prefill, decode):
    return H.ScheduleResult(prefill, decode, 0)


def _decode_request(H, rid, prompt, gen):
    r = H.Request(rid, prompt, 10, [])
    r.force_state(H.DECODING, len(prompt), gen)
    return r


def _prefill_request(H, rid, prompt, offset=0):
    r = H.Request(rid, prompt, 10, [])
    r.force_state(H.PREFILLING, offset, [])
    return r


def test_batch_empty(H):  # batch_builder_tests.zig:44-59
    b = H.build_batch(_sched_result(H, [], []))
    assert b.total_tokens == 0 and b.num_requests == 0 and b.batched_tokens.shape == (0,)


def test_batch_single_prefill_and_decode(H):  # batch_builder_tests.zig:61-138
    b = H.build_batch(_sched_result(H, [_prefill_request(H, 1, [10, 20, 30])], []))
    assert b.batched_tokens.tolist() == [10, 20, 30] and b.position_ids.tolist() == [0, 1, 2]
    b = H.build_batch(_sched_result(H, [], [_decode_request(H, 2, [1, 2, 3], [42])]))
    assert b.batched_tokens.tolist() == [42] and b.position_ids.tolist() == [3]


def test_batch_mixed_isolation(H):  # batch_builder_tests.zig:140-193
    r1 = _prefill_request(H, 1, [100, 200])
    r2 = _decode_request(H, 2, [300, 400, 500], [600])
    b = H.build_batch(_sched_result(H, [r1], [r2]))
    assert b.total_tokens == 3 and b.num_requests == 2
    assert b.batched_tokens.tolist() == [100, 200, 600]
    assert b.cu_seqlens.tolist() == [0, 2, 3] and b.row_to_req.tolist() == [0, 0, 1]
    expect = {(0, 0): True, (1, 0): True, (1, 1): True, (0, 1): False, (0, 2): False, (1, 2): False,
              (2, 0): False, (2, 1): False, (2, 2): True}
    for (r, c), v in expect.items():
        assert H.is_attending(b.attention_mask, r, c) == v
        assert H.is_attending_ragged(b.cu_seqlens, r, c) == v


def test_batch_ignores_max_prefill_tokens(H):  # integration_tests.zig:798-857
    s = H.Scheduler(H.SchedBlockManager(32), 3)
    r1 = H.Request(1, [1, 2], 10, [])
    s.add_request(r1)
    s.schedule()
    s.postprocess([(1, 50)])
    r2 = H.Request(2, [10, 20, 30, 40, 50, 60, 70], 10, [])
    s.add_request(r2)
    res = s.schedule()
    b = H.build_batch(res)
    assert b.total_tokens == 8  # 7 prompt tokens (uncapped) + 1 decode token
    assert not H.is_attending(b.attention_mask, 0, 7) and not H.is_attending(b.attention_mask, 7, 6)
    bc = H.build_batch(res, chunked=True, max_prefill_tokens=3)
    assert bc.total_tokens == 4 and bc.position_ids.tolist() == [0, 1, 2, 2]
    s.postprocess([(1, 51), (2, 0)])
    assert r1.state == H.DECODING and r2.state == H.PREFILLING and r2.prefill_offset == 3


def test_property_attention_isolation(H):  # batch_builder_tests.zig:318-477 (Property 11), 100 cases
    rng = np.random.default_rng(11)
    for _ in range(100):
        pre = [_prefill_request(H, i, rng.integers(0, 1000, int(rng.integers(1, 9))).tolist())
               for i in range(int(rng.integers(0, 4)))]
        dec = [_decode_request(H, 100 + i, rng.integers(0, 1000, int(rng.integers(1, 9))).tolist(),
                               rng.integers(0, 1000, int(rng.integers(1, 4))).tolist())
               for i in range(int(rng.integers(0, 5)))]
        b = H.build_batch(_sched_result(H, pre, dec))
        lens = [len(r.prompt_tokens) for r in pre] + [1] * len(dec)
        assert b.total_tokens == sum(lens)
        if b.total_tokens == 0:
            continue
        cu = np.concatenate([[0], np.cumsum(lens)])
        assert b.cu_seqlens.tolist() == cu.tolist()
        for r in range(b.total_tokens):
            for c in range(b.total_tokens):
                same = np.searchsorted(cu, r, "right") == np.searchsorted(cu, c, "right")
                assert H.is_attending(b.attention_mask, r, c) == bool(same and c <= r)


# ---- src/tests/kvcache_tests.zig: BlockManager ------------------------------------------------


def test_bm_alloc_free(H):  # kvcache_tests.zig:432-536
    bm = H.PagedBlockManager(8)
    assert bm.free_count() == 8 and bm.used_count() == 0
    assert bm.allocate_blocks(1, 3) == [0, 1, 2]
    assert bm.free_count() == 5 and bm.blocks_of(1) == [0, 1, 2]
    with pytest.raises(H.InsufficientBlocks):
        bm.allocate_blocks(2, 6)
    assert bm.allocate_blocks(2, 2) == [3, 4]
    bm.free_blocks_of(1)
    assert bm.free_count() == 6
    bm.free_blocks_of(77)  # unknown id: no-op
    assert bm.free_count() == 6
    assert bm.allocate_blocks(3, 2) == [2, 1]  # LIFO: last freed first (paged.zig:117,156)
    assert bm.can_allocate(4) and not bm.can_allocate(5)


def test_bm_copy_on_write(H):  # kvcache_tests.zig:538-594
    bm = H.PagedBlockManager(4)
    (bid,) = bm.allocate_blocks(1, 1)
    assert bm.copy_on_write(bid) == bid
    bm.set_ref(bid, 2)
    cow = bm.copy_on_write(bid)
    assert cow != bid and bm.get_ref(bid) == 1 and bm.get_ref(cow) == 1 and bm.is_used(cow)
    with pytest.raises(H.InvalidBlockId):
        bm.copy_on_write(99)
    one = H.PagedBlockManager(1)
    (b0,) = one.allocate_blocks(1, 1)
    one.set_ref(b0, 2)
    with pytest.raises(H.InsufficientBlocks):
        one.copy_on_write(b0)


def test_bm_shared_free(H):  # kvcache_tests.zig:596-629
    bm = H.PagedBlockManager(4)
    (bid,) = bm.allocate_blocks(1, 1)
    bm.set_ref(bid, 2)
    bm.share(2, bid)
    before = bm.free_count()
    bm.free_blocks_of(2)
    assert bm.get_ref(bid) == 1 and bm.is_used(bid) and bm.free_count() == before
    bm.free_blocks_of(1)
    assert bm.get_ref(bid) == 0 and not bm.is_used(bid) and bm.free_count() == before + 1


def test_bm_hash_and_prefix(H):  # kvcache_tests.zig:654-723
    toks = [1, 2, 3, 4, 5, 6, 7, 8]
    assert H.hash_block(0, toks[:4]) == H.hash_block(0, toks[:4])
    assert H.hash_block(0, toks[:4]) != H.hash_block(1, toks[:4])
    assert H.hash_block(0, toks[:4]) != H.hash_block(0, toks[4:])
    bm = H.PagedBlockManager(8)
    b = bm.allocate_blocks(1, 2)
    h0 = H.hash_block(0, toks[:4])
    bm.set_tokens_used(b[0], 4)
    bm.register_block_hash(b[0], h0)
    h1 = H.hash_block(h0, toks[4:])
    bm.set_tokens_used(b[1], 4)
    bm.register_block_hash(b[1], h1)
    assert bm.find_cached_prefix(toks, 4) == b
    assert bm.get_ref(b[0]) == 2 and bm.get_ref(b[1]) == 2
    assert bm.find_cached_prefix([9, 9, 9, 9], 4) == []
    assert bm.find_cached_prefix(toks, 0) == []
    assert bm.find_cached_prefix(toks[:4] + [0, 0, 0, 0], 4) == [b[0]]


def test_hash_matches_oracle(H):
    """The product and the oracle must produce identical hash chains (same block tables)."""
    from oracle import ref_host

    rng = np.random.default_rng(13)
    for _ in range(20):
        t = rng.integers(0, 2**32, int(rng.integers(1, 40)), dtype=np.uint64).tolist()
        p = int(rng.integers(0, 2**63))
        assert H.hash_block(p, t) == ref_host.hash_block(p, t)


def test_property_block_conservation(H):  # kvcache_tests.zig:739-923 (Property 8), 100 cases
    from oracle import ref_host

    rng = np.random.default_rng(8)
    for _ in range(100):
        total = int(rng.integers(4, 40))
        bm, ref = H.PagedBlockManager(total), ref_host.PagedBlockManager(total)
        live = []
        for _op in range(40):
            op = rng.integers(0, 3)
            if op == 0:
                rid, n = int(rng.integers(1, 1000)), int(rng.integers(1, 5))
                try:
                    want = ref.allocate_blocks(rid, n)
                except ref_host.InsufficientBlocks:
                    with pytest.raises(H.InsufficientBlocks):
                        bm.allocate_blocks(rid, n)
                    continue
                assert bm.allocate_blocks(rid, n) == want
                live.append(rid)
            elif op == 1 and live:
                rid = live.pop(int(rng.integers(0, len(live))))
                ref.free_blocks_of(rid)
                bm.free_blocks_of(rid)
            elif op == 2 and live:
                rid = live[int(rng.integers(0, len(live)))]
                blocks = ref.blocks_of(rid)
                if blocks:
                    bid = blocks[0]
                    ref.set_ref(bid, ref.get_ref(bid) + 1)
                    bm.set_ref(bid, bm.get_ref(bid) + 1)
                    try:
                        want = ref.copy_on_write(bid)
                    except ref_host.InsufficientBlocks:
                        with pytest.raises(H.InsufficientBlocks):
                            bm.copy_on_write(bid)
                        ref.set_ref(bid, ref.get_ref(bid) - 1)
                        bm.set_ref(bid, bm.get_ref(bid) - 1)
                        continue
                    got = bm.copy_on_write(bid)
                    assert got == want
                    # keep conservation: hand the copy to the request, drop the fake share
                    ref.share(rid, want)
                    bm.share(rid, got)
            assert bm.free_count() + bm.used_count() == total
            assert bm.free_count() == ref.free_count()


def test_scheduler_with_real_block_manager(H):  # scheduler.zig:37-43 initWithReal
    real = H.PagedBlockManager(2)
    bm = H.SchedBlockManager(real=real)
    s = H.Scheduler(bm, 512)
    reqs = [H.Request(i, [1, 2, 3], 1, []) for i in (1, 2, 3)]
    for r in reqs:
        s.add_request(r)
    res = s.schedule()
    assert [r.id for r in res.prefill_requests] == [1, 2] and res.blocks_needed == 1
    assert list(reqs[0].block_ids) == [0] and list(reqs[1].block_ids) == [1]
    s.postprocess([(1, 5), (2, 6)])
    assert real.free_count() == 2
    res = s.schedule()
    assert [r.id for r in res.prefill_requests] == [3] and list(reqs[2].block_ids) == [1]  # LIFO: last freed first


def test_greedy_first_strict_max(H):  # sampling.zig:22-39
    assert H.greedy(np.array([1.0, 3.0, 3.0, 2.0], np.float32)) == 1
    assert H.greedy(np.array([5.0], np.float32)) == 0


# ---- extensions: removal of one request, preemption by recomputation, admission hold ----------
# (src/engine/engine_loop.zig:687-754 handleBatchError, src/engine/request_state.zig:182-189 cancel
# flag; preemption has no reference counterpart).  Oracle and product must agree.


def test_remove_running_request_frees_its_blocks_only(H):
    bm = H.SchedBlockManager(4)
    s = H.Scheduler(bm, 512)
    a, b = H.Request(1, [1, 2, 3], 8, []), H.Request(2, [4, 5], 8, [])
    s.add_request(a)
    s.add_request(b)
    s.schedule()
    s.postprocess([(1, 10), (2, 11)])
    assert bm.free_count() == 2
    s.remove(a, 12)
    assert a.state == H.DONE and a.error == 12 and list(a.generated_tokens) == [10]
    assert bm.free_count() == 3 and s.active_count() == 1
    r = s.schedule()
    assert [q.id for q in r.decode_requests] == [2] and not r.prefill_requests
    s.postprocess([(2, 12)])
    assert list(b.generated_tokens) == [11, 12] and b.error == 0


def test_remove_waiting_request(H):
    s = H.Scheduler(H.SchedBlockManager(0), 512)
    a = H.Request(1, [1, 2, 3], 8, [])
    s.add_request(a)
    assert s.schedule().is_empty()
    s.remove(a, 12)
    assert a.state == H.DONE and s.active_count() == 0


def test_preempt_folds_output_into_prompt_and_resumes(H):
    bm = H.SchedBlockManager(4)
    s = H.Scheduler(bm, 2)
    a = H.Request(1, [1, 2, 3], 5, [])
    s.add_request(a)
    s.schedule(); s.postprocess([(1, 0)])       # chunk [1, 2]
    s.schedule(); s.postprocess([(1, 50)])      # chunk [3] -> first token
    s.schedule(); s.postprocess([(1, 51)])      # decode
    assert a.seq_len() == 5 and list(a.generated_tokens) == [50, 51]
    s.preempt(a)
    assert a.state == H.WAITING and a.prefill_offset == 0 and bm.free_count() == 4
    assert list(a.prompt_tokens) == [1, 2, 3, 50, 51] and list(a.generated_tokens) == [50, 51]
    assert a.seq_len() == 0
    # second prefill: three chunks of two, the last one yields the next output token
    for tok in (0, 0, 52):
        r = s.schedule()
        assert [q.id for q in r.prefill_requests] == [1]
        s.postprocess([(1, tok)])
    assert a.state == H.DECODING and list(a.generated_tokens) == [50, 51, 52] and a.seq_len() == 6
    r = s.schedule()
    assert [q.id for q in r.decode_requests] == [1]
    s.postprocess([(1, 53)])
    s.schedule(); s.postprocess([(1, 54)])
    assert a.state == H.DONE and list(a.generated_tokens) == [50, 51, 52, 53, 54]  # max_tokens counts all five


def test_preempted_request_waits_ahead_of_newcomers_and_hold_blocks_admission(H):
    bm = H.SchedBlockManager(2)
    s = H.Scheduler(bm, 512)
    a, b, c = H.Request(1, [1], 4, []), H.Request(2, [2], 4, []), H.Request(3, [3], 4, [])
    s.add_request(a)
    s.add_request(b)
    s.schedule(); s.postprocess([(1, 7), (2, 8)])
    s.add_request(c)
    s.preempt(b)
    s.hold_admission(True)
    r = s.schedule()
    assert [q.id for q in r.decode_requests] == [1] and not r.prefill_requests and r.blocks_needed == 2
    s.hold_admission(False)
    r = s.schedule()
    assert [q.id for q in r.prefill_requests] == [2]  # b first: one block free, c keeps waiting
    assert r.blocks_needed == 1


def test_admission_budget_in_pages_keeps_arrival_order(H):
    """With a page budget, a waiting request is promoted only while ceil((prompt + 1) / 32) pages of the
    budget are left, and the first one that does not fit stops the promotions of that call (nobody
    overtakes it); without a budget one free block admits, as in src/scheduler.zig:291-293."""
    s = H.Scheduler(H.SchedBlockManager(64), 512)
    reqs = [H.Request(i + 1, list(range(n)), 4, []) for i, n in enumerate((31, 64, 200, 10))]  # 1, 3, 7, 1 pages
    for r in reqs:
        s.add_request(r)
    s.set_admission_budget(5)
    r = s.schedule()
    assert [q.id for q in r.prefill_requests] == [1, 2] and r.blocks_needed == 2  # 3 needs 7 > 1 left; 4 waits behind it
    s.set_admission_budget(7)
    r = s.schedule()
    assert [q.id for q in r.prefill_requests] == [1, 2, 3] and r.blocks_needed == 1
    s.set_admission_budget(None)
    r = s.schedule()
    assert [q.id for q in r.prefill_requests] == [1, 2, 3, 4]
