"""The tiny LLaMA configuration end to end through the engine step (b200_engine_*): 4 layers, hidden
512, 8 query / 2 KV heads, head_dim 64, FFN 1408, vocab 32000, N(0,0.02) weights, a continuous batch
of 8 requests with seeded prompt lengths 16..256, greedy decode for 64 steps, 32-token pages, chunked
prefill.  Every token the engine emits is checked against the fp32 oracle running that request alone
at B=1 on the same token history: it must be the oracle's argmax unless the oracle's top-2 gap is
below twice the logit error measured on that very row, and then it must lie within that bound of the
maximum.  The number of sequences that equal the free-running oracle from the first to the last token
is printed and pinned."""
import numpy as np
import pytest

from oracle import ref_host, ref_math

pytestmark = pytest.mark.gpu

CFG = ref_math.LlamaConfig(n_layers=4, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1408, vocab=32000)
N_REQ, N_STEPS = 8, 64
# Sequences (of 8) whose 64 greedy ids equal the free-running fp32 oracle on a B200; the others part
# from it at a near-tie that the per-token check below accepts.
IDENTICAL_PINNED = 1


def _bits(a):
    return (ref_math.bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def _build_model(dev, cfg, weights):
    model = dev.LlamaModel(cfg.n_layers, cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab,
                           max_rows=1024, max_reqs=16, max_seqs=16, rms_eps=cfg.eps, rope_theta=cfg.theta)
    names = {"wq": 0, "wk": 1, "wv": 2, "wo": 3, "gate": 4, "up": 5, "down": 6}
    for l in range(cfg.n_layers):
        for nm, which in names.items():
            model.set_linear(l, which, dev.Q_BF16, _bits(weights[f"l{l}.{nm}"]))
        model.set_norm(l, 0, _bits(weights[f"l{l}.attn_norm"]))
        model.set_norm(l, 1, _bits(weights[f"l{l}.ffn_norm"]))
    model.set_linear(0, 7, dev.Q_BF16, _bits(weights["lm_head"]))
    model.set_norm(-1, 0, _bits(weights["final_norm"]))
    model.set_embedding(_bits(weights["embed"]))
    model.finalize()
    return model


def _check_against_oracle(cfg, weights, prompt, got, tag):
    """Greedy ids equal the fp32 oracle up to the first near-tie; a divergence is the runner-up."""
    o = ref_math.LlamaB1(cfg, weights)
    logits = o.forward(prompt)
    for j, g in enumerate(got):
        tok = ref_host.greedy(logits)
        if g != tok:
            top2 = np.sort(logits)[-2:]
            assert top2[1] - top2[0] < 2e-2 * np.abs(logits).max(), (tag, j, float(top2[1] - top2[0]))
            assert g == int(np.argsort(logits)[-2]), (tag, j)
            return False
        logits = o.forward([tok])
    return True


def test_config1_greedy_decode_matches_oracle():
    from dmlx_b200 import device as dev

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 128, 16, 16, cfg.n_heads, max_rows=1024,
                          attn_scratch_chunks=8192)
    eng = dev.Engine(model, kv, max_prefill_tokens=96)  # prompts above 96 tokens prefill in chunks
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, cfg.vocab, int(rng.integers(16, 257))).tolist() for _ in range(N_REQ)]
    # requests arrive over the first steps: continuous batching with mixed prefill + decode steps
    arrivals = {0: [0, 1, 2], 1: [3], 2: [4, 5], 4: [6], 7: [7]}
    # one oracle per request, fed the engine's own tokens (so every token is checked, also after a near-tie)
    oracles = {i + 1: ref_math.LlamaB1(cfg, weights) for i in range(N_REQ)}
    fed = {i + 1: 0 for i in range(N_REQ)}        # prompt tokens the oracle has consumed
    emitted = {i + 1: [] for i in range(N_REQ)}
    diverged = set()
    rel_worst, near_ties, checked = 0.0, 0, 0
    step = 0
    while (eng.active_count() > 0 or step <= max(arrivals)) and step < 400:
        for i in arrivals.get(step, []):
            eng.submit(i + 1, prompts[i], N_STEPS)
        joined = dict(eng.step())
        batch = eng.last_batch()
        logits = model.last_logits(len(batch))
        for row, rid in enumerate(batch):
            o, prompt = oracles[rid], prompts[rid - 1]
            if fed[rid] < len(prompt):      # a prefill chunk (the engine's chunking: 96 tokens)
                n = min(96, len(prompt) - fed[rid])
                want = o.forward(prompt[fed[rid]:fed[rid] + n])
                fed[rid] += n
            else:
                want = o.forward([emitted[rid][-1]])
            if rid not in joined:
                continue                    # a chunk that is not the last one: its token is dropped
            got = joined[rid]
            err = float(np.abs(logits[row] - want).max())
            rel_worst = max(rel_worst, err / float(np.abs(want).max()))
            best = ref_host.greedy(want)
            top2 = np.sort(want)[-2:]
            checked += 1
            if top2[1] - top2[0] > 2 * err:
                assert got == best, (rid, len(emitted[rid]), float(top2[1] - top2[0]), err)
            elif got != best:
                assert want[best] - want[got] <= 2 * err, (rid, len(emitted[rid]), float(want[best] - want[got]), err)
                near_ties += 1
                diverged.add(rid)
            emitted[rid].append(got)
        step += 1
    assert eng.active_count() == 0
    assert eng.free_pages() == 128  # every page returned (src/scheduler.zig:371-380)
    assert rel_worst <= 2e-2, rel_worst
    for i in range(N_REQ):
        got, done = eng.result(i + 1)
        assert done and len(got) == N_STEPS and got == emitted[i + 1]
    identical = N_REQ - len(diverged)
    print(f"greedy ids: {identical} of {N_REQ} sequences identical to the fp32 oracle over {N_STEPS} steps; "
          f"{near_ties} near-tie tokens of {checked}; worst logit error {rel_worst:.2e} of the row maximum")
    assert identical >= IDENTICAL_PINNED, (identical, sorted(diverged))
    eng.close()
    model.close()
    kv.close()


def _run_engine(dev, cfg, model, prompts, n_new, n_pages, max_pages_per_seq=16, chunk=64, hook=None):
    kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, n_pages, 16, max_pages_per_seq, cfg.n_heads,
                          max_rows=1024, attn_scratch_chunks=8192)
    eng = dev.Engine(model, kv, max_prefill_tokens=chunk)
    for i, p in enumerate(prompts):
        eng.submit(i + 1, p, n_new)
    steps = 0
    while eng.active_count() > 0 and steps < 2000:
        eng.step()
        steps += 1
        if hook:
            hook(eng, kv, steps)
    out = {i + 1: eng.result(i + 1) for i in range(len(prompts))}
    status = {i + 1: eng.request_status(i + 1) for i in range(len(prompts))}
    stats = eng.pressure_stats()
    free, err, active = eng.free_pages(), kv.error_word(), eng.active_count()
    refs = sum(kv.ref_counts())
    eng.close()
    kv.close()
    return out, status, stats, (free, err, active, refs, steps)


def test_pool_too_small_defers_and_preempts_instead_of_failing():
    """Six requests that need 30 pages between them in a pool of 20: admission takes one page each
    (src/scheduler.zig:242,291-293), decode growth then finds the pool empty (src/kvcache/paged.zig:525-531).
    The step must not fail: requests whose growth does not fit wait, and when all are blocked the
    youngest gives its pages back and is prefilled again later.  Every request still delivers all its
    tokens, equal to the oracle's (and to an unpressured run's, up to near-ties), and every page returns."""
    from dmlx_b200 import device as dev
    from dmlx_b200 import _lib

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (100, 90, 110, 95, 120, 105)]
    n_new = 40
    roomy, st_r, stats_r, (free_r, err_r, act_r, refs_r, _) = _run_engine(dev, cfg, model, prompts, n_new, 64)
    assert stats_r == (0, 0, 0) and (free_r, err_r, act_r, refs_r) == (64, 0, 0, 0)
    tight, st_t, stats_t, (free_t, err_t, act_t, refs_t, steps_t) = _run_engine(dev, cfg, model, prompts, n_new, 20)
    assert (free_t, err_t, act_t, refs_t) == (20, 0, 0, 0), (free_t, err_t, act_t, refs_t)
    assert stats_t[0] > 0 and stats_t[2] == 0, stats_t  # requests waited for pages, nobody failed
    same = 0
    for i, p in enumerate(prompts):
        got, done = tight[i + 1]
        assert done and len(got) == n_new and st_t[i + 1] == _lib.OK
        _check_against_oracle(cfg, weights, p, got, i)
        same += got == roomy[i + 1][0]
    assert same >= 3, same  # a recomputed cache may flip a near-tie, most sequences do not meet one
    model.close()


def test_two_requests_blocked_on_the_same_step_preempt_the_younger():
    """Two requests of equal length in a pool that holds both prompts but not both outputs: at the step
    where each needs its fifth page none is free and both are blocked.  The younger one gives its pages
    back, waits (its whole prompt, now including what it has generated, must fit before it returns), is
    prefilled again and finishes with the tokens the oracle decodes for it."""
    from dmlx_b200 import device as dev
    from dmlx_b200 import _lib

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    rng = np.random.default_rng(15)
    prompts = [rng.integers(0, cfg.vocab, 96).tolist() for _ in range(2)]
    out, status, stats, (free, err, active, refs, steps) = _run_engine(dev, cfg, model, prompts, 40, 8)
    assert (free, err, active, refs) == (8, 0, 0, 0)
    assert stats[1] == 1 and stats[2] == 0, stats   # exactly one preemption, nobody failed
    for rid in (1, 2):
        got, done = out[rid]
        assert done and len(got) == 40 and status[rid] == _lib.OK
        _check_against_oracle(cfg, weights, prompts[rid - 1], got, rid)
    model.close()


def test_cancel_waiting_prefilling_and_decoding_requests():
    """b200_engine_cancel (RequestState.cancelled, src/engine/request_state.zig:118,182-189): a request
    leaves at once wherever it is, its pages return, what it produced stays readable, and the other
    requests decode what they decode without it."""
    from dmlx_b200 import device as dev
    from dmlx_b200 import _lib

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (40, 200, 50, 30)]
    kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 32, 3, 16, cfg.n_heads, max_rows=1024,
                          attn_scratch_chunks=8192)   # three sequence slots: the fourth request waits
    eng = dev.Engine(model, kv, max_prefill_tokens=64)
    for i, p in enumerate(prompts):
        eng.submit(i + 1, p, 12)
    eng.step()
    eng.step()                      # 1 and 3 decode, 2 is in the middle of its prefill, 4 waits for a slot
    assert eng.request_slot(4) == -1
    held_before = 32 - eng.free_pages()
    eng.cancel(2)                   # mid-prefill: 128 of 200 prompt tokens cached = 4 pages
    assert eng.request_status(2) == _lib.ERR_CANCELLED and eng.result(2) == ([], True)
    assert 32 - eng.free_pages() == held_before - 4
    eng.cancel(4)                   # still waiting
    assert eng.request_status(4) == _lib.ERR_CANCELLED and eng.active_count() == 2
    for _ in range(3):
        eng.step()
    got3_before = eng.result(3)[0]
    eng.cancel(3)                   # decoding
    assert eng.request_status(3) == _lib.ERR_CANCELLED and eng.result(3) == (got3_before, True) and len(got3_before) == 5
    with pytest.raises(_lib.B200Error):
        eng.cancel(99)
    steps = 0
    while eng.active_count() > 0 and steps < 100:
        eng.step()
        steps += 1
    got1, done1 = eng.result(1)
    assert done1 and len(got1) == 12 and eng.request_status(1) == _lib.OK
    _check_against_oracle(cfg, weights, prompts[0], got1, 1)
    _check_against_oracle(cfg, weights, prompts[2], got3_before, 3)
    assert eng.free_pages() == 32 and sum(kv.ref_counts()) == 0 and kv.error_word() == 0
    eng.close()
    model.close()
    kv.close()


def test_sequence_that_outgrows_its_page_table_fails_alone():
    """Per-request isolation (handleBatchError, src/engine/engine_loop.zig:687-754): a sequence that
    reaches the length its page table holds (3 pages = 96 tokens here) ends with CacheOverflow's code,
    keeps the tokens it produced, and the rest of the batch finishes normally.  A prompt that can never
    fit is refused at submission."""
    from dmlx_b200 import device as dev
    from dmlx_b200 import _lib

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (80, 20, 33)]
    out, status, stats, (free, err, active, refs, _) = _run_engine(dev, cfg, model, prompts, 40, 24, max_pages_per_seq=3)
    assert (free, err, active, refs) == (24, 0, 0, 0)
    got1, done1 = out[1]
    assert done1 and status[1] == _lib.ERR_CAPACITY and len(got1) == 96 - 80 + 1 and stats[2] == 1
    for rid in (2, 3):
        got, done = out[rid]
        assert done and status[rid] == _lib.OK and len(got) == 40
        _check_against_oracle(cfg, weights, prompts[rid - 1], got, rid)
    _check_against_oracle(cfg, weights, prompts[0], got1, 1)
    kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 24, 4, 3, cfg.n_heads, max_rows=1024)
    eng = dev.Engine(model, kv, max_prefill_tokens=64)
    with pytest.raises(_lib.B200Error) as ei:
        eng.submit(1, list(range(96)), 4)
    assert ei.value.status == _lib.ERR_CAPACITY
    eng.close()
    kv.close()
    model.close()


@pytest.mark.parametrize("own_stream", [False, True])  # True: decode steps are replayed as CUDA graphs
def test_flagged_step_leaves_state_intact_and_can_be_retried(own_stream):
    """A model step whose page reservation is flagged (pool exhausted) must change nothing: not the
    pool (the reservation is all or nothing) and not the sequences' next input tokens.  Once a page is
    free the same step is run again and the token stream equals that of a run that never lacked pages."""
    import contextlib

    import torch

    from dmlx_b200 import device as dev
    from dmlx_b200 import _lib

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    ctx = (lambda: torch.cuda.stream(torch.cuda.Stream())) if own_stream else contextlib.nullcontext
    rng = np.random.default_rng(10)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (62, 40)]

    def run(n_pages, starve):
        kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, n_pages, 4, 8, cfg.n_heads, max_rows=1024)
        for s in (0, 1):
            kv.alloc(s, 1)
        if starve:
            kv.alloc(2, n_pages - 4)  # a third slot holds every page the two sequences will not own after prefill
        descs = [(0, len(prompts[0]), 0, 0), (1, len(prompts[1]), 0, len(prompts[0]))]
        toks, _ = model.step(kv, descs, prompts[0] + prompts[1])
        stream = [list(map(int, toks))]
        flagged = 0
        for _ in range(6):
            d = [(0, 1, kv.seq_len(0), -1), (1, 1, kv.seq_len(1), -1)]
            try:
                toks, _ = model.step(kv, d, [])
            except _lib.B200Error as e:
                assert e.status == _lib.ERR_INSUFFICIENT_BLOCKS and starve
                flagged += 1
                kv.release([2])       # the pages come back; same step again
                toks, _ = model.step(kv, d, [])
            stream.append(list(map(int, toks)))
        lens = (kv.seq_len(0), kv.seq_len(1))
        kv.close()
        return stream, flagged, lens

    with ctx():
        want, f0, lens0 = run(12, False)
        got, f1, lens1 = run(12, True)
    torch.cuda.synchronize()
    assert f0 == 0 and f1 == 1          # sequence 0 needs its third page at 64 tokens and finds none
    assert lens0 == lens1 == (62 + 6, 40 + 6)
    assert got == want
    model.close()


def test_decode_graph_survives_growth_of_the_matmul_scratch():
    """Captured decode steps carry the address of the split-K scratch.  A later, larger matmul makes the
    library grow that scratch; the old buffer must stay alive for the graphs that still write to it.
    Decode steps replayed after the growth must produce what the same steps produce without it."""
    import torch

    from dmlx_b200 import device as dev

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    rng = np.random.default_rng(12)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (50, 70, 33)]
    big = dev.QWeight.random(dev.Q_AFFINE4_G64, 8192, 256, seed=3)
    xb = torch.zeros(4096, 256, dtype=torch.bfloat16, device="cuda")

    def run(grow):
        kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 32, 4, 8, cfg.n_heads, max_rows=1024)
        off, descs, flat = 0, [], []
        for s, p in enumerate(prompts):
            kv.alloc(s, 1)
            descs.append((s, len(p), 0, off))
            flat += p
            off += len(p)
        toks, _ = model.step(kv, descs, flat)
        stream = [list(map(int, toks))]
        for j in range(8):
            if grow and j == 4:
                # 4096 rows x 8192 columns of f32 partials on the CUDA-core path: twice the initial scratch
                dev.qmm(big, xb, path=dev.QMM_SIMT)
                torch.cuda.synchronize()
            d = [(s, 1, kv.seq_len(s), -1) for s in range(len(prompts))]
            toks, _ = model.step(kv, d, [])
            stream.append(list(map(int, toks)))
        logits = model.last_logits(len(prompts)).copy()
        kv.close()
        return stream, logits

    with torch.cuda.stream(torch.cuda.Stream()):  # the legacy default stream cannot be captured
        s0, l0 = run(False)
        s1, l1 = run(True)
    torch.cuda.synchronize()
    assert s0 == s1 and np.array_equal(l0, l1)
    assert dev.qmm_error_word() == 0
    del big
    model.close()


def test_prefix_sharing_through_engine():
    """Config 5 in small: requests that share a prompt prefix take over the donor's full pages by
    reference count when they start their prefill (findCachedPrefix, src/kvcache/paged.zig:234-265),
    prefill only their own suffix in chunks, copy a shared page on write, and still decode what the
    oracle decodes for the whole prompt.  Integer state is checked exactly: tokens taken over,
    reference counts of the shared pages, every page returned at the end."""
    from dmlx_b200 import device as dev

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 96, 16, 16, cfg.n_heads, max_rows=1024,
                          attn_scratch_chunks=8192)
    eng = dev.Engine(model, kv, max_prefill_tokens=64)
    eng.set_prefix_sharing(True)
    rng = np.random.default_rng(9)
    prefix = rng.integers(0, cfg.vocab, 100).tolist()  # 3 full pages + 4 tokens
    suffix_lens = [20, 5, 70, 33, 1, 64]
    prompts = [prefix + rng.integers(0, cfg.vocab, n).tolist() for n in suffix_lens]
    prompts.append(rng.integers(0, cfg.vocab, 50).tolist())  # unrelated prompt
    n_new = 12
    eng.submit(1, prompts[0], n_new)  # the donor prefills 120 tokens in two chunks
    for _ in range(3):
        eng.step()
    for i in range(1, len(prompts)):
        eng.submit(i + 1, prompts[i], n_new)
    eng.step()  # the sharers start: 96 tokens each come from the donor's pages
    donor_pages = kv.block_table(0)[:3]
    refs = kv.ref_counts()
    assert [eng.shared_tokens(i + 1) for i in range(len(prompts))] == [0, 96, 96, 96, 96, 96, 0]
    assert [refs[p] for p in donor_pages] == [6, 6, 6]
    steps = 0
    while eng.active_count() > 0 and steps < 200:
        eng.step()
        steps += 1
    assert eng.active_count() == 0 and kv.error_word() == 0
    assert eng.free_pages() == 96 and sum(kv.ref_counts()) == 0
    exact = 0
    for i, p in enumerate(prompts):
        got, done = eng.result(i + 1)
        assert done and len(got) == n_new
        exact += _check_against_oracle(cfg, weights, p, got, i)
    assert exact >= 1
    eng.close()
    model.close()
    kv.close()


def test_step_token_budget_defers_prefill_chunks():
    """b200_engine_set_max_step_tokens: with a budget smaller than the prompts waiting, prefill chunks
    queue up over several steps (a request left out of a step keeps its cursor,
    src/scheduler.zig:335-349 advances only requests it gets an output for); decode rows never wait.
    Results still equal the oracle, every page comes back."""
    from dmlx_b200 import device as dev

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 64, 16, 16, cfg.n_heads, max_rows=1024,
                          attn_scratch_chunks=8192)
    eng = dev.Engine(model, kv, max_prefill_tokens=64)
    eng.set_max_step_tokens(100)
    rng = np.random.default_rng(77)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (150, 40, 90, 64, 200)]
    for i, p in enumerate(prompts):
        eng.submit(i + 1, p, 10)
    steps, max_rows_seen = 0, 0
    while eng.active_count() > 0 and steps < 300:
        eng.step()
        steps += 1
    assert eng.active_count() == 0 and kv.error_word() == 0 and eng.free_pages() == 64
    # 544 prompt tokens at <= 100 per step cannot finish in fewer steps than this
    assert steps >= 6 + 9
    exact = 0
    for i, p in enumerate(prompts):
        got, done = eng.result(i + 1)
        assert done and len(got) == 10
        exact += _check_against_oracle(cfg, weights, p, got, i)
    assert exact >= 1
    eng.close()
    model.close()
    kv.close()


@pytest.mark.parametrize("kv_dtype_name", ["KV_BF16", "KV_FP8_E4M3"])
def test_prefix_restored_from_disk_serves_later_requests(tmp_path, kv_dtype_name):
    """Prefix pages that outlive their request (src/kvcache/prefix_disk.zig:96-293): the prompt blocks
    of a running request are saved to disk; a second engine with a fresh pool restores them into a
    parked slot, publishes it, and requests with the same leading blocks take them over by reference
    count instead of prefilling them.  Decoded ids equal the oracle's for the whole prompt (bf16
    pool) or the ids of a control engine that prefilled everything (FP8 pool); every page returns."""
    from dmlx_b200 import device as dev
    from dmlx_b200.prefix_store import PrefixDiskStore

    cfg = CFG
    kv_dtype = getattr(dev, kv_dtype_name)
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    store = PrefixDiskStore(str(tmp_path / "cold"))
    rng = np.random.default_rng(21)
    first = rng.integers(0, cfg.vocab, 100).tolist()  # 3 full blocks + 4 tokens
    later = [first[:96] + rng.integers(0, cfg.vocab, n).tolist() for n in (9, 40)] + [first[:64] + rng.integers(0, cfg.vocab, 30).tolist()]
    n_new = 8

    def pool():
        return dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 48, 8, 16, cfg.n_heads, max_rows=1024,
                                attn_scratch_chunks=8192, kv_dtype=kv_dtype)

    kv_a = pool()
    eng = dev.Engine(model, kv_a, max_prefill_tokens=64)
    eng.submit(1, first, n_new)
    eng.step()
    eng.step()  # 100 prompt tokens in two chunks
    assert store.save_prefix(kv_a, eng.request_slot(1), first) == 3
    while eng.active_count() > 0:
        eng.step()
    assert eng.request_slot(99) == -1
    eng.close()
    kv_a.close()

    def serve(with_store):
        kv = pool()
        e = dev.Engine(model, kv, max_prefill_tokens=64)
        slot = None
        if with_store:
            e.set_prefix_sharing(True)
            slot = e.park_slot()
            restored = store.restore_prefix(kv, slot, first)  # every stored block of that prompt
            assert restored == 96
            e.publish_prefix(slot, first[:restored])
            assert e.free_pages() == 48 - 3
        for i, p in enumerate(later):
            e.submit(i + 1, p, n_new)
        steps = 0
        while e.active_count() > 0 and steps < 100:
            e.step()
            steps += 1
            if with_store and steps == 1:
                assert [e.shared_tokens(i + 1) for i in range(3)] == [96, 96, 64]
                parked = kv.block_table(slot)
                assert [kv.ref_counts()[p] for p in parked] == [4, 4, 3]
        assert e.active_count() == 0 and kv.error_word() == 0
        out = [e.result(i + 1)[0] for i in range(3)]
        if with_store:
            assert e.free_pages() == 48 - 3  # only the parked prefix is left
            e.drop_prefix(slot)
        assert e.free_pages() == 48 and sum(kv.ref_counts()) == 0
        e.close()
        kv.close()
        return out

    got = serve(True)
    if kv_dtype == dev.KV_BF16:
        assert sum(_check_against_oracle(cfg, weights, p, g, i) for i, (p, g) in enumerate(zip(later, got))) >= 1
    else:
        control = serve(False)
        # the chunking differs between the two runs, and with it the bf16 rounding of what is
        # quantised into the pages: sequences may part at a near-tie, their first tokens rarely do
        assert all(len(g) == n_new for g in got)
        assert sum(a[0] == b[0] for a, b in zip(got, control)) >= 2, (got, control)
    model.close()


def test_prefix_tier_lru_between_pool_and_disk(tmp_path):
    """PrefixTier: prompts' blocks are written to disk while their requests run; later requests find
    them restored into parked slots (hot tier) and take them over; when the parked pages exceed the
    cap the least recently used prefix leaves the pool and is restored from disk again on its next
    use.  Integer state is checked exactly (tokens taken over, evictions, restores, pages)."""
    from dmlx_b200 import device as dev
    from dmlx_b200.prefix_store import PrefixDiskStore, PrefixTier

    cfg = CFG
    weights = ref_math.random_llama_weights(cfg, seed=2026)
    model = _build_model(dev, cfg, weights)
    kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 64, 8, 16, cfg.n_heads, max_rows=1024,
                          attn_scratch_chunks=8192)
    eng = dev.Engine(model, kv, max_prefill_tokens=128)
    tier = PrefixTier(eng, kv, PrefixDiskStore(str(tmp_path / "cold")), max_parked_pages=5)
    rng = np.random.default_rng(33)
    pa = rng.integers(0, cfg.vocab, 100).tolist()  # 3 full blocks
    pb = rng.integers(0, cfg.vocab, 70).tolist()   # 2 full blocks
    pc = rng.integers(0, cfg.vocab, 130).tolist()  # 4 full blocks

    def run(rid, prompt, n_new=4):
        taken = tier.prepare(prompt)
        eng.submit(rid, prompt, n_new)
        eng.step()
        wrote = tier.retire(rid, prompt)
        while eng.active_count() > 0:
            eng.step()
        assert eng.shared_tokens(rid) == taken
        return taken, wrote, eng.result(rid)[0]

    assert run(1, pa)[:2] == (0, 3) and run(2, pb)[:2] == (0, 2) and run(3, pc)[:2] == (0, 4)
    assert tier.parked_pages() == 0 and eng.free_pages() == 64
    # second round: everything comes from disk into parked slots; the cap of 5 pages holds a + b, then c evicts both
    sa = pa[:96] + rng.integers(0, cfg.vocab, 20).tolist()
    sb = pb[:64] + rng.integers(0, cfg.vocab, 11).tolist()
    sc = pc[:128] + rng.integers(0, cfg.vocab, 9).tolist()
    ta, wa, out_a = run(11, sa)
    assert (ta, wa) == (96, 0) and tier.parked_pages() == 3 and tier.restored_blocks == 3
    tb, _, _ = run(12, sb)
    assert tb == 64 and tier.parked_pages() == 5 and tier.evictions == 0
    ta2, _, out_a2 = run(13, sa)  # hot hit: no restore, and a becomes the most recently used
    assert ta2 == 96 and tier.restored_blocks == 5 and out_a2 == out_a
    tc, _, _ = run(14, sc)        # 4 more pages: b (least recently used) goes first, then a
    assert tc == 128 and tier.evictions == 2 and tier.parked_pages() == 4
    tb2, _, _ = run(15, sb)       # b again: 4 + 2 > 5, so c is evicted and b restored from disk
    assert tb2 == 64 and tier.evictions == 3 and tier.restored_blocks == 11 and tier.parked_pages() == 2
    assert eng.free_pages() == 64 - 2 and kv.error_word() == 0
    exact = _check_against_oracle(cfg, weights, sa, out_a, "a") + _check_against_oracle(cfg, weights, sa, out_a2, "a2")
    assert exact >= 0
    while tier.evict_lru():
        pass
    assert eng.free_pages() == 64 and sum(kv.ref_counts()) == 0
    eng.close()
    model.close()
    kv.close()


def test_step_with_rope_and_append_fed_from_partial_sums_equals_the_two_kernel_step():
    """With head_dim 128 and a bf16 pool the model step hands the q/k/v projection's split-K partial sums to
    RoPE + append (b200_kv_rope_append_partials).  Prefill of three prompts and 12 decode steps, fused against
    unfused on the same model: same tokens, bit-identical logits of the last step, bit-identical pages."""
    import torch

    from dmlx_b200 import device as dev

    # int4 weights generated on the device, hidden 2048: the q/k/v projection (1024 x 2048) splits K at these row counts
    cfg = ref_math.LlamaConfig(n_layers=3, hidden=2048, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1408, vocab=32000)
    model = dev.LlamaModel(cfg.n_layers, cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab,
                           max_rows=1024, max_reqs=16, max_seqs=16, rms_eps=cfg.eps, rope_theta=cfg.theta)
    model.random_init(dev.Q_AFFINE4_G64, seed=5)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (45, 130, 7)]

    def run(fused):
        model.set_fused_qkv_rope(fused)
        kv = dev.PagedKVCache(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 32, 4, 8, cfg.n_heads, max_rows=1024)
        kv.set_free_order(list(range(32)))
        off, descs, flat = 0, [], []
        for s, p in enumerate(prompts):
            kv.alloc(s, 1)
            descs.append((s, len(p), 0, off))
            flat += p
            off += len(p)
        before = model.launch_count()
        toks, _ = model.step(kv, descs, flat)
        prefill_launches = model.launch_count() - before
        stream = [list(map(int, toks))]
        for _ in range(12):
            d = [(s, 1, kv.seq_len(s), -1) for s in range(len(prompts))]
            toks, _ = model.step(kv, d, [])
            stream.append(list(map(int, toks)))
        logits = model.last_logits(len(prompts)).copy()
        pages = [[t.view(torch.int16).cpu().numpy() for t in kv.gather(l, s)] for l in range(cfg.n_layers) for s in range(len(prompts))]
        assert kv.error_word() == 0
        kv.close()
        return stream, logits, pages, prefill_launches

    with torch.cuda.stream(torch.cuda.Stream()):  # decode steps replay as graphs on a capturable stream
        s0, l0, p0, n0 = run(False)
        s1, l1, p1, n1 = run(True)
    model.set_fused_qkv_rope(True)
    assert s0 == s1
    assert np.array_equal(l0, l1)
    for (k0, v0), (k1, v1) in zip(p0, p1):
        assert np.array_equal(k0, k1) and np.array_equal(v0, v1)
    assert n1 == n0 - cfg.n_layers   # the prefill step: one launch less per layer (the projection's finish pass)

