"""Sampling beyond greedy (src/sampling.zig:42-375).  CPU: the oracle on hand-computed cases and the
PRNG on the published xoshiro256++ / SplitMix64 vectors, in the oracle and in the library's host
code.  GPU: b200_sample_rows against the oracle on the same logits and uniform variates.

Token equality is exact except where the uniform variate (or top_p) lies within TOL of the
cumulative probability that decides the outcome: the device's exp and its parallel whole-vocabulary
sums differ from the CPU's in the last bits.  A different token must then be the neighbour that owns
the adjoining interval (ref_sampling.acceptable_tokens)."""
import math

import numpy as np
import pytest

from oracle import ref_sampling as rs

TOL = 2e-5
LN = [math.log(v) for v in (1.0, 2.0, 3.0, 4.0)]  # softmax = 0.1, 0.2, 0.3, 0.4


def test_oracle_hand_cases():
    x = np.array(LN, np.float32)
    assert [rs.temperature_sample(x, 1.0, r)[0] for r in (0.05, 0.25, 0.55, 0.95)] == [0, 1, 2, 3]
    # top-2: tokens 3 (4/7) and 2 (3/7) in that order
    assert [rs.top_k_top_p(x, 1.0, 2, 1.0, r)[0] for r in (0.5, 0.6)] == [3, 2]
    # top-p 0.5 over all four: 0.4, then 0.7 > 0.5 closes the nucleus at two candidates
    assert [rs.top_k_top_p(x, 1.0, 4, 0.5, r)[0] for r in (0.5, 0.6)] == [3, 2]
    # equal scores keep index order (stable sort): top-2 of four equal logits is {0, 1}
    eq = np.ones(4, np.float32)
    assert [rs.top_k_top_p(eq, 1.0, 2, 1.0, r)[0] for r in (0.2, 0.7)] == [0, 1]
    # temperature sharpens: at T = 0.5 the weights are 1, 4, 9, 16 (/30)
    assert [rs.temperature_sample(x, 0.5, r)[0] for r in (0.02, 0.1, 0.4, 0.6)] == [0, 1, 2, 3]
    assert rs.temperature_sample(x, 0.0, 0.99)[0] == 3 and rs.greedy(eq) == 0
    # penalty once per occurrence: 2 -> 1 -> 0.5, -2 -> -4
    assert rs.apply_repetition_penalty(np.array([2.0, -2.0, 1.0], np.float32), [0, 0, 1, 7], 2.0).tolist() == [0.5, -4.0, 1.0]
    assert abs(rs.logprob(np.zeros(2, np.float32), 1) + math.log(2.0)) < 1e-6
    # SamplerConfig.sample: top_k >= vocab with top_p >= 1 takes the index-order path
    assert rs.sampler_config_sample(x, 1.0, 50, 1.0, 0.25)[0] == 1
    assert rs.sampler_config_sample(x, 1.0, 2, 1.0, 0.6)[0] == 2
    assert rs.acceptable_tokens(x, 1.0, 2, 1.0, 0.6, 0.0) == {2}
    assert rs.acceptable_tokens(x, 1.0, 2, 1.0, 4.0 / 7.0, 1e-3) == {2, 3}


XOSHIRO_1234 = [41943041, 58720359, 3588806011781223, 3591011842654386, 9228616714210784205, 9973669472204895162,
                14011001112246962877, 12406186145184390807, 15849039046786891736, 10450023813501588000]
SPLITMIX_1234567 = [6457827717110365317, 3203168211198807973, 9817491932198370423, 4593380528125082431]


def test_prng_known_answers_oracle_and_library():
    from dmlx_b200 import host

    o = rs.Xoshiro256(0)
    o.s = [1, 2, 3, 4]
    assert [o.next_u64() for _ in range(10)] == XOSHIRO_1234
    h = host.Prng(0)
    h.set_state([1, 2, 3, 4])
    assert [h.next_u64() for _ in range(10)] == XOSHIRO_1234
    assert rs.Xoshiro256(1234567).s == SPLITMIX_1234567  # the seeding draws are SplitMix64's outputs
    # the library and the oracle agree draw for draw, and the floats are uniform on [0, 1)
    a, b = rs.Xoshiro256(42), host.Prng(42)
    fa = [a.next_f32() for _ in range(4000)]
    fb = [b.next_f32() for _ in range(4000)]
    assert fa == fb
    assert all(0.0 <= v < 1.0 for v in fa) and abs(np.mean(fa) - 0.5) < 0.02
    assert a.next_u64() == b.next_u64()


# ---------------------------------------------------------------------------------------------------------
def _check_rows(dev, logits_t, x32, rows, context=None):
    import torch

    tokens, lp = dev.sample_rows(logits_t, rows, context=context)
    torch.cuda.synchronize()
    tokens, lp = tokens.cpu().numpy(), lp.cpu().numpy()
    exact = 0
    for i, row in enumerate(rows):
        t, k, p, u = row[:4]
        pen = row[4] if len(row) > 4 else 1.0
        ctx = context[i] if context is not None else None
        want, want_lp, _ = rs.sampler_config_sample(x32[i], t, k, p, u, pen, ctx)
        if int(tokens[i]) == want:
            exact += 1
            assert abs(float(lp[i]) - want_lp) < 2e-4 * max(1.0, abs(want_lp)), (i, row, float(lp[i]), want_lp)
        else:
            ok = rs.acceptable_tokens(x32[i], t, k, p, u, TOL, pen, ctx)
            assert int(tokens[i]) in ok, (i, row, int(tokens[i]), want, sorted(ok)[:8])
    return exact


CASES = [(0.7, 50, 1.0), (1.0, 50, 0.9), (1.3, 1, 1.0), (0.6, 0, 0.8), (1.0, 0, 1.0), (0.8, 3000, 0.95), (0.0, 50, 1.0),
         (1.0, 2048, 1.0), (1.0, 2049, 1.0), (1.0, 50000, 0.5), (0.9, 7, 0.3), (2.0, 100, 0.999), (1.0, 50, 1.5)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name,vocab", [("bfloat16", 32000), ("float32", 32000), ("bfloat16", 4099), ("float32", 130)])
def test_sample_rows_match_oracle(dtype_name, vocab):
    """Every branch of SamplerConfig.sample: greedy, the index-order softmax, top-k below and above
    the chunk capacity of the kernel (2048), top-p cuts, k = 1, k > vocab, p > 1; vocabularies with
    and without 16-byte rows.  bf16 logits carry many exactly equal scores, so the index-order tie
    rule of the stable sort is exercised at every cut."""
    import torch

    from dmlx_b200 import device as dev

    rng = np.random.default_rng(31 + vocab)
    rows = [(t, k, p, float(np.float32(rng.random()))) for (t, k, p) in CASES for _ in range(3)]
    # edge variates: 0 picks the first candidate, the largest float below 1 the last
    rows += [(1.0, 50, 0.9, 0.0), (1.0, 0, 1.0, 0.0), (1.0, 50, 1.0, float(np.nextafter(np.float32(1), np.float32(0)))),
             (1.0, 0, 1.0, float(np.nextafter(np.float32(1), np.float32(0))))]
    x = rng.normal(0.0, 3.0, (len(rows), vocab)).astype(np.float32)
    t = torch.tensor(x, device="cuda").to(getattr(torch, dtype_name)).contiguous()
    x32 = t.float().cpu().numpy()
    exact = _check_rows(dev, t, x32, rows)
    assert exact >= int(0.9 * len(rows)), (exact, len(rows))


@pytest.mark.gpu
def test_all_equal_logits_and_tiny_vocab():
    import torch

    from dmlx_b200 import device as dev

    # all scores equal: candidates are token ids in order, each with probability 1/k
    t = torch.zeros((6, 5000), dtype=torch.bfloat16, device="cuda")
    rows = [(1.0, 4, 1.0, 0.10), (1.0, 4, 1.0, 0.30), (1.0, 4, 1.0, 0.60), (1.0, 4, 1.0, 0.90), (1.0, 3000, 1.0, 0.5),
            (0.0, 4, 1.0, 0.9)]
    tokens, _ = dev.sample_rows(t, rows)
    assert tokens.cpu().tolist()[:4] == [0, 1, 2, 3] and tokens.cpu().tolist()[5] == 0
    assert tokens.cpu().tolist()[4] in (1499, 1500, 1501)  # 3000 equal candidates over two chunks
    one = torch.tensor([[0.5]], dtype=torch.float32, device="cuda")
    for row in [(1.0, 50, 1.0, 0.7), (1.0, 1, 0.5, 0.7), (0.0, 1, 1.0, 0.7)]:
        tok, lp = dev.sample_rows(one, [row])
        assert tok.item() == 0 and abs(lp.item()) < 1e-6
    x = np.array([LN], np.float32)
    for r, want in ((0.05, 0), (0.25, 1), (0.55, 2), (0.95, 3)):
        assert dev.sample_rows(torch.tensor(x, device="cuda"), [(1.0, 0, 1.0, r)])[0].item() == want
    for r, want in ((0.5, 3), (0.6, 2)):
        assert dev.sample_rows(torch.tensor(x, device="cuda"), [(1.0, 2, 1.0, r)])[0].item() == want
        assert dev.sample_rows(torch.tensor(x, device="cuda"), [(1.0, 4, 0.5, r)])[0].item() == want


@pytest.mark.gpu
def test_repetition_penalty_rows():
    import torch

    from dmlx_b200 import device as dev

    rng = np.random.default_rng(8)
    vocab, n = 8192, 12
    x = rng.normal(0.0, 3.0, (n, vocab)).astype(np.float32)
    ctx = []
    for i in range(n):
        top = np.argsort(-x[i])[:6].tolist()  # penalise the likeliest tokens, some of them repeatedly
        ctx.append([] if i == 3 else top + top[:2] * (i % 3) + [vocab + 5] + rng.integers(0, vocab, 40).tolist())
    rows = [((0.0 if i % 4 == 0 else 0.8), 50, 0.95, float(np.float32(rng.random())), (1.0 if i == 5 else 1.3)) for i in range(n)]
    for dtype in (torch.float32, torch.bfloat16):
        t = torch.tensor(x, device="cuda").to(dtype).contiguous()
        x32 = t.float().cpu().numpy()
        exact = _check_rows(dev, t, x32, rows, context=ctx)
        assert exact >= n - 2
        assert torch.equal(t.float().cpu(), torch.tensor(x32))  # the input logits are left untouched
    # greedy under the penalty moves off the penalised maximum
    want = [rs.sampler_config_sample(x[i], 0.0, 50, 1.0, 0.0, 1.3, ctx[i])[0] for i in (0, 4, 8)]
    assert want != [int(np.argmax(x[i])) for i in (0, 4, 8)]


@pytest.mark.gpu
def test_draw_frequencies_follow_the_softmax():
    """20000 rows of the same 16 logits with variates from the library's PRNG: the token histogram
    matches the softmax over the top 8 within 4 standard deviations."""
    import torch

    from dmlx_b200 import device as dev, host

    rng = np.random.default_rng(4)
    base = rng.normal(0, 1.5, 16).astype(np.float32)
    n = 20000
    prng = host.Prng(99)
    rows = [(1.0, 8, 1.0, prng.next_f32()) for _ in range(n)]
    t = torch.tensor(np.tile(base, (n, 1)), device="cuda")
    tokens, _ = dev.sample_rows(t, rows, logprobs=False)
    hist = np.bincount(tokens.cpu().numpy(), minlength=16)
    order = np.argsort(-base, kind="stable")[:8]
    p = np.exp(base[order] - base[order].max())
    p /= p.sum()
    assert hist.sum() == n and set(np.nonzero(hist)[0]) <= set(order.tolist())
    sigma = np.sqrt(n * p * (1 - p))
    assert np.all(np.abs(hist[order] - n * p) < 4 * sigma + 1), (hist[order], n * p)


@pytest.mark.gpu
def test_engine_request_with_sampler():
    """A request with a sampler draws one variate per output token from its own PRNG and the step
    samples on the device: every token is one the oracle accepts for that step's logits and that
    variate; the same seed reproduces the tokens, a request without a sampler stays greedy."""
    from dmlx_b200 import device as dev

    def run(seed, with_sampler=True, steps=10):
        model = dev.LlamaModel(2, 256, 4, 2, 64, 512, 4096, max_rows=256, max_reqs=8, max_seqs=8)
        model.random_init(dev.Q_AFFINE4_G64, seed=5)
        kv = dev.PagedKVCache(2, 2, 64, 32, 8, 8, 4, max_rows=256)
        eng = dev.Engine(model, kv, max_prefill_tokens=16)
        prompt = list(range(40, 40 + 37))  # three prefill chunks: only the last one draws
        eng.submit(1, prompt, steps)
        eng.submit(2, prompt[:9], steps)  # greedy companion in the same batch
        if with_sampler:
            eng.set_sampler(1, 0.9, 12, 0.95, seed)
        oracle_prng = rs.Xoshiro256(seed)
        n_seen = 0
        while eng.active_count() > 0:
            outs = eng.step()
            ids = [r for r, _ in outs]
            if with_sampler and 1 in ids:
                # whenever request 1 gets an output every row of the step does, so its place in the
                # outputs is its row (steps where it is still prefilling draw nothing)
                row = ids.index(1)
                logits = model.last_logits(len(outs))
                u = oracle_prng.next_f32()
                ok = rs.acceptable_tokens(logits[row], 0.9, 12, 0.95, u, TOL)
                assert outs[row][1] in ok, (n_seen, outs[row][1], sorted(ok))
                n_seen += 1
        got1, done1 = eng.result(1)
        got2, done2 = eng.result(2)
        assert n_seen == (steps if with_sampler else 0)
        assert done1 and done2 and len(got1) == steps and len(got2) == steps
        for o in (eng, model, kv):
            o.close()
        return got1, got2

    a1, a2 = run(7)
    b1, b2 = run(7)
    c1, c2 = run(8)
    g1, g2 = run(7, with_sampler=False)
    assert a1 == b1 and a2 == b2 == c2 == g2
    assert a1 != g1 or c1 != g1  # sampling at temperature 0.9 leaves the greedy path for some seed
