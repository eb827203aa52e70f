"""GPU parity of MoE routing, grouping, the ragged grouped matmul and the whole layer against the
oracle (src/moe_router.zig:55-164, src/models/deepseek_v4.zig:546-681,721-848,1010-1056)."""
import numpy as np
import pytest
import torch

from oracle import ref_math

pytestmark = pytest.mark.gpu


def _bits(a):
    return (ref_math.bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def _close(got, want):
    g, w = np.asarray(got, np.float64).reshape(-1), np.asarray(want, np.float64).reshape(-1)
    return np.abs(g - w).max() / max(np.abs(w).max(), 1e-30), g @ w / (np.linalg.norm(g) * np.linalg.norm(w) + 1e-30)


@pytest.mark.parametrize("scoring", ["softmax", "sigmoid", "sqrtsoftplus"])
def test_route_matches_gate_forward(scoring):
    """Expert indices equal the oracle's wherever its decision margin is above f32 rounding of the
    scoring function; weights within 1e-5 relative."""
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(18)
    n, e, k = 512, 256, 6
    logits = rng.normal(0, 1, (n, e)).astype(np.float32)
    bias = rng.normal(0, 0.02, e).astype(np.float32)
    w_ref, i_ref = ref_math.gate_forward(logits, bias, k, route_scale=1.5, scoring=scoring)
    sc = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}[scoring]
    idx, w, counts = dev.moe_route(torch.tensor(logits, device="cuda"), k, torch.tensor(bias, device="cuda"), sc, 1.5)
    idx, w = idx.cpu().numpy().astype(np.uint32), w.cpu().numpy()
    same = (idx == i_ref).all(axis=1)
    assert same.mean() >= 0.99, same.mean()
    assert np.allclose(w[same], w_ref[same], rtol=2e-5, atol=1e-9)
    assert counts.cpu().numpy().sum() == n * k
    assert np.array_equal(counts.cpu().numpy(), np.bincount(idx.reshape(-1), minlength=e))
    for t in np.where(~same)[0]:  # a disagreement is a swap at a near-tie: same set, or one expert exchanged
        assert len(set(idx[t].tolist()) ^ set(i_ref[t].tolist())) in (0, 2)


def test_route_tie_rule():
    """Equal scores: the larger expert index wins and comes last (ascending stable argsort, last k;
    src/moe_router.zig:59-73)."""
    from dmlx_b200 import device as dev

    logits = torch.zeros((3, 8), dtype=torch.float32, device="cuda")
    idx, w, _ = dev.moe_route(logits, 3)
    assert idx.cpu().numpy().tolist() == [[5, 6, 7]] * 3
    assert ref_math.topk_route(np.zeros((1, 8), np.float32), 3).tolist() == [[5, 6, 7]]
    assert np.allclose(w.cpu().numpy(), 1.0 / 8)


def test_group_bit_exact():
    """order / inv_order / offsets equal a stable host sort (src/models/deepseek_v4.zig:747-784)."""
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(3)
    for n, e, k, tile in ((4096, 256, 6, 128), (37, 8, 2, 16), (1, 4, 4, 64)):
        p = rng.random(e) ** 3  # skewed load
        idx = np.stack([rng.choice(e, k, replace=False, p=p / p.sum()) for _ in range(n)]).astype(np.int32)
        counts = np.bincount(idx.reshape(-1), minlength=e).astype(np.int32)
        off, order, inv, items, n_items = dev.moe_group(torch.tensor(idx, device="cuda"), torch.tensor(counts, device="cuda"), tile)
        o_ref, i_ref, tok_ref, off_ref = ref_math.group_by_expert(idx, e)
        assert np.array_equal(off.cpu().numpy(), off_ref)
        assert np.array_equal(order.cpu().numpy(), o_ref) and np.array_equal(inv.cpu().numpy(), i_ref)
        ni = int(n_items.cpu()[0])
        it = items.cpu().numpy()[:ni]
        assert ni == sum(-(-c // tile) for c in counts)
        covered = np.zeros(n * k, np.int32)
        for ex, r0, rows, _ in it:
            assert off_ref[ex] <= r0 and r0 + rows <= off_ref[ex + 1] and 0 < rows <= tile
            covered[r0:r0 + rows] += 1
        assert (covered == 1).all()


@pytest.fixture
def _restore_grouped_path():
    yield
    from dmlx_b200 import device as dev

    dev.set_qmm_grouped_block_scaled(True)  # the library default


@pytest.mark.parametrize("mode_name", ["mxfp4", "affine4", "mxfp4_block_scaled"])
def test_moe_layer_matches_oracle(mode_name, _restore_grouped_path):
    from dmlx_b200 import device as dev

    # "mxfp4" runs the grouped matmuls on the dequantising kernel, the third variant on tcgen05.mma
    # kind::mxf8f6f4 (the default for MXFP4 weights)
    dev.set_qmm_grouped_block_scaled(mode_name == "mxfp4_block_scaled")
    mode_name = "mxfp4" if mode_name == "mxfp4_block_scaled" else mode_name
    rng = np.random.default_rng(11)
    n, d, e, inter, k = 70, 256, 8, 128, 2
    x = ref_math.bf16_round(rng.normal(0, 1, (n, d)))
    wg = ref_math.bf16_round(rng.normal(0, 0.3, (e, d)))
    bias = rng.normal(0, 0.01, e).astype(np.float32)

    def make(n_e, rows, cols):
        """-> (QWeight, dequantised [n_e, rows, cols])"""
        if mode_name == "mxfp4":
            packed = rng.integers(0, 256, (n_e * rows, cols // 2), dtype=np.uint8)
            scales = rng.integers(118, 122, (n_e * rows, cols // 32), dtype=np.uint8)
            w = dev.QWeight(dev.Q_MXFP4_G32, packed, scales, None, rows, cols, n_experts=n_e)
            return w, ref_math.dequantize_mxfp4(packed, scales).reshape(n_e, rows, cols)
        wf = rng.normal(0, 0.05, (n_e * rows, cols)).astype(np.float32)
        packed, s, b = ref_math.quantize_affine4(wf)
        w = dev.QWeight(dev.Q_AFFINE4_G64, packed, _bits(s), _bits(b), rows, cols, n_experts=n_e)
        return w, ref_math.dequantize_affine4(packed, s, b).reshape(n_e, rows, cols)

    gu, gu_deq = make(e, 2 * inter, d)      # rows interleaved: 2i = gate_i, 2i+1 = up_i
    down, down_deq = make(e, d, inter)
    sgu, sgu_deq = make(1, 2 * inter, d)
    sdown, sdown_deq = make(1, d, inter)
    gate = dev.QWeight(dev.Q_BF16, _bits(wg), np.zeros(1, np.uint8), None, e, d)
    layer = dev.MoELayer(d, e, inter, k, gate, gu, down, sgu, sdown, bias=bias, route_scale=1.5, swiglu_limit=10.0,
                         tile_rows=32, max_tokens=128)
    got = layer.forward(torch.tensor(x, device="cuda").bfloat16()).float().cpu().numpy()
    assert dev.qmm_error_word() == 0
    idx, wts, off = layer.last_routing(n)
    # routing against the oracle on bf16 logits (the reference's matmul output dtype)
    logits = ref_math.bf16_round(x.astype(np.float64) @ wg.astype(np.float64).T)
    w_ref, i_ref = ref_math.gate_forward(logits, bias, k, route_scale=1.5)
    same = (idx == i_ref).all(axis=1)
    assert same.mean() >= 0.95
    assert np.array_equal(off, ref_math.group_by_expert(idx, e)[3])
    # layer output against the oracle evaluated with the routing the device chose
    routed = ref_math.switch_glu(x, idx, wts, gu_deq[:, 0::2], gu_deq[:, 1::2], down_deq, limit=10.0)
    shared = ref_math.expert_forward(x, sgu_deq[0, 0::2], sgu_deq[0, 1::2], sdown_deq[0], limit=0.0)
    rel, cos = _close(got, routed + shared)
    assert rel <= 2e-2 and cos >= 0.9995, (rel, cos)


@pytest.mark.parametrize("tile_rows", [128, 112])  # 112: two accumulator sets in tensor memory, work items alternate
def test_moe_layer_at_full_size_against_the_oracle_on_sampled_tokens(tile_rows, _restore_grouped_path):
    """The MoE workload's own shape: hidden 4096, 256 routed experts of intermediate 2048 plus a shared
    expert, top-6 softmax routing with a skewed per-expert bias, 4096 tokens in one step, MXFP4 weights
    generated on the device.  Routing and grouping are checked for all tokens; the layer output of 10
    sampled tokens is compared with the oracle, which reads the experts' weights back from the device
    (b200_qweight_export) and evaluates each sampled token through its six experts and the shared one."""
    # (10 tokens x 7 experts: reading a weight back costs more than evaluating it)
    from dmlx_b200 import device as dev

    rng = np.random.default_rng(4)
    n, d, e, inter, k = 4096, 4096, 256, 2048, 6
    x = ref_math.bf16_round(rng.normal(0, 1, (n, d)))
    wg = ref_math.bf16_round(rng.normal(0, 0.02, (e, d)))
    bias = (rng.normal(0, 1, e) * 0.004).astype(np.float32)
    gate = dev.QWeight(dev.Q_BF16, _bits(wg), np.zeros(1, np.uint8), None, e, d)
    gu = dev.QWeight.random(dev.Q_MXFP4_G32, 2 * inter, d, e, seed=21)
    down = dev.QWeight.random(dev.Q_MXFP4_G32, d, inter, e, seed=22)
    sgu = dev.QWeight.random(dev.Q_MXFP4_G32, 2 * inter, d, 1, seed=23)
    sdown = dev.QWeight.random(dev.Q_MXFP4_G32, d, inter, 1, seed=24)
    layer = dev.MoELayer(d, e, inter, k, gate, gu, down, sgu, sdown, bias=bias, route_scale=1.5, swiglu_limit=10.0,
                         tile_rows=tile_rows, max_tokens=n)
    got = layer.forward(torch.tensor(x, device="cuda").bfloat16()).float().cpu().numpy()
    assert dev.qmm_error_word() == 0
    idx, wts, off = layer.last_routing(n)
    logits = ref_math.bf16_round(x.astype(np.float64) @ wg.astype(np.float64).T)
    w_ref, i_ref = ref_math.gate_forward(logits, bias, k, route_scale=1.5)
    same = (idx == i_ref).all(axis=1)
    assert same.mean() >= 0.97, same.mean()   # the rest are swaps at near-ties of bf16 logits
    # the device's gate matmul and the oracle may round a logit to neighbouring bf16 values (one ulp of a
    # logit near 4 is 2^-6, i.e. 1.6 % of its softmax weight): most weights agree closely, all within 5 %
    dev_rel = np.abs(wts[same] - w_ref[same]) / w_ref[same]
    assert np.median(dev_rel) <= 1e-3 and dev_rel.max() <= 5e-2, (float(np.median(dev_rel)), float(dev_rel.max()))
    assert np.array_equal(off, ref_math.group_by_expert(idx, e)[3])
    counts = np.diff(off)
    assert counts.sum() == n * k and counts.max() > 2 * counts.mean()  # the bias skews the load
    # the oracle's matmuls run in its C twin (cross-checked against the numpy oracle in tests/test_oracle_c.py)
    from oracle import ref_c

    def expert_out(xt, gu_w, down_w, ex, limit):
        p, s, _ = gu_w.export(int(ex))
        y = ref_c.qmm_mxfp4(p, s, xt)[0].astype(np.float64)
        a = ref_math.limited_swiglu(y[0::2], y[1::2], limit).astype(np.float32)
        q, t, _ = down_w.export(int(ex))
        return ref_c.qmm_mxfp4(q, t, a[None, :])[0].astype(np.float64)

    for tkn in rng.choice(n, 10, replace=False):
        xt = x[tkn:tkn + 1]
        want = expert_out(xt, sgu, sdown, 0, 0.0)
        for j in range(k):
            want = want + float(wts[tkn, j]) * expert_out(xt, gu, down, idx[tkn, j], 10.0)
        rel, cos = _close(got[tkn], want)
        assert rel <= 2e-2 and cos >= 0.9995, (int(tkn), rel, cos)


def test_ep_plan_groups_only_the_local_experts():
    """b200_ep_plan for every rank of a group of four, on one GPU: of the assignments of all tokens a rank
    keeps those whose expert it holds, grouped by local expert in a stable order; the others are marked -1
    in inv_order.  Against a stable host sort of the same subset (src/models/deepseek_v4.zig:747-784)."""
    import ctypes as C

    from dmlx_b200 import _lib

    rng = np.random.default_rng(8)
    n, e, k, world, tile = 1000, 64, 6, 4, 32
    p = rng.random(e) ** 2
    idx = np.stack([rng.choice(e, k, replace=False, p=p / p.sum()) for _ in range(n)]).astype(np.uint32)
    counts = np.bincount(idx.reshape(-1), minlength=e).astype(np.int32)
    d_idx, d_counts = torch.tensor(idx.astype(np.int64), device="cuda").to(torch.int32), torch.tensor(counts, device="cuda")
    el, a = e // world, n * k
    for rank in range(world):
        local = torch.empty(a, dtype=torch.int32, device="cuda")
        off = torch.empty(el + 1, dtype=torch.int32, device="cuda")
        order = torch.full((a,), -7, dtype=torch.int32, device="cuda")
        inv = torch.empty(a, dtype=torch.int32, device="cuda")
        items = torch.empty((el + a // tile + 1, 4), dtype=torch.int32, device="cuda")
        n_items = torch.zeros(1, dtype=torch.int32, device="cuda")
        _lib.check(_lib.lib.b200_ep_plan(d_idx.data_ptr(), d_counts.data_ptr(), n, k, e, rank, world, tile, local.data_ptr(),
                                         off.data_ptr(), order.data_ptr(), inv.data_ptr(), items.data_ptr(), n_items.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        flat = idx.reshape(-1).astype(np.int64)
        mine = np.nonzero((flat >= rank * el) & (flat < (rank + 1) * el))[0]
        want_order = mine[np.argsort(flat[mine], kind="stable")]
        want_off = np.concatenate([[0], np.cumsum(counts[rank * el:(rank + 1) * el])])
        m = len(mine)
        assert np.array_equal(off.cpu().numpy(), want_off) and want_off[-1] == m
        assert np.array_equal(order.cpu().numpy()[:m], want_order)
        want_inv = np.full(a, -1, np.int64)
        want_inv[want_order] = np.arange(m)
        assert np.array_equal(inv.cpu().numpy(), want_inv)
        ni = int(n_items.cpu()[0])
        covered = np.zeros(m, np.int32)
        for ex, r0, rows, _ in items.cpu().numpy()[:ni]:
            assert want_off[ex] <= r0 and r0 + rows <= want_off[ex + 1] and 0 < rows <= tile
            covered[r0:r0 + rows] += 1
        assert (covered == 1).all()


@pytest.mark.parametrize("mode_name", ["mxfp4", "affine4"])
def test_expert_parallel_layer_with_a_group_of_one_equals_the_plain_layer(mode_name, _restore_grouped_path):
    """The expert-parallel code path (dispatch, replicated routing, plan, grouped matmuls on the rows that
    exist, f32 partial sums, combine, shared expert) with a communicator of one rank, where both
    collectives are identities: its output must equal the plain layer's on the same weights, and the
    watchdog must see the stream finish."""
    import torch.distributed as dist

    from dmlx_b200 import device as dev
    from dmlx_b200 import expert_parallel as ep

    rng = np.random.default_rng(12)
    n, d, e, inter, k = 90, 256, 8, 128, 2
    x = torch.tensor(ref_math.bf16_round(rng.normal(0, 1, (n, d))), device="cuda").bfloat16()
    wg = ref_math.bf16_round(rng.normal(0, 0.3, (e, d)))
    bias = rng.normal(0, 0.01, e).astype(np.float32)
    mode = dev.Q_MXFP4_G32 if mode_name == "mxfp4" else dev.Q_AFFINE4_G64
    gate = dev.QWeight(dev.Q_BF16, _bits(wg), np.zeros(1, np.uint8), None, e, d)
    gu = dev.QWeight.random(mode, 2 * inter, d, e, seed=1)
    down = dev.QWeight.random(mode, d, inter, e, seed=2)
    sgu = dev.QWeight.random(mode, 2 * inter, d, 1, seed=3)
    sdown = dev.QWeight.random(mode, d, inter, 1, seed=4)
    plain = dev.MoELayer(d, e, inter, k, gate, gu, down, sgu, sdown, bias=bias, route_scale=1.5, tile_rows=32, max_tokens=128)
    want = plain.forward(x).float().cpu().numpy()
    comm = ep.Communicator(0, 1)
    layer = ep.ExpertParallelMoE(comm, d, e, inter, k, gate, gu, down, sgu, sdown, bias=bias, route_scale=1.5, tile_rows=32,
                                 max_tokens=128)
    got = layer.forward(x)
    comm.wait(timeout_ms=5000)
    got = got.float().cpu().numpy()
    assert dev.qmm_error_word() == 0
    rel, cos = _close(got, want)
    # same kernels and the same rows; only the sum over k runs in f32 here (and is rounded once)
    assert rel <= 1e-2 and cos >= 0.9999, (rel, cos)
    layer.close()
    comm.close()
    plain.close()
