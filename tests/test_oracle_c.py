"""The C twin of the oracle (timed as the CPU baseline) agrees with the numpy oracle that is pinned
on the reference's golden vectors."""
import numpy as np

from oracle import ref_c, ref_math


def _bf16_bits(x):
    return (ref_math.bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def test_c_paged_attention_matches_numpy_oracle():
    rng = np.random.default_rng(0)
    hq, hkv, d = 8, 2, 64
    ctx = np.array([1, 33, 100, 0, 64], np.int32)
    n_pages = 16
    perm = rng.permutation(n_pages)
    table = np.zeros((len(ctx), 4), np.int32)
    k_pool = np.zeros((n_pages, hkv, 32, d), np.float32)
    v_pool = np.zeros((n_pages, hkv, 32, d), np.float32)
    ks, vs, nxt = [], [], 0
    for s, c in enumerate(ctx):
        k = ref_math.bf16_round(rng.normal(0, 1, (c, hkv, d)))
        v = ref_math.bf16_round(rng.normal(0, 1, (c, hkv, d)))
        ks.append(k)
        vs.append(v)
        for t in range(c):
            if t % 32 == 0:
                table[s, t // 32] = perm[nxt]
                nxt += 1
            k_pool[table[s, t // 32], :, t % 32] = k[t]
            v_pool[table[s, t // 32], :, t % 32] = v[t]
    q = rng.normal(0, 1, (len(ctx), hq, d)).astype(np.float32)
    got = ref_c.paged_attention_decode(_bf16_bits(k_pool), _bf16_bits(v_pool), table, ctx, hq, hkv, d, q)
    for s, c in enumerate(ctx):
        want = ref_math.gqa_attention_decode(q[s], ks[s], vs[s]) if c else np.zeros((hq, d), np.float32)
        assert np.allclose(got[s], want, atol=2e-5)


def test_c_qmm_matches_numpy_oracle():
    rng = np.random.default_rng(1)
    w = rng.normal(0, 0.02, (96, 256)).astype(np.float32)
    packed, s, b = ref_math.quantize_affine4(w)
    x = rng.normal(0, 1, (3, 256)).astype(np.float32)
    assert np.allclose(ref_c.qmm_affine4(packed, s, b, x), ref_math.qmm(x, ref_math.dequantize_affine4(packed, s, b)), atol=1e-4)
    pk = rng.integers(0, 256, (64, 64), dtype=np.uint8)
    sc = rng.integers(120, 130, (64, 4), dtype=np.uint8)
    x = rng.normal(0, 1, (2, 128)).astype(np.float32)
    want = ref_math.qmm(x, ref_math.dequantize_mxfp4(pk, sc))
    assert np.allclose(ref_c.qmm_mxfp4(pk, sc, x), want, rtol=1e-4, atol=1e-3 * np.abs(want).max())
    assert ref_c.num_threads() >= 1
