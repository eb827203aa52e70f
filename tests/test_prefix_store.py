"""Prefix-page persistence: the block file format (src/kvcache/prefix_disk.zig:80-83, 96-293) on CPU,
and save -> fresh pool -> restore through the C-ABI on the GPU (bit-exact pages, equal attention)."""
import json
import os
import struct

import numpy as np
import pytest

from dmlx_b200 import prefix_store as ps


def test_block_file_is_a_safetensors_container(tmp_path):
    rng = np.random.default_rng(5)
    k = rng.integers(0, 2 ** 16, (1, 2, 32, 64)).astype(np.uint16)
    v = rng.integers(0, 2 ** 16, (1, 2, 32, 64)).astype(np.uint16)
    sc = rng.normal(0, 1, 2).astype(np.float32)
    path = str(tmp_path / "prefix_00000000deadbeef.safetensors")
    ps.write_safetensors(path, {"layer_0_keys": ("BF16", k), "layer_0_values": ("BF16", v), "layer_0_key_scales": ("F32", sc)},
                         {"layer_count": 1, "block_size": 32, "block_hash": 0xDEADBEEF})
    raw = open(path, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    assert n % 8 == 0
    header = json.loads(raw[8 : 8 + n])
    assert header["__metadata__"] == {"layer_count": "1", "block_size": "32", "block_hash": str(0xDEADBEEF)}
    assert header["layer_0_keys"]["dtype"] == "BF16" and header["layer_0_keys"]["shape"] == [1, 2, 32, 64]
    a, b = header["layer_0_values"]["data_offsets"]
    assert raw[8 + n + a : 8 + n + b] == v.tobytes()
    assert len(raw) == 8 + n + 2 * k.nbytes + sc.nbytes  # offsets tile the data section exactly
    tensors, meta = ps.read_safetensors(path)
    assert np.array_equal(tensors["layer_0_keys"], k) and np.array_equal(tensors["layer_0_values"], v)
    assert np.array_equal(tensors["layer_0_key_scales"], sc)
    assert meta["block_hash"] == str(0xDEADBEEF)
    assert not os.path.exists(path + ".tmp")


def test_block_names_and_chained_hashes(tmp_path):
    from dmlx_b200 import host

    store = ps.PrefixDiskStore(str(tmp_path / "cache"))
    assert os.path.isdir(store.dir)
    assert os.path.basename(store.block_path(0x1234)) == "prefix_0000000000001234.safetensors"
    ids = list(range(100, 100 + 75))
    chain = ps.chain_hashes(ids)
    assert len(chain) == 2  # only full blocks
    h0 = host.hash_block(0, ids[:32])
    assert chain == [h0, host.hash_block(h0, ids[32:64])]
    # the same second block after a different first block hashes differently
    assert ps.chain_hashes([7] * 32 + ids[32:64])[1] != chain[1]
    assert not store.has_block(chain[0])


def test_load_block_rejects_a_renamed_file(tmp_path):
    store = ps.PrefixDiskStore(str(tmp_path))
    z = np.zeros((1, 1, 32, 8), np.uint16)
    ps.write_safetensors(store.block_path(2), {"layer_0_keys": ("BF16", z), "layer_0_values": ("BF16", z)},
                         {"layer_count": 1, "block_size": 32, "block_hash": 1})
    with pytest.raises(ValueError):
        store.load_block(2)


@pytest.mark.gpu
@pytest.mark.parametrize("kv_dtype_name", ["KV_BF16", "KV_FP8_E4M3"])
def test_save_restore_round_trip(tmp_path, kv_dtype_name):
    import torch

    from dmlx_b200 import device as dev
    from oracle import ref_math

    kv_dtype = getattr(dev, kv_dtype_name)
    L, hq, hkv, d, n_tok = 2, 8, 2, 128, 32 * 5 + 9
    rng = np.random.default_rng(77)
    ids = rng.integers(0, 32000, n_tok).tolist()

    def pool(order_seed):
        kv = dev.PagedKVCache(L, hkv, d, 24, 4, 8, hq, max_rows=256, kv_dtype=kv_dtype)
        kv.set_free_order(np.random.default_rng(order_seed).permutation(24).tolist())
        return kv

    a = pool(1)
    a.reserve(dev.pack_desc_array([(0, n_tok, 0, -1)]).cuda())
    for l in range(L):
        k = ref_math.bf16_round(rng.normal(0, 1 + l, (n_tok, hkv, d)).astype(np.float32))
        v = ref_math.bf16_round(rng.normal(0, 1, (n_tok, hkv, d)).astype(np.float32))
        a.append(l, torch.tensor(k, device="cuda").bfloat16(), torch.tensor(v, device="cuda").bfloat16())
    torch.cuda.synchronize()
    store = ps.PrefixDiskStore(str(tmp_path / "pfx"))
    assert store.save_prefix(a, 0, ids) == 5
    assert store.save_prefix(a, 0, ids) == 0  # already on disk
    assert sorted(os.listdir(store.dir)) == sorted(os.path.basename(store.block_path(h)) for h in ps.chain_hashes(ids))

    b = pool(2)  # another page order: the restored table differs, the contents must not
    assert store.restore_prefix(b, 1, ids) == 160
    assert b.seq_len(1) == 160 and len(b.block_table(1)) == 5
    assert b.block_table(1) != a.block_table(0)[:5]
    for l in range(L):
        for pa, pb in zip(a.block_table(0)[:5], b.block_table(1)):
            for x, y in zip(a.page_raw(l, pa), b.page_raw(l, pb)):
                assert np.array_equal(x, y)
        ka, va = a.gather(l, 0)
        kb, vb = b.gather(l, 1)
        assert torch.equal(ka[:160], kb) and torch.equal(va[:160], vb)
    # attention over the restored slot equals attention over the first 160 tokens of the original
    q = torch.tensor(rng.normal(0, 1, (1, hq, d)).astype(np.float32), device="cuda").bfloat16()
    ctx = torch.tensor([160], dtype=torch.int32, device="cuda")
    out_a = a.attention(1, q, torch.tensor([0], dtype=torch.int32, device="cuda"), ctx)
    out_b = b.attention(1, q, torch.tensor([1], dtype=torch.int32, device="cuda"), ctx)
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b)
    assert a.error_word() == 0 and b.error_word() == 0

    # the restored slot keeps growing like any other: its next token lands in a fresh sixth page
    b.reserve(dev.pack_desc_array([(1, 1, 160, -1)]).cuda())
    torch.cuda.synchronize()
    assert b.seq_len(1) == 161 and len(b.block_table(1)) == 6

    # a prompt that is all full blocks leaves its last block to compute; unknown prompts restore nothing
    c = pool(3)
    assert store.restore_prefix(c, 0, ids[:160]) == 128
    assert store.restore_prefix(c, 2, [1] * 64) == 0 and c.seq_len(2) == 0
    # a pool of another shape refuses the files
    other = dev.PagedKVCache(L, hkv, 64, 24, 4, 8, hq, max_rows=256, kv_dtype=kv_dtype)
    with pytest.raises(ValueError):
        store.restore_prefix(other, 0, ids)
    for p in (a, b, c, other):
        p.close()
