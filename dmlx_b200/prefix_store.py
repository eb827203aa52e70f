"""On-disk store of prefix pages: the host side of PrefixDiskCache (src/kvcache/prefix_disk.zig).

One safetensors file per 32-token block at ``{dir}/prefix_{hash:016x}.safetensors`` (:80-83) holding
``layer_{i}_keys`` / ``layer_{i}_values`` in the page shape ``[1, n_kv_heads, 32, head_dim]``
(src/kvcache/paged.zig:459-464) and the metadata ``layer_count``, ``block_size``, ``block_hash``,
``layer_{i}_ndim``, ``layer_{i}_shape_{d}`` as decimal strings (:131-168).  FP8 pools add
``layer_{i}_key_scales`` / ``layer_{i}_value_scales`` (f32 per kv head) — no reference counterpart.

Block hashes are chained over the block's token ids (hashBlock, src/kvcache/paged.zig:224-230).
This library chains FNV-1a-64 (``b200_hash_block``) where the reference uses Zig's Wyhash, so the
two never read each other's files by name; the container format and tensor names are the same.

Saving copies pages device -> host -> file; restoring allocates pages for an empty sequence slot,
loads them and sets the slot's length, after which the slot decodes as if it had prefilled those
tokens itself.  The safetensors container is written and parsed here (8-byte little-endian header
length, JSON header, raw little-endian data): no third-party package is needed.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

_DTYPES = {"BF16": np.uint16, "U8": np.uint8, "F32": np.float32}


def write_safetensors(path: str, tensors: Dict[str, Tuple[str, np.ndarray]], metadata: Dict[str, str]) -> None:
    """tensors: name -> (safetensors dtype tag, array whose bytes are stored as they are)."""
    header: Dict[str, object] = {"__metadata__": {k: str(v) for k, v in metadata.items()}}
    blobs: List[bytes] = []
    off = 0
    for name in sorted(tensors):
        tag, arr = tensors[name]
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": tag, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    os.replace(tmp, path)  # a reader never sees a half-written block


def read_safetensors(path: str) -> Tuple[Dict[str, np.ndarray], Dict[str, str]]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    meta = header.pop("__metadata__", {})
    out = {}
    for name, info in header.items():
        a, b = info["data_offsets"]
        out[name] = np.frombuffer(data[a:b], dtype=_DTYPES[info["dtype"]]).reshape(info["shape"])
    return out, meta


def chain_hashes(token_ids: Sequence[int], block_size: int = 32) -> List[int]:
    """Chained hash of every full block of the prompt (prev hash seeds the next block)."""
    from .host import hash_block

    out, h = [], 0
    for b in range(len(token_ids) // block_size):
        h = hash_block(h, token_ids[b * block_size:(b + 1) * block_size])
        out.append(h)
    return out


class PrefixDiskStore:
    """PrefixDiskCache.{init, hasBlock, saveBlock, loadBlock, restorePrefix} over a device page pool."""

    def __init__(self, cache_dir: str, block_size: int = 32):
        self.dir, self.block_size = cache_dir, block_size
        os.makedirs(cache_dir, exist_ok=True)

    def block_path(self, block_hash: int) -> str:
        return os.path.join(self.dir, f"prefix_{block_hash & (2 ** 64 - 1):016x}.safetensors")

    def has_block(self, block_hash: int) -> bool:
        return os.path.exists(self.block_path(block_hash))

    # -- one block ---------------------------------------------------------------------------
    def save_block(self, kv, page: int, block_hash: int) -> None:
        c = kv.cfg
        fp8 = c.kv_dtype != 0
        tensors, meta = {}, {"layer_count": c.n_layers, "block_size": self.block_size, "block_hash": block_hash}
        shape = (1, c.n_kv_heads, c.page_size, c.head_dim)
        for l in range(c.n_layers):
            k, v, ks, vs = kv.page_raw(l, page)
            tag = "U8" if fp8 else "BF16"
            tensors[f"layer_{l}_keys"] = (tag, k.reshape(shape))
            tensors[f"layer_{l}_values"] = (tag, v.reshape(shape))
            if fp8:
                tensors[f"layer_{l}_key_scales"] = ("F32", ks)
                tensors[f"layer_{l}_value_scales"] = ("F32", vs)
            meta[f"layer_{l}_ndim"] = len(shape)
            for d, dim in enumerate(shape):
                meta[f"layer_{l}_shape_{d}"] = dim
        write_safetensors(self.block_path(block_hash), tensors, meta)

    def load_block(self, block_hash: int):
        tensors, meta = read_safetensors(self.block_path(block_hash))
        if int(meta.get("block_size", -1)) != self.block_size or int(meta.get("block_hash", -1)) != block_hash:
            raise ValueError(f"{self.block_path(block_hash)}: metadata does not match the requested block")
        return tensors, meta

    # -- a sequence's prefix -----------------------------------------------------------------
    def save_prefix(self, kv, seq: int, token_ids: Sequence[int]) -> int:
        """Store every full block of `seq` (holding the K/V of token_ids) that is not on disk yet.
        Returns the number of blocks written."""
        table = kv.block_table(seq)
        n_full = min(kv.seq_len(seq), len(token_ids)) // self.block_size
        written = 0
        for b, h in enumerate(chain_hashes(token_ids[: n_full * self.block_size], self.block_size)):
            if not self.has_block(h):
                self.save_block(kv, table[b], h)
                written += 1
        return written

    def restore_prefix(self, kv, seq: int, token_ids: Sequence[int]) -> int:
        """Fill the empty slot `seq` with the longest run of leading blocks of token_ids found on disk
        (at least one prompt token is always left to compute).  Returns the tokens restored."""
        c = kv.cfg
        hashes = chain_hashes(token_ids, self.block_size)
        n = 0
        while n < len(hashes) and self.has_block(hashes[n]):
            n += 1
        while n > 0 and n * self.block_size >= len(token_ids):
            n -= 1
        if n == 0:
            return 0
        fp8 = c.kv_dtype != 0
        want_shape, want_dtype = (1, c.n_kv_heads, c.page_size, c.head_dim), (np.uint8 if fp8 else np.uint16)
        blocks = []
        for b in range(n):  # every block is checked before the pool is touched
            tensors, meta = self.load_block(hashes[b])
            if int(meta["layer_count"]) != c.n_layers:
                raise ValueError("stored block has a different layer count")
            for l in range(c.n_layers):
                for name in (f"layer_{l}_keys", f"layer_{l}_values"):
                    t = tensors[name]
                    if tuple(t.shape) != want_shape or t.dtype != want_dtype:
                        raise ValueError("stored block does not match the pool's page shape or element type")
                if fp8 and (f"layer_{l}_key_scales" not in tensors or f"layer_{l}_value_scales" not in tensors):
                    raise ValueError("stored FP8 block has no scales")
            blocks.append(tensors)
        pages = kv.alloc(seq, n)
        for b, tensors in enumerate(blocks):
            for l in range(c.n_layers):
                kv.page_load(l, pages[b], tensors[f"layer_{l}_keys"], tensors[f"layer_{l}_values"],
                             tensors.get(f"layer_{l}_key_scales"), tensors.get(f"layer_{l}_value_scales"))
        kv.set_len(seq, n * self.block_size)
        return n * self.block_size


class PrefixTier:
    """Two tiers for prompt prefixes around one engine: hot = parked sequence slots of the engine's
    page pool (shared into requests by reference count), cold = a PrefixDiskStore.  Least recently
    used parked prefixes are dropped when the parked pages would exceed `max_parked_pages` (their
    blocks stay on disk), the policy of TieredKVCache (src/kvcache/tiered.zig:96-275: access counter,
    findLRUPage, evict to safetensors, restore on access) applied to whole prefixes instead of single
    pages of a live sequence.
    """

    def __init__(self, engine, kv, store: PrefixDiskStore, max_parked_pages: int):
        self.engine, self.kv, self.store, self.max_parked_pages = engine, kv, store, max_parked_pages
        self._parked: Dict[int, dict] = {}  # slot -> {"chain": [...], "pages": n, "used": tick}
        self._tick = 0
        self.restored_blocks = 0
        self.evictions = 0
        engine.set_prefix_sharing(True)

    def parked_pages(self) -> int:
        return sum(e["pages"] for e in self._parked.values())

    def _touch(self, slot: int):
        self._tick += 1
        self._parked[slot]["used"] = self._tick

    def evict_lru(self) -> bool:
        if not self._parked:
            return False
        slot = min(self._parked, key=lambda s: self._parked[s]["used"])
        self.engine.drop_prefix(slot)
        del self._parked[slot]
        self.evictions += 1
        return True

    def prepare(self, token_ids: Sequence[int]) -> int:
        """Call before submitting a request: makes the longest stored run of its leading blocks
        available in the hot tier.  Returns the tokens a new request can take over."""
        bs = self.store.block_size
        chain = chain_hashes(token_ids, bs)
        on_disk = 0
        while on_disk < len(chain) and self.store.has_block(chain[on_disk]):
            on_disk += 1
        best_slot, best = None, 0
        for slot, e in self._parked.items():
            n = 0
            while n < len(chain) and n < len(e["chain"]) and chain[n] == e["chain"][n]:
                n += 1
            if n > best:
                best_slot, best = slot, n
        if best_slot is not None and best >= on_disk:
            self._touch(best_slot)
            return best * bs
        if on_disk == 0 or on_disk > self.max_parked_pages:
            if best_slot is not None:
                self._touch(best_slot)
            return best * bs
        while self.parked_pages() + on_disk > self.max_parked_pages or self.engine.free_pages() < on_disk:
            if not self.evict_lru():
                return 0
        slot = self.engine.park_slot()
        # restore_prefix leaves the last block out when the prompt ends on a block boundary; a parked
        # prefix has no token of its own to compute, so ask for every stored block
        restored = self.store.restore_prefix(self.kv, slot, list(token_ids[: on_disk * bs]) + [0])
        self.engine.publish_prefix(slot, token_ids[:restored])
        self._parked[slot] = {"chain": chain[: restored // bs], "pages": restored // bs, "used": 0}
        self._touch(slot)
        self.restored_blocks += restored // bs
        return restored

    def retire(self, rid: int, prompt: Sequence[int]) -> int:
        """Call while request `rid` is still running and has prefilled its prompt: writes its full
        prompt blocks that are not on disk yet.  Returns the blocks written."""
        slot = self.engine.request_slot(rid)
        return self.store.save_prefix(self.kv, slot, prompt) if slot >= 0 else 0
