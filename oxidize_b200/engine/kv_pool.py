"""Paged KV cache: real storage behind block ids, plus the block allocator.

Allocator semantics follow the reference's ``BlockPool`` (``paged_attention/block_pool.rs``):
free list, per-block reference counts, a global prefix cache keyed by an FNV-1a hash over the
*whole prefix up to the block end* (``block_pool.rs:11-18``, ``scheduler/prefix_cache.rs:26-31``)
with LRU eviction of unreferenced cached blocks, and copy-on-write when a shared block is
written.  Unlike the reference, whose pool "owns no KV bytes" (``block_pool.rs:28-37``), every
block id here addresses device memory:

    data[layer]   : [num_blocks, n_kv_heads, 2 (K,V), page, head_dim]   f16/bf16/f32, or
                    uint8 codes (q8: head_dim bytes, q4: head_dim/2 bytes)
    scales[layer] : [num_blocks, n_kv_heads, 2, page, head_dim/32] f32   (q8/q4 only)

so one (block, head, K) tile of a 16-token page with head_dim 128 is 4 KB contiguous — one
TMA box / one fully coalesced burst in the attention kernels.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

FNV_OFFSET = 0xCBF29CE484222325
FNV_PRIME = 0x100000001B3
_MASK64 = (1 << 64) - 1


def block_hash(tokens: Sequence[int], h: int = FNV_OFFSET) -> int:
    """FNV-1a-style 64-bit hash (multiply, then xor the token), continuing from ``h``."""
    for t in tokens:
        h = (h * FNV_PRIME) & _MASK64
        h ^= int(t) & _MASK64
    return h


class OutOfBlocks(RuntimeError):
    """No free block and nothing evictable (``SchedulerError::OutOfMemory``)."""


class BlockPool:
    """Host-side allocator over ``num_blocks`` physical pages."""

    def __init__(self, num_blocks: int, page_size: int = 16, enable_prefix_cache: bool = True):
        self.num_blocks = num_blocks
        self.page_size = page_size
        self.enable_prefix_cache = enable_prefix_cache
        self.ref = [0] * num_blocks
        self.hash_of: List[Optional[int]] = [None] * num_blocks
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))  # pop() yields 0,1,2,...
        self.cache: Dict[int, int] = {}
        # cached blocks with ref == 0, oldest first (evictable)
        self.lru: "OrderedDict[int, None]" = OrderedDict()
        self.hits = 0
        self.misses = 0

    # ---- counts
    @property
    def num_free(self) -> int:
        return len(self.free) + len(self.lru)

    @property
    def num_used(self) -> int:
        return self.num_blocks - self.num_free

    # ---- allocate / free
    def allocate(self) -> int:
        if self.free:
            b = self.free.pop()
        elif self.lru:
            b, _ = self.lru.popitem(last=False)
            h = self.hash_of[b]
            if h is not None and self.cache.get(h) == b:
                del self.cache[h]
            self.hash_of[b] = None
        else:
            raise OutOfBlocks("KV block pool exhausted")
        self.ref[b] = 1
        return b

    def can_allocate(self, n: int) -> bool:
        return self.num_free >= n

    def incref(self, b: int) -> None:
        if self.ref[b] == 0:
            self.lru.pop(b, None)
        self.ref[b] += 1

    def release(self, b: int) -> None:
        if self.ref[b] <= 0:
            raise RuntimeError(f"double free of KV block {b}")
        self.ref[b] -= 1
        if self.ref[b] == 0:
            if self.hash_of[b] is not None and self.cache.get(self.hash_of[b]) == b:
                self.lru[b] = None  # stays cached until evicted
            else:
                self.hash_of[b] = None
                self.free.append(b)

    def release_all(self, blocks: Sequence[int]) -> None:
        for b in reversed(list(blocks)):
            self.release(b)

    # ---- prefix cache
    def lookup(self, h: int) -> Optional[int]:
        if not self.enable_prefix_cache:
            return None
        b = self.cache.get(h)
        if b is None:
            self.misses += 1
            return None
        self.hits += 1
        self.incref(b)
        return b

    def publish(self, b: int, h: int) -> None:
        """Register a *full* block under its prefix hash (first writer wins)."""
        if not self.enable_prefix_cache or h in self.cache:
            return
        self.cache[h] = b
        self.hash_of[b] = h

    def is_shared(self, b: int) -> bool:
        return self.ref[b] > 1

    def match_prefix(self, tokens: Sequence[int]) -> Tuple[List[int], int]:
        """Longest run of cached full blocks covering a prefix of ``tokens``.

        Returns (blocks with their refs taken, number of tokens covered).  The last prompt
        token is never served from cache so that prefill still produces logits."""
        if not self.enable_prefix_cache:
            return [], 0
        out: List[int] = []
        h = FNV_OFFSET
        ps = self.page_size
        n_full = (len(tokens) - 1) // ps
        for i in range(n_full):
            h = block_hash(tokens[i * ps : (i + 1) * ps], h)
            b = self.lookup(h)
            if b is None:
                break
            out.append(b)
        return out, len(out) * ps


def make_block_pool(num_blocks: int, page_size: int = 16, enable_prefix_cache: bool = True):
    """The C++ pool (``csrc/runtime.cpp``) when the host runtime library is available, else the
    Python one; both hand out the same block ids for the same sequence of calls."""
    from . import native

    if native.lib() is not None:
        return native.NativeBlockPool(num_blocks, page_size, enable_prefix_cache)
    return BlockPool(num_blocks, page_size, enable_prefix_cache)


KV_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "q8": torch.uint8, "q4": torch.uint8}


@dataclass
class KVCacheSpec:
    n_layers: int
    n_kv_heads: int
    head_dim: int
    page_size: int = 16
    dtype_name: str = "bf16"

    def bytes_per_block(self) -> int:
        e = self.n_kv_heads * 2 * self.page_size
        if self.dtype_name == "q8":
            per = e * (self.head_dim + self.head_dim // 32 * 4)
        elif self.dtype_name == "q4":
            per = e * (self.head_dim // 2 + self.head_dim // 32 * 4)
        else:
            per = e * self.head_dim * torch.empty(0, dtype=KV_DTYPES[self.dtype_name]).element_size()
        return per * self.n_layers


class KVCache:
    """Device storage for all layers' pages (this rank's KV heads only)."""

    def __init__(self, spec: KVCacheSpec, num_blocks: int, device="cpu"):
        if spec.dtype_name not in KV_DTYPES:
            raise ValueError(f"kv dtype must be one of {sorted(KV_DTYPES)}")
        if spec.dtype_name in ("q8", "q4") and spec.head_dim % 32:
            raise ValueError("quantized KV needs head_dim % 32 == 0")
        self.spec = spec
        self.num_blocks = num_blocks
        self.page_size = spec.page_size
        self.dtype_name = spec.dtype_name
        self.device = torch.device(device)
        hd = spec.head_dim
        inner = hd if spec.dtype_name != "q4" else hd // 2
        shape = (num_blocks, spec.n_kv_heads, 2, spec.page_size, inner)
        self.data = [torch.zeros(shape, dtype=KV_DTYPES[spec.dtype_name], device=self.device) for _ in range(spec.n_layers)]
        self.scales: List[Optional[torch.Tensor]] = [None] * spec.n_layers
        if spec.dtype_name in ("q8", "q4"):
            sshape = (num_blocks, spec.n_kv_heads, 2, spec.page_size, hd // 32)
            self.scales = [torch.zeros(sshape, dtype=torch.float32, device=self.device) for _ in range(spec.n_layers)]

    def copy_block(self, src: int, dst: int) -> None:
        """Copy-on-write support: duplicate one page in every layer."""
        aux = getattr(self, "conv", None)  # the convolution layers' rows of a hybrid model live in a second cache
        if aux is not None:
            aux.copy_block(src, dst)
        for l in range(self.spec.n_layers):
            self.data[l][dst].copy_(self.data[l][src])
            if self.scales[l] is not None:
                self.scales[l][dst].copy_(self.scales[l][src])

    def nbytes(self) -> int:
        n = sum(d.numel() * d.element_size() for d in self.data)
        n += sum(s.numel() * 4 for s in self.scales if s is not None)
        return n

    # ---- runtime state save/load (KvCache::save_to_file / load_from_file, kv_cache/cache.rs:423-445)
    def state_dict(self, blocks: Sequence[int]) -> dict:
        idx = torch.tensor(list(blocks), dtype=torch.long, device=self.device)
        out = {"version": 1, "spec": self.spec.__dict__.copy(), "data": [d[idx].cpu() for d in self.data]}
        if self.scales[0] is not None:
            out["scales"] = [s[idx].cpu() for s in self.scales]
        return out

    def load_state_dict(self, state: dict, blocks: Sequence[int]) -> None:
        if state.get("version") != 1:
            raise ValueError("unsupported KV snapshot version")
        idx = torch.tensor(list(blocks), dtype=torch.long, device=self.device)
        for l, d in enumerate(state["data"]):
            self.data[l][idx] = d.to(self.device)
        if "scales" in state:
            for l, s in enumerate(state["scales"]):
                self.scales[l][idx] = s.to(self.device)
