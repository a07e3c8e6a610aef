"""ctypes bindings to ``liboxbrt.so``, the C++ host runtime (``csrc/runtime.cpp``).

``NativeBlockPool`` has the interface and the exact block-id order of ``kv_pool.BlockPool`` (which
remains the executable specification and the fallback when the library cannot be built).
``OXB_NATIVE_RUNTIME=0`` switches it off.  (A C++ builder for the decode step's staging arrays was
measured too: collecting the per-sequence state from Python costs as much as filling the arrays, so
the batch builder stays in ``runner.py``.)
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence, Tuple

import numpy as np

_lib = None
_tried = False


def lib():
    """The loaded library, or None when disabled or unavailable."""
    global _lib, _tried
    if _tried:
        return _lib
    _tried = True
    if os.environ.get("OXB_NATIVE_RUNTIME", "1") == "0":
        return None
    try:
        from ..build import CSRC, build_runtime

        # Load what is there; build only when nothing is (several ranks start at once, and a rebuild
        # triggered by file times after a copy would have them all write the same file).
        path = os.path.join(CSRC, "liboxbrt.so")
        if not os.path.exists(path):
            path = build_runtime()
        if not path:
            return None
        L = ctypes.CDLL(path)
    except Exception:
        return None
    vp, i32, i64, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64
    L.oxbrt_block_hash.argtypes, L.oxbrt_block_hash.restype = [vp, i64, u64], u64
    L.oxbrt_pool_create.argtypes, L.oxbrt_pool_create.restype = [i32, i32, i32], vp
    L.oxbrt_pool_destroy.argtypes = [vp]
    L.oxbrt_pool_allocate.argtypes = [vp]
    L.oxbrt_pool_incref.argtypes = [vp, i32]
    L.oxbrt_pool_release.argtypes = [vp, i32]
    L.oxbrt_pool_lookup.argtypes = [vp, u64]
    L.oxbrt_pool_publish.argtypes = [vp, i32, u64]
    L.oxbrt_pool_ref.argtypes = [vp, i32]
    L.oxbrt_pool_num_free.argtypes = [vp]
    L.oxbrt_pool_stats.argtypes = [vp, vp]
    L.oxbrt_pool_hash_of.argtypes, L.oxbrt_pool_hash_of.restype = [vp, i32, ctypes.POINTER(i32)], u64
    L.oxbrt_pool_match_prefix.argtypes = [vp, vp, i64, vp, i32]
    _lib = L
    return _lib


class _RefView:
    """``pool.ref[b]`` on the native pool."""

    def __init__(self, pool):
        self._p = pool

    def __getitem__(self, b: int) -> int:
        return self._p._L.oxbrt_pool_ref(self._p._h, int(b))

    def __len__(self) -> int:
        return self._p.num_blocks


class NativeBlockPool:
    def __init__(self, num_blocks: int, page_size: int = 16, enable_prefix_cache: bool = True):
        L = lib()
        if L is None:
            raise RuntimeError("liboxbrt is not available")
        self._L = L
        self.num_blocks, self.page_size, self.enable_prefix_cache = num_blocks, page_size, enable_prefix_cache
        self._h = L.oxbrt_pool_create(num_blocks, page_size, 1 if enable_prefix_cache else 0)
        if not self._h:
            raise ValueError("invalid block pool geometry")
        self.ref = _RefView(self)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._L.oxbrt_pool_destroy(h)

    def _stats(self):
        out = (ctypes.c_int64 * 5)()
        self._L.oxbrt_pool_stats(self._h, out)
        return list(out)

    @property
    def num_free(self) -> int:
        return self._L.oxbrt_pool_num_free(self._h)

    @property
    def num_used(self) -> int:
        return self.num_blocks - self.num_free

    @property
    def hits(self) -> int:
        return self._stats()[3]

    @property
    def misses(self) -> int:
        return self._stats()[4]

    def allocate(self) -> int:
        b = self._L.oxbrt_pool_allocate(self._h)
        if b < 0:
            from .kv_pool import OutOfBlocks

            raise OutOfBlocks("KV block pool exhausted")
        return b

    def can_allocate(self, n: int) -> bool:
        return self.num_free >= n

    def incref(self, b: int) -> None:
        self._L.oxbrt_pool_incref(self._h, int(b))

    def release(self, b: int) -> None:
        if self._L.oxbrt_pool_release(self._h, int(b)) != 0:
            raise RuntimeError(f"double free of KV block {b}")

    def release_all(self, blocks: Sequence[int]) -> None:
        for b in reversed(list(blocks)):
            self.release(b)

    def lookup(self, h: int) -> Optional[int]:
        b = self._L.oxbrt_pool_lookup(self._h, ctypes.c_uint64(h))
        return None if b < 0 else b

    def publish(self, b: int, h: int) -> None:
        self._L.oxbrt_pool_publish(self._h, int(b), ctypes.c_uint64(h))

    def is_shared(self, b: int) -> bool:
        return self.ref[b] > 1

    def hash_of_block(self, b: int) -> Optional[int]:
        has = ctypes.c_int(0)
        h = self._L.oxbrt_pool_hash_of(self._h, int(b), ctypes.byref(has))
        return h if has.value else None

    def match_prefix(self, tokens: Sequence[int]) -> Tuple[List[int], int]:
        if not self.enable_prefix_cache or len(tokens) == 0:
            return [], 0
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty(max(1, (len(t) - 1) // self.page_size), dtype=np.int32)
        n = self._L.oxbrt_pool_match_prefix(self._h, t.ctypes.data, len(t), out.ctypes.data, len(out))
        return out[:n].tolist(), n * self.page_size


def block_hash(tokens: Sequence[int], h: int) -> int:
    L = lib()
    t = np.ascontiguousarray(tokens, dtype=np.int32)
    return int(L.oxbrt_block_hash(t.ctypes.data, len(t), ctypes.c_uint64(h)))
