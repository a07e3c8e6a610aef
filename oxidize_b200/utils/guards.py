"""Canary bands around buffers that kernels write into.

A kernel that writes past the end (or before the start) of its output lands in the band instead of in
someone else's data; ``verify`` then names the buffer.  The bands are plain bytes of a fixed pattern next to
the payload inside ONE allocation, so the check works on any device and costs two small comparisons.

The reference runs its C port's tests under ASan / UBSan (``oxidize-c/Makefile:87-93``) and has no device-side
checker; this is the equivalent for device buffers, where a sanitizer is not available.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

GUARD_BYTES = 256
PATTERN = 0xA5


class MemoryGuardError(RuntimeError):
    pass


class GuardedAllocator:
    """Hands out tensors that sit between two canary bands and remembers them for ``verify``."""

    def __init__(self) -> None:
        self._live: List[Tuple[str, torch.Tensor, int]] = []  # (name, raw uint8 allocation, payload bytes)

    def empty(self, numel: int, dtype: torch.dtype, device, name: str = "buffer", zero: bool = False) -> torch.Tensor:
        item = torch.empty(0, dtype=dtype).element_size()
        nbytes = int(numel) * item
        pad = (-nbytes) % 16  # keep the trailing band 16-byte aligned, as the payload is
        raw = torch.empty(GUARD_BYTES + nbytes + pad + GUARD_BYTES, dtype=torch.uint8, device=device)
        raw[:GUARD_BYTES] = PATTERN
        raw[GUARD_BYTES + nbytes:] = PATTERN
        payload = raw[GUARD_BYTES:GUARD_BYTES + nbytes].view(dtype)
        if zero:
            payload.zero_()
        self._live.append((name, raw, nbytes))
        return payload

    def verify(self) -> None:
        """Raise MemoryGuardError naming every buffer whose bands no longer hold the pattern."""
        bad: Dict[str, str] = {}
        for name, raw, nbytes in self._live:
            head = raw[:GUARD_BYTES]
            tail = raw[GUARD_BYTES + nbytes:]
            if not bool((head == PATTERN).all()):
                bad[name] = "written before its start"
            elif not bool((tail == PATTERN).all()):
                first = int((tail != PATTERN).nonzero()[0])
                bad[name] = f"written {first} bytes past its end"
        if bad:
            raise MemoryGuardError("; ".join(f"{k}: {v}" for k, v in bad.items()))

    def forget(self, t: torch.Tensor) -> None:
        """Stop tracking the allocation that backs ``t`` (a buffer that is being replaced)."""
        p = t.data_ptr()
        self._live = [(n, r, b) for n, r, b in self._live if r.data_ptr() + GUARD_BYTES != p]

    def __len__(self) -> int:
        return len(self._live)
