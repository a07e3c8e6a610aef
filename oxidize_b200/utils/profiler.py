"""In-process decode profiler, NVTX ranges and value tracing.

* ``OXIDIZE_DECODE_PROFILE=1`` — every operator call through :mod:`oxidize_b200.ops` is timed
  (CUDA events on the launching stream for device tensors, ``perf_counter`` on the CPU path) and
  accumulated per (operator, shape); ``report()`` prints calls, total and mean time, like the
  reference's per-shape GEMV profile (``compute/tensor/kernels/gemv.rs:380-452``).  Event timing
  needs eager launches, so the engine does not capture CUDA graphs while the profiler is on.
* ``OXIDIZE_NVTX=1`` — the same call sites open NVTX ranges (visible in Nsight Systems / Compute).
* ``OXIDIZE_TRACE_FWD=1`` — per-layer checksums of the hidden state (sum, mean |x|, max |x|) are
  printed from the layer loop, the equivalent of ``OXIDIZE_TRACE_FWD`` / ``OXIDIZE_TRACE_VALS``
  (``model/inference.rs:22-31``); use it to find the first layer where two builds diverge.
"""
from __future__ import annotations

import atexit
import functools
import os
import sys
import time
from collections import defaultdict
from typing import Callable, Dict, List, Tuple

import torch

PROFILE = os.environ.get("OXIDIZE_DECODE_PROFILE", "0") == "1"
NVTX = os.environ.get("OXIDIZE_NVTX", "0") == "1"
TRACE_FWD = os.environ.get("OXIDIZE_TRACE_FWD", "0") == "1"

_acc: Dict[Tuple[str, str], List[float]] = defaultdict(lambda: [0, 0.0])  # (op, shape) -> [calls, ms]
_pending: List[Tuple[Tuple[str, str], "torch.cuda.Event", "torch.cuda.Event"]] = []


def enabled() -> bool:
    return PROFILE


def _shape_key(args) -> str:
    parts = []
    for a in args[:2]:
        if isinstance(a, torch.Tensor):
            parts.append("x".join(str(d) for d in a.shape))
        elif hasattr(a, "out_features"):
            parts.append(f"W{a.out_features}x{a.in_features}")
    return " ".join(parts)


def _drain() -> None:
    if not _pending:
        return
    torch.cuda.synchronize()
    for key, e0, e1 in _pending:
        a = _acc[key]
        a[0] += 1
        a[1] += e0.elapsed_time(e1)
    _pending.clear()


def instrument(name: str) -> Callable:
    """Decorator for the operator front door; a no-op unless profiling or NVTX is switched on."""

    def deco(fn):
        if not (PROFILE or NVTX):
            return fn

        @functools.wraps(fn)
        def wrapped(*args, **kw):
            on_gpu = any(isinstance(a, torch.Tensor) and a.is_cuda for a in args)
            if NVTX and on_gpu:
                torch.cuda.nvtx.range_push(name)
            try:
                if not PROFILE:
                    return fn(*args, **kw)
                key = (name, _shape_key(args))
                if on_gpu:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    out = fn(*args, **kw)
                    e1.record()
                    _pending.append((key, e0, e1))
                    if len(_pending) >= 4096:
                        _drain()
                    return out
                t0 = time.perf_counter()
                out = fn(*args, **kw)
                a = _acc[key]
                a[0] += 1
                a[1] += (time.perf_counter() - t0) * 1e3
                return out
            finally:
                if NVTX and on_gpu:
                    torch.cuda.nvtx.range_pop()

        return wrapped

    return deco


def report(file=None) -> str:
    """Accumulated per-(operator, shape) times, largest first."""
    if torch.cuda.is_available():
        _drain()
    rows = sorted(_acc.items(), key=lambda kv: -kv[1][1])
    total = sum(v[1] for _, v in rows) or 1.0
    lines = [f"{'operator':<18}{'shape':<34}{'calls':>8}{'total ms':>12}{'mean us':>10}{'share':>8}"]
    for (op, shape), (calls, ms) in rows:
        lines.append(f"{op:<18}{shape:<34}{calls:>8}{ms:>12.3f}{ms / max(calls, 1) * 1e3:>10.1f}{ms / total * 100:>7.1f}%")
    text = "\n".join(lines)
    if file is not None:
        print(text, file=file)
    return text


def reset() -> None:
    _acc.clear()
    _pending.clear()


def trace_hidden(layer: int, h: torch.Tensor, residual) -> None:
    """One line per layer: checksums of the hidden state (h + residual)."""
    x = h.float() if residual is None else h.float() + residual.float()
    print(f"[trace] layer {layer:3d} sum={x.sum().item():+.6e} mean_abs={x.abs().mean().item():.6e} "
          f"max_abs={x.abs().max().item():.6e}", file=sys.stderr)


if PROFILE:
    atexit.register(lambda: report(sys.stderr))
