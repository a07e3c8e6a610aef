"""Sampling parameters and the host sampler (the oracle for the device sampler kernels).

Restates the reference's sampler contract (``oxidize-core/src/model/sampling.rs:268-463``):
validation errors first; greedy shortcut when ``temperature <= 0`` or ``top_k == 1`` with no
penalties; additive OpenAI-style frequency/presence penalties over ``recent_tokens``
(``:697-735``); softmax with temperature over the full vocabulary; sort descending; top-k;
top-p (keep through the first index whose cumulative mass reaches p); min-p
(``p >= min_p * p_max``); typical; tail-free; inverse-CDF draw with
``target = random * sum(kept)``; degenerate sums fall back to greedy.  Speculative
accept/reject is ``speculative_decode`` (``sampling.rs:492-623``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


class SamplingError(ValueError):
    pass


@dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    min_p: Optional[float] = None
    typical_p: Optional[float] = None
    tail_free_z: Optional[float] = None
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_window: int = 64
    seed: Optional[int] = None
    max_tokens: int = 128
    stop_token_ids: Tuple[int, ...] = ()
    stop_sequences: Tuple[Tuple[int, ...], ...] = ()
    ignore_eos: bool = False
    tie: str = "lowest"  # argmax tie rule: lowest (C port) | highest (Rust engine)
    mirostat_tau: Optional[float] = None  # Mirostat v2 target surprise (bits); None = off
    mirostat_eta: float = 0.1
    grammar: Optional[object] = None  # engine.constrained.TokenGrammar: only tokens it allows can be drawn

    def validate(self) -> None:
        if self.top_k is not None and self.top_k == 0:
            raise SamplingError("top_k must be >= 1")
        for name in ("top_p", "min_p", "typical_p", "tail_free_z"):
            v = getattr(self, name)
            if v is not None and not (0.0 < v <= 1.0):
                raise SamplingError(f"{name} must be in (0, 1]")
        if self.frequency_penalty < 0 or self.presence_penalty < 0:
            raise SamplingError("penalties must be non-negative")
        if self.max_tokens < 0:
            raise SamplingError("max_tokens must be >= 0")
        if self.mirostat_tau is not None and not (self.mirostat_tau > 0 and self.mirostat_eta > 0):
            raise SamplingError("mirostat_tau and mirostat_eta must be positive")

    @property
    def is_greedy(self) -> bool:
        return (self.temperature <= 0.0 or self.top_k == 1) and not self.has_penalties

    @property
    def has_penalties(self) -> bool:
        return self.frequency_penalty > 0 or self.presence_penalty > 0

    @property
    def needs_host_sampler(self) -> bool:
        """Knobs the device sampler kernel does not implement: those rows are drawn on the host from
        their logits (penalties, typical / tail-free filters, Mirostat, grammar constraint)."""
        return (self.has_penalties or self.typical_p is not None or self.tail_free_z is not None
                or self.mirostat_tau is not None or self.grammar is not None)

    @property
    def has_filters(self) -> bool:
        return any(v is not None for v in (self.top_k, self.top_p, self.min_p, self.typical_p, self.tail_free_z))


GREEDY = SamplingParams(temperature=0.0)


def argmax_np(logits: np.ndarray, tie: str = "lowest") -> int:
    if tie == "highest":
        return int(len(logits) - 1 - np.argmax(logits[::-1]))
    return int(np.argmax(logits))


def apply_penalties(logits: np.ndarray, recent: Sequence[int], freq_pen: float, pres_pen: float) -> np.ndarray:
    if not recent or (freq_pen <= 0 and pres_pen <= 0):
        return logits
    out = logits.copy()
    ids, counts = np.unique(np.asarray(recent, dtype=np.int64), return_counts=True)
    ok = (ids >= 0) & (ids < len(out))
    out[ids[ok]] -= freq_pen * counts[ok] + pres_pen
    return out


def mirostat_v2(logits: np.ndarray, p: SamplingParams, random: float, state: dict) -> int:
    """Mirostat v2 (sampling.rs Mirostat variant): drop tokens whose surprise exceeds ``mu``, draw from
    the rest, then move ``mu`` toward the target surprise ``tau`` by ``eta`` times the error."""
    mu = state.setdefault("mirostat_mu", 2.0 * p.mirostat_tau)
    t = p.temperature if p.temperature > 0 else 1.0
    z = (logits.astype(np.float64) - float(np.max(logits))) / t
    probs = np.exp(z)
    probs /= probs.sum()
    order = np.argsort(-probs, kind="stable")
    sp = probs[order]
    surprise = -np.log2(np.maximum(sp, 1e-300))
    keep = max(1, int(np.sum(surprise <= mu)))
    ps = sp[:keep] / sp[:keep].sum()
    j = min(int(np.searchsorted(np.cumsum(ps), random, side="right")), keep - 1)
    state["mirostat_mu"] = mu - p.mirostat_eta * (float(-np.log2(max(ps[j], 1e-300))) - p.mirostat_tau)
    return int(order[j])


def sample(logits: np.ndarray, p: SamplingParams, random: float, recent: Sequence[int] = (),
           suppressed: Sequence[int] = (), state: Optional[dict] = None) -> int:
    """Draw one token from float32 ``logits`` using the uniform ``random`` in [0, 1).  ``state`` is the
    request's mutable sampler state (Mirostat's running ``mu``, the grammar's parse stacks)."""
    if not (0.0 <= random < 1.0):
        raise SamplingError("random must be in [0, 1)")
    p.validate()
    logits = np.asarray(logits, dtype=np.float32)
    if len(suppressed):
        logits = logits.copy()
        logits[np.asarray(suppressed, dtype=np.int64)] = -np.inf
    if p.grammar is not None and state is not None:
        allowed = p.grammar.allowed_tokens(state)
        if allowed is not None:
            masked = np.full_like(logits, -np.inf)
            idx = np.asarray(sorted(t for t in allowed if 0 <= t < len(logits)), dtype=np.int64)
            masked[idx] = logits[idx]
            logits = masked
    if p.mirostat_tau is not None and state is not None and math.isfinite(float(np.max(logits))):
        if p.has_penalties:
            logits = apply_penalties(logits, list(recent)[-p.repetition_window:], p.frequency_penalty, p.presence_penalty)
        return mirostat_v2(logits, p, random, state)
    if p.is_greedy:
        return argmax_np(logits, p.tie)
    if p.has_penalties:
        logits = apply_penalties(logits, list(recent)[-p.repetition_window:], p.frequency_penalty, p.presence_penalty)
    if p.temperature <= 0.0 or p.top_k == 1:
        return argmax_np(logits, p.tie)
    m = float(np.max(logits))
    if not math.isfinite(m):
        return argmax_np(logits, p.tie)
    probs = np.exp((logits - m) / p.temperature, dtype=np.float64)
    total = probs.sum()
    if not (total > 0 and math.isfinite(total)):
        return argmax_np(logits, p.tie)
    if not p.has_filters:
        # single-pass inverse CDF in index order (sample_unfiltered, sampling.rs:465-490)
        cdf = np.cumsum(probs)
        idx = int(np.searchsorted(cdf, random * total, side="right"))
        return min(idx, len(probs) - 1)
    probs = probs / total
    order = np.argsort(-probs, kind="stable")
    sp = probs[order]
    keep = len(sp)
    if p.top_k is not None:
        keep = min(keep, p.top_k)
    if p.top_p is not None:
        c = np.cumsum(sp[:keep])
        keep = min(keep, int(np.searchsorted(c, p.top_p, side="left")) + 1)
    if p.min_p is not None:
        keep = min(keep, max(1, int(np.sum(sp[:keep] >= p.min_p * sp[0]))))
    idxs = order[:keep]
    ps = sp[:keep]
    if p.typical_p is not None and keep > 1:
        ent = -np.sum(ps * np.log(np.maximum(ps, 1e-300)))
        dev = np.abs(-np.log(np.maximum(ps, 1e-300)) - ent)
        o2 = np.argsort(dev, kind="stable")
        c = np.cumsum(ps[o2])
        k2 = int(np.searchsorted(c, p.typical_p * c[-1], side="left")) + 1
        sel = np.sort(o2[:k2])
        idxs, ps = idxs[sel], ps[sel]
    if p.tail_free_z is not None and len(ps) > 2:
        d2 = np.abs(np.diff(np.diff(ps)))
        s = d2.sum()
        if s > 0:
            c = np.cumsum(d2 / s)
            k2 = int(np.searchsorted(c, p.tail_free_z, side="left")) + 1
            k2 = max(1, min(len(ps), k2))
            idxs, ps = idxs[:k2], ps[:k2]
    ksum = ps.sum()
    if not (ksum > 0 and math.isfinite(ksum)):
        return argmax_np(logits, p.tie)
    c = np.cumsum(ps)
    j = int(np.searchsorted(c, random * ksum, side="right"))
    return int(idxs[min(j, len(idxs) - 1)])


def probs_from_logits(logits: np.ndarray, temperature: float) -> np.ndarray:
    l = np.asarray(logits, dtype=np.float64)
    if temperature <= 0:
        out = np.zeros_like(l)
        out[int(np.argmax(l))] = 1.0
        return out
    l = (l - l.max()) / temperature
    e = np.exp(l)
    return e / e.sum()


def speculative_accept(draft_tokens: Sequence[int], draft_probs: Optional[Sequence[np.ndarray]],
                       target_logits: np.ndarray, p: SamplingParams, randoms: Sequence[float]) -> Tuple[List[int], int]:
    """Verify K drafted tokens against K+1 rows of target logits.

    Greedy: accept while the target argmax equals the draft.  Otherwise accept token i with
    probability min(1, p_i/q_i); on the first rejection resample from normalise(max(p-q,0)).
    If all K are accepted a bonus token is drawn from target row K.  Returns
    (emitted tokens, number of drafts accepted)."""
    K = len(draft_tokens)
    out: List[int] = []
    greedy = p.is_greedy or draft_probs is None
    for i in range(K):
        if greedy:
            t = argmax_np(target_logits[i], p.tie)
            if t == draft_tokens[i]:
                out.append(t)
                continue
            out.append(t)
            return out, i
        pt = probs_from_logits(target_logits[i], p.temperature)
        q = np.asarray(draft_probs[i], dtype=np.float64)
        d = int(draft_tokens[i])
        ratio = pt[d] / q[d] if q[d] > 0 else 1.0
        if randoms[2 * i] < min(1.0, ratio):
            out.append(d)
            continue
        resid = np.maximum(pt - q, 0.0)
        s = resid.sum()
        if s <= 0:
            out.append(argmax_np(target_logits[i], p.tie))
        else:
            c = np.cumsum(resid)
            out.append(int(min(np.searchsorted(c, randoms[2 * i + 1] * s, side="right"), len(c) - 1)))
        return out, i
    if greedy:
        out.append(argmax_np(target_logits[K], p.tie))
    else:
        out.append(sample(target_logits[K], p, randoms[2 * K] if len(randoms) > 2 * K else 0.0))
    return out, K


class RequestRng:
    """One uniform f32 per token; seeded requests are reproducible (``seed`` → one stream)."""

    def __init__(self, seed: Optional[int]):
        self.rng = np.random.default_rng(seed)

    def next(self) -> float:
        v = float(np.float32(self.rng.random()))
        return min(v, 0.99999994)
