"""Request middleware pieces: API-key auth, rate / concurrency limits, Prometheus metrics and
the structured audit log.

Behaviour follows the reference server: keys from ``OXIDIZE_API_KEY`` / ``OXIDIZE_API_KEYS``
accepted as ``x-api-key`` or ``Authorization: Bearer`` and compared in constant time
(``oxidize-server/src/auth.rs:44,84,122``); 64 requests/s, 8 in flight, 128 queued by default
(``limits.rs:21-35``); metric names as in ``metrics.rs:48-100``; JSON audit records with request
id, key hash, model, token counts, duration and stop reason (``audit.rs:37-170``).
"""
from __future__ import annotations

import hashlib
import hmac
import json
import os
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

OPEN_PATHS = ("/healthz", "/livez", "/readyz", "/metrics", "/openapi.json")


# --------------------------------------------------------------------------- auth
def load_api_keys(env=os.environ) -> List[str]:
    keys: List[str] = []
    one = env.get("OXIDIZE_API_KEY", "").strip()
    if one:
        keys.append(one)
    for k in env.get("OXIDIZE_API_KEYS", "").split(","):
        k = k.strip()
        if k:
            keys.append(k)
    return keys


def extract_key(headers) -> Optional[str]:
    k = headers.get("x-api-key")
    if k:
        return k.strip()
    auth = headers.get("authorization", "")
    if auth.lower().startswith("bearer "):
        return auth[7:].strip()
    return None


def key_is_valid(presented: Optional[str], keys: Iterable[str]) -> bool:
    if presented is None:
        return False
    ok = False
    for k in keys:  # no early exit: constant time over the key list
        ok |= hmac.compare_digest(presented.encode(), k.encode())
    return ok


def key_hash(presented: Optional[str]) -> Optional[str]:
    return None if not presented else hashlib.sha256(presented.encode()).hexdigest()[:16]


# --------------------------------------------------------------------------- limits
@dataclass
class LimitConfig:
    max_requests_per_second: float = 64.0
    max_in_flight: int = 8
    max_queued: int = 128
    max_body_bytes: int = 10 * 1024 * 1024


class RequestLimiter:
    """Token bucket for the request rate plus in-flight / queued admission counters."""

    def __init__(self, cfg: Optional[LimitConfig] = None, clock=time.monotonic):
        self.cfg = cfg or LimitConfig()
        self.clock = clock
        self._tokens = self.cfg.max_requests_per_second
        self._last = clock()
        self.in_flight = 0
        self.queued = 0
        self._lock = threading.Lock()

    def try_acquire(self) -> Optional[str]:
        """None when admitted, else the reason for a 429."""
        with self._lock:
            now = self.clock()
            rate = self.cfg.max_requests_per_second
            self._tokens = min(rate, self._tokens + (now - self._last) * rate)
            self._last = now
            if self._tokens < 1.0:
                return "rate_limited"
            if self.in_flight >= self.cfg.max_in_flight + self.cfg.max_queued:
                return "queue_full"
            self._tokens -= 1.0
            self.in_flight += 1
            self.queued = max(0, self.in_flight - self.cfg.max_in_flight)
            return None

    def release(self) -> None:
        with self._lock:
            self.in_flight = max(0, self.in_flight - 1)
            self.queued = max(0, self.in_flight - self.cfg.max_in_flight)


# --------------------------------------------------------------------------- metrics
class Metrics:
    def __init__(self):
        from prometheus_client import CollectorRegistry, Counter, Gauge, Histogram

        self.registry = CollectorRegistry()
        r = self.registry
        self.requests_total = Counter("oxidize_requests_total", "HTTP requests", ["method", "path", "status"], registry=r)
        self.request_duration = Histogram("oxidize_request_duration_seconds", "Request latency", ["method", "path"],
                                          registry=r)
        self.in_flight = Gauge("oxidize_requests_in_flight", "Requests in flight", registry=r)
        self.tokens_generated = Counter("oxidize_tokens_generated_total", "Completion tokens", registry=r)
        self.tokens_prompt = Counter("oxidize_tokens_prompt_total", "Prompt tokens", registry=r)
        self.tokens_per_second = Gauge("oxidize_tokens_per_second", "Decode speed of the last request", registry=r)
        self.queue_depth = Gauge("oxidize_queue_depth", "Requests waiting for the engine", registry=r)
        self.queue_wait = Histogram("oxidize_queue_wait_duration_seconds", "Time to first token", registry=r)
        self.cache_hits = Counter("oxidize_cache_hits_total", "Prefix cache hits (blocks)", registry=r)
        self.cache_misses = Counter("oxidize_cache_misses_total", "Prefix cache misses (blocks)", registry=r)
        self.errors = Counter("oxidize_errors_total", "Errors", ["kind"], registry=r)
        self.rate_limited = Counter("oxidize_rate_limited_total", "Requests rejected by limits", ["reason"], registry=r)
        self.spec_acceptance = Gauge("oxidize_speculative_acceptance_rate", "Draft tokens accepted / proposed", registry=r)

    def render(self) -> bytes:
        from prometheus_client import generate_latest

        return generate_latest(self.registry)


# --------------------------------------------------------------------------- audit
class AuditLogger:
    """One JSON object per line; never raises into the request path."""

    def __init__(self, path: Optional[str] = None, stream=None, enabled: bool = True):
        self.enabled = enabled
        self._lock = threading.Lock()
        self._fh = open(path, "a", buffering=1) if path else (stream if stream is not None else sys.stderr)
        self.records = 0

    def log(self, event: str, **fields) -> None:
        if not self.enabled:
            return
        rec = {"ts": round(time.time(), 3), "event": event}
        rec.update({k: v for k, v in fields.items() if v is not None})
        try:
            with self._lock:
                self._fh.write(json.dumps(rec, separators=(",", ":")) + "\n")
                self.records += 1
        except Exception:
            pass

    def request(self, request_id: str, key: Optional[str], model: str, prompt_tokens: int, completion_tokens: int,
                duration_s: float, stop_reason: Optional[str], path: str, status: int = 200) -> None:
        self.log("request", request_id=request_id, key_hash=key_hash(key), model=model, prompt_tokens=prompt_tokens,
                 completion_tokens=completion_tokens, duration_ms=round(duration_s * 1e3, 2), stop_reason=stop_reason,
                 path=path, status=status)

    def security(self, kind: str, path: str, remote: Optional[str] = None) -> None:
        self.log("security", kind=kind, path=path, remote=remote)
