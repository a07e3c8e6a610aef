"""Failure detection on the host: heartbeats between rank processes, staleness eviction, a
step watchdog, and a timeout wrapper for collectives.

Mirrors the reference's mechanisms — heartbeat staleness eviction (``mesh/topology.rs:126``,
15 s in ``mesh/discovery.rs:297``), the 60 s collective timeout returning
``TimedResult::{Ok, TimedOut, Err}`` (``mesh/fault_tolerance.rs:13-27,80-114``) and the runner
status update it emits — for a single-box job whose ranks share a ``TCPStore``.  Nothing here
touches a GPU: device-side waits are bounded inside the kernels and report through the device
status word, which :func:`check_device_status` turns into an exception between steps.
"""
from __future__ import annotations

import enum
import os
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

DEFAULT_COLLECTIVE_TIMEOUT_S = 60.0
DEFAULT_STALE_AFTER_S = 15.0


class RunnerStatus(enum.Enum):
    RUNNING = "running"
    FAILED = "failed"
    SHUTDOWN = "shutdown"


@dataclass
class TimedResult:
    status: str  # ok | timed_out | error
    value: object = None
    error: Optional[BaseException] = None
    elapsed_s: float = 0.0

    @property
    def ok(self) -> bool:
        return self.status == "ok"


def eval_with_timeout(fn: Callable[[], object], timeout_s: float = DEFAULT_COLLECTIVE_TIMEOUT_S,
                      on_failure: Optional[Callable[[str], None]] = None) -> TimedResult:
    """Run ``fn`` on a worker thread; give up after ``timeout_s`` (the thread is left to finish
    or die with the process, as with the reference's abandoned future)."""
    box: Dict[str, object] = {}

    def run():
        try:
            box["v"] = fn()
        except BaseException as e:  # noqa: BLE001
            box["e"] = e

    t0 = time.monotonic()
    th = threading.Thread(target=run, daemon=True)
    th.start()
    th.join(timeout_s)
    dt = time.monotonic() - t0
    if th.is_alive():
        if on_failure:
            on_failure("timed_out")
        return TimedResult("timed_out", elapsed_s=dt)
    if "e" in box:
        if on_failure:
            on_failure("error")
        return TimedResult("error", error=box["e"], elapsed_s=dt)  # type: ignore[arg-type]
    return TimedResult("ok", box.get("v"), elapsed_s=dt)


class MemoryStore:
    """In-process stand-in for TCPStore (tests, single-process runs)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k: str, v) -> None:
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        with self._lock:
            return self._d[k]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


class Heartbeat:
    """Each rank writes ``hb/<rank> = <monotonic stamp>`` every ``interval_s``; a rank whose
    stamp is older than ``stale_after_s`` — or that announced its exit — is reported dead."""

    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0,
                 stale_after_s: float = DEFAULT_STALE_AFTER_S, clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.stale_after_s, self.clock = interval_s, stale_after_s, clock
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.started_at = clock()

    @classmethod
    def from_env(cls, rank: int, world: int, port_offset: int = 17, **kw) -> "Heartbeat":
        from datetime import timedelta

        import torch.distributed as dist

        host = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = int(os.environ.get("MASTER_PORT", "29511")) + port_offset
        store = dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=timedelta(seconds=60),
                              wait_for_workers=False)
        return cls(store, rank, world, **kw)

    def beat(self) -> None:
        self.store.set(f"hb/{self.rank}", repr(self.clock()))

    def start(self) -> None:
        self.beat()

        def loop():
            while not self._stop.wait(self.interval_s):
                try:
                    self.beat()
                except Exception:
                    return

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self, announce_exit: bool = False) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if announce_exit:
            try:
                self.store.set(f"exit/{self.rank}", "1")
            except Exception:
                pass

    def dead_ranks(self) -> List[int]:
        now = self.clock()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if self.store.check([f"exit/{r}"]):
                    dead.append(r)
                    continue
                if not self.store.check([f"hb/{r}"]):
                    if now - self.started_at > self.stale_after_s:
                        dead.append(r)
                    continue
                stamp = float(self.store.get(f"hb/{r}").decode())
                if now - stamp > self.stale_after_s:
                    dead.append(r)
            except Exception:
                dead.append(r)
        return dead


class StepWatchdog:
    """Marks the engine unhealthy when a step overruns its deadline (``/readyz`` then answers 503
    and in-flight requests are drained with an error)."""

    def __init__(self, deadline_s: float = 30.0, on_trip: Optional[Callable[[float], None]] = None):
        self.deadline_s = deadline_s
        self.on_trip = on_trip
        self.status = RunnerStatus.RUNNING
        self._t0: Optional[float] = None
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def begin_step(self) -> None:
        with self._lock:
            self._t0 = time.monotonic()

    def end_step(self) -> None:
        with self._lock:
            self._t0 = None

    def _loop(self) -> None:
        while not self._stop.wait(min(0.05, self.deadline_s / 4)):
            with self._lock:
                t0 = self._t0
            if t0 is not None and time.monotonic() - t0 > self.deadline_s and self.status is RunnerStatus.RUNNING:
                self.status = RunnerStatus.FAILED
                if self.on_trip:
                    self.on_trip(time.monotonic() - t0)

    @property
    def healthy(self) -> bool:
        return self.status is RunnerStatus.RUNNING

    def close(self) -> None:
        self._stop.set()
        self.status = RunnerStatus.SHUTDOWN if self.status is RunnerStatus.RUNNING else self.status


class DeviceFault(RuntimeError):
    pass


STATUS_NAMES = {1: "TMA full-barrier wait timed out", 2: "TMA empty-barrier wait timed out",
                3: "accumulator wait timed out", 4: "peer flag wait timed out (a rank is missing or late)",
                5: "split-K rendezvous timed out", 6: "bad argument"}


def check_device_status() -> None:
    """Raise if any bounded device-side wait gave up since the last check."""
    from ..ops import cuda as C

    code, detail, count = C.status(reset=True)
    if code != 0:
        raise DeviceFault(f"device status {code} ({STATUS_NAMES.get(code, 'unknown')}), detail={detail}, events={count}")
