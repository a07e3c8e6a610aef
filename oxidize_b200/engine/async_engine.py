"""Background engine thread for serving: one thread owns the ``LLM`` and all mutable serving
state; HTTP handlers talk to it through queues.

Role of the reference's ``BatchedEngineHandle`` / ``engine_loop``
(``oxidize-server/src/runtime/batched_engine.rs:45-284``): submit over a channel, one batched
forward per iteration over all active sequences, per-token routing to the caller, cancellation
when the caller's channel is closed (``:194-218``), and — after a failed forward — every
in-flight request is answered with an error and the engine keeps serving (``:266-284``).
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

from ..parallel.health import RunnerStatus, StepWatchdog
from .llm import LLM, RequestOutput
from .sampler import SamplingParams


@dataclass
class StreamEvent:
    request_id: str
    new_token_ids: List[int]
    text_delta: str
    finished: bool
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    prompt_tokens: int = 0
    completion_tokens: int = 0
    queue_wait_s: float = 0.0


@dataclass
class _Pending:
    request_id: str
    prompt: Any
    params: SamplingParams
    sink: Callable[[StreamEvent], None]
    submitted: float = field(default_factory=time.perf_counter)
    suppressed: Sequence[int] = ()


class AsyncEngine:
    def __init__(self, llm: LLM, step_deadline_s: float = 60.0, name: str = "oxidize-batch-engine", control=None):
        self.llm = llm
        self.control = control  # SpmdControl when follower ranks mirror this engine
        self._step_admits: List[Any] = []
        self._step_aborts: List[str] = []
        self._inbox: "queue.Queue[Any]" = queue.Queue()
        self._sinks: Dict[str, Callable[[StreamEvent], None]] = {}
        self._detok: Dict[str, Any] = {}
        self._sent: Dict[str, int] = {}
        self._meta: Dict[str, _Pending] = {}
        self._stop = threading.Event()
        self.watchdog = StepWatchdog(step_deadline_s)
        self.failures = 0
        self.tokens_generated = 0
        self.prompt_tokens = 0
        self._ids = 0
        self._lock = threading.Lock()
        self._thread = threading.Thread(target=self._loop, name=name, daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ caller side
    def next_id(self, prefix: str = "req") -> str:
        with self._lock:
            self._ids += 1
            return f"{prefix}-{self._ids}"

    def submit(self, prompt, params: SamplingParams, sink: Callable[[StreamEvent], None],
               request_id: Optional[str] = None) -> str:
        rid = request_id or self.next_id()
        self._inbox.put(_Pending(rid, prompt, params, sink))
        return rid

    def cancel(self, request_id: str) -> None:
        self._inbox.put(("cancel", request_id))

    def call(self, fn: Callable[[LLM], Any], timeout: Optional[float] = None) -> Any:
        """Run ``fn(llm)`` on the engine thread between two steps (the engine, its pools and its CUDA stream belong to
        that thread) and return its result; an exception raised by ``fn`` is raised here."""
        import concurrent.futures

        fut: "concurrent.futures.Future" = concurrent.futures.Future()
        self._inbox.put(("call", fn, fut))
        return fut.result(timeout)

    def embed(self, prompts, pooling: str = "mean"):
        if self.control is not None:
            raise NotImplementedError("embeddings are served by single-rank engines")
        return self.call(lambda llm: llm.embed(prompts, pooling))

    @property
    def healthy(self) -> bool:
        return self.watchdog.healthy and self._thread.is_alive()

    @property
    def queue_depth(self) -> int:
        return self._inbox.qsize() + len(self.llm.scheduler.waiting)

    def shutdown(self, timeout: float = 5.0) -> None:
        self._stop.set()
        self._inbox.put(("wake", None))
        self._thread.join(timeout)
        if self.control is not None:
            self.control.leader_sync([], [], stop=True)
        self.watchdog.close()

    async def stream(self, prompt, params: SamplingParams, request_id: Optional[str] = None):
        """Async generator of :class:`StreamEvent`; cancels the sequence if the consumer goes away."""
        loop = asyncio.get_running_loop()
        q: "asyncio.Queue[StreamEvent]" = asyncio.Queue()
        rid = self.submit(prompt, params, lambda ev: loop.call_soon_threadsafe(q.put_nowait, ev), request_id)
        try:
            while True:
                ev = await q.get()
                yield ev
                if ev.finished:
                    return
        finally:
            self.cancel(rid)

    def generate_blocking(self, prompt, params: SamplingParams, timeout: Optional[float] = None) -> List[StreamEvent]:
        done = threading.Event()
        evs: List[StreamEvent] = []

        def sink(ev: StreamEvent):
            evs.append(ev)
            if ev.finished:
                done.set()

        self.submit(prompt, params, sink)
        if not done.wait(timeout):
            raise TimeoutError("generation timed out")
        return evs

    # ------------------------------------------------------------------ engine thread
    def _admit(self, p: _Pending) -> None:
        try:
            self.llm.add_request(p.prompt, p.params, p.request_id)
        except Exception as e:  # noqa: BLE001 - reported to the caller
            p.sink(StreamEvent(p.request_id, [], "", True, "error", error=str(e)))
            return
        if self.control is not None:
            seq = self.llm._seqs[p.request_id]
            self._step_admits.append((p.request_id, list(seq.prompt), p.params))
        self._sinks[p.request_id] = p.sink
        self._sent[p.request_id] = 0
        self._meta[p.request_id] = p
        tok = self.llm.tokenizer
        self._detok[p.request_id] = tok.streaming_detokenizer() if tok is not None else None

    def _drain_inbox(self, block: bool) -> None:
        try:
            item = self._inbox.get(timeout=0.05) if block else self._inbox.get_nowait()
        except queue.Empty:
            return
        while True:
            if isinstance(item, _Pending):
                self._admit(item)
            elif isinstance(item, tuple) and item[0] == "cancel":
                rid = item[1]
                if rid in self._sinks:
                    self.llm.abort(rid)
                    self._forget(rid)
                    if self.control is not None:
                        self._step_aborts.append(rid)
            elif isinstance(item, tuple) and item[0] == "call":
                _, fn, fut = item
                if fut.set_running_or_notify_cancel():
                    try:
                        fut.set_result(fn(self.llm))
                    except BaseException as e:  # noqa: BLE001 - handed to the caller
                        fut.set_exception(e)
            try:
                item = self._inbox.get_nowait()
            except queue.Empty:
                return

    def _forget(self, rid: str) -> None:
        for d in (self._sinks, self._sent, self._detok, self._meta):
            d.pop(rid, None)

    def _route(self, ro: RequestOutput) -> None:
        sink = self._sinks.get(ro.request_id)
        if sink is None:
            return
        sent = self._sent[ro.request_id]
        new = ro.token_ids[sent:]
        self._sent[ro.request_id] = len(ro.token_ids)
        det = self._detok.get(ro.request_id)
        eos = self.llm.eos_token_id
        text = ""
        if det is not None:
            for t in new:
                if t == eos or self.llm.tokenizer.special_tokens.is_special(t):
                    continue
                text += det.push(t)
            if ro.finished:
                text += det.finish()
        meta = self._meta.get(ro.request_id)
        wait = 0.0 if ro.ttft is None or meta is None else max(0.0, ro.ttft)
        self.tokens_generated += len(new)
        ev = StreamEvent(ro.request_id, list(new), text, ro.finished, ro.finish_reason,
                         prompt_tokens=len(ro.prompt_token_ids), completion_tokens=len(ro.token_ids), queue_wait_s=wait)
        if ro.finished:
            self.prompt_tokens += len(ro.prompt_token_ids)
            self._forget(ro.request_id)
        sink(ev)

    def _fail_all(self, msg: str) -> None:
        self.failures += 1
        for rid, sink in list(self._sinks.items()):
            try:
                self.llm.abort(rid)
            except Exception:
                pass
            sink(StreamEvent(rid, [], "", True, "error", error=msg))
            self._forget(rid)

    def _loop(self) -> None:
        if self.llm.device.type == "cuda":
            import torch

            torch.cuda.set_device(self.llm.device)  # this thread launches on the replica's own GPU
        while not self._stop.is_set():
            self._drain_inbox(block=not self.llm.has_unfinished)
            if self.control is not None and (self._step_admits or self._step_aborts or self.llm.has_unfinished):
                self.control.leader_sync(self._step_admits, self._step_aborts)
                self._step_admits, self._step_aborts = [], []
            if not self.llm.has_unfinished:
                continue
            self.watchdog.begin_step()
            try:
                outs = self.llm.step()
            except Exception as e:  # noqa: BLE001 - engine survives a failed step
                self.watchdog.end_step()
                self._fail_all(f"engine step failed: {e}")
                continue
            self.watchdog.end_step()
            for ro in outs:
                self._route(ro)



class ReplicaRouter:
    """Data parallelism for serving: several complete engine replicas (each an :class:`AsyncEngine` with its own model
    copy, KV pool and GPU or tensor-parallel group) behind one front.  A request goes to the healthy replica with the
    fewest requests in flight (round robin among equals) and stays there; the router exposes the surface the HTTP layer
    uses of a single engine.  The reference scales out the same way, one engine per node behind its mesh front
    (``oxidize-core/src/mesh``); here the replicas share a process and a box."""

    def __init__(self, engines: List[AsyncEngine]):
        if not engines:
            raise ValueError("need at least one replica")
        self.engines = list(engines)
        self._owner: Dict[str, int] = {}
        self._inflight = [0] * len(self.engines)
        self._rr = 0
        self._lock = threading.Lock()
        self._ids = 0

    # the HTTP layer reads tokenizer, chat template and pool gauges from `.llm`
    @property
    def llm(self) -> LLM:
        return self.engines[0].llm

    def next_id(self, prefix: str = "req") -> str:
        with self._lock:
            self._ids += 1
            return f"{prefix}-{self._ids}"

    def _pick(self) -> int:
        with self._lock:
            n = len(self.engines)
            order = [(self._rr + i) % n for i in range(n)]
            live = [i for i in order if self.engines[i].healthy] or order
            best = min(live, key=lambda i: self._inflight[i])
            self._rr = (best + 1) % n
            self._inflight[best] += 1
            return best

    def submit(self, prompt, params: SamplingParams, sink: Callable[[StreamEvent], None],
               request_id: Optional[str] = None) -> str:
        rid = request_id or self.next_id()
        i = self._pick()
        with self._lock:
            self._owner[rid] = i

        def routed(ev: StreamEvent) -> None:
            if ev.finished:
                with self._lock:
                    if self._owner.pop(rid, None) is not None:
                        self._inflight[i] = max(0, self._inflight[i] - 1)
            sink(ev)

        return self.engines[i].submit(prompt, params, routed, rid)

    def embed(self, prompts, pooling: str = "mean"):
        with self._lock:
            live = [e for e in self.engines if e.healthy] or self.engines
            self._rr += 1
            eng = live[self._rr % len(live)]
        return eng.embed(prompts, pooling)

    def cancel(self, request_id: str) -> None:
        with self._lock:
            i = self._owner.pop(request_id, None)
            if i is not None:
                self._inflight[i] = max(0, self._inflight[i] - 1)
        if i is not None:
            self.engines[i].cancel(request_id)

    async def stream(self, prompt, params: SamplingParams, request_id: Optional[str] = None):
        loop = asyncio.get_running_loop()
        q: "asyncio.Queue[StreamEvent]" = asyncio.Queue()
        rid = self.submit(prompt, params, lambda ev: loop.call_soon_threadsafe(q.put_nowait, ev), request_id)
        try:
            while True:
                ev = await q.get()
                yield ev
                if ev.finished:
                    return
        finally:
            self.cancel(rid)

    def generate_blocking(self, prompt, params: SamplingParams, timeout: Optional[float] = None) -> List[StreamEvent]:
        done = threading.Event()
        evs: List[StreamEvent] = []

        def sink(ev: StreamEvent):
            evs.append(ev)
            if ev.finished:
                done.set()

        self.submit(prompt, params, sink)
        if not done.wait(timeout):
            raise TimeoutError("generation timed out")
        return evs

    @property
    def healthy(self) -> bool:
        return any(e.healthy for e in self.engines)

    @property
    def queue_depth(self) -> int:
        return sum(e.queue_depth for e in self.engines)

    @property
    def tokens_generated(self) -> int:
        return sum(e.tokens_generated for e in self.engines)

    @property
    def prompt_tokens(self) -> int:
        return sum(e.prompt_tokens for e in self.engines)

    @property
    def failures(self) -> int:
        return sum(e.failures for e in self.engines)

    @property
    def watchdog(self):
        return self.engines[0].watchdog

    def load(self) -> List[int]:
        """Requests in flight per replica."""
        with self._lock:
            return list(self._inflight)

    def shutdown(self, timeout: float = 5.0) -> None:
        for e in self.engines:
            e.shutdown(timeout)
