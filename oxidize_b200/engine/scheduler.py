"""Continuous-batching scheduler over the paged KV pool.

Policy is the reference's (``paged_attention/scheduler/core.rs:114-243``): each step first
gives every fully-prefilled running sequence its one decode token, then continues partial
prefills in chunks, then admits waiting sequences FCFS — all under one token budget and a
cap on running sequences.  Full prompt blocks are published to / served from the prefix cache
(``scheduler/prefix_cache.rs``), a shared last block is copied before a decode writes into it
(``:200-216``), and when the pool runs dry the youngest running sequence is preempted: its
blocks are released, cache entries kept, and it re-queues at the *front*
(``:169-196``).  Defaults mirror ``scheduler/config.rs:17-25`` (512 batched tokens, chunk 16,
8 running); serving configs raise them.

What the reference lacks and this adds: block ids address real KV bytes, many sequences run
per step, several rows per sequence per step (speculative verify), and a shortest-job-first
admission option (the C port's policy knob, ``oxidize-c/include/oxidize/continuous_batching.h:30-50``).
"""
from __future__ import annotations

import enum
import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from .kv_pool import FNV_OFFSET, BlockPool, OutOfBlocks, block_hash
from .sampler import RequestRng, SamplingParams


class SeqStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 512
    prefill_chunk_size: int = 16
    max_num_running_seqs: int = 8
    policy: str = "fcfs"  # fcfs | sjf
    enable_prefix_cache: bool = True
    max_model_len: int = 1 << 20
    # > 0: every layer attends over at most this many latest positions, so pages that lie wholly before the window of the
    # next query are handed back to the pool while the sequence runs (the reference keeps a ring of `window` rows per layer,
    # oxidize-core/src/compute/kv_cache/cache.rs; with pages the ring becomes "free what fell out of the window")
    attention_window: int = 0


class Sequence:
    _ids = itertools.count()

    def __init__(self, prompt: Sequence[int], params: SamplingParams, request_id: Optional[str] = None,
                 arrival: float = 0.0):
        self.seq_id = next(Sequence._ids)
        self.request_id = request_id if request_id is not None else str(self.seq_id)
        self.prompt: List[int] = list(prompt)
        self.output: List[int] = []
        self.params = params
        self.status = SeqStatus.WAITING
        self.blocks: List[int] = []
        self.num_computed = 0  # tokens whose KV is in the cache
        self.finish_reason: Optional[str] = None
        self.rng = RequestRng(params.seed)
        self.arrival = arrival
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self._hash_state = FNV_OFFSET  # rolling prefix hash up to the last published block
        self._published = 0  # number of blocks published to the prefix cache
        self.draft_tokens: List[int] = []  # speculative rows scheduled this step
        self.num_cached_tokens = 0
        # leading pages already returned to the pool (sliding-window models); their slots in `blocks` repeat the id of the
        # first live page so that the block table stays a table of valid ids
        self._released = 0
        # prompt positions whose embedding comes from the request (image tokens) and the rows [n, hidden] that go there;
        # such a sequence neither reads nor feeds the prefix cache (its placeholder tokens do not identify its content)
        self.embed_positions: List[int] = []
        self.input_embeds = None

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def remaining_prefill(self) -> int:
        # tokens not yet in KV, excluding the last sampled token that the next decode feeds
        return max(0, len(self.prompt) - self.num_computed) if not self.output else 0

    @property
    def is_finished(self) -> bool:
        return self.status is SeqStatus.FINISHED

    def token_at(self, i: int) -> int:
        return self.prompt[i] if i < len(self.prompt) else self.output[i - len(self.prompt)]


@dataclass
class ScheduledSeq:
    seq: Sequence
    start: int  # first position fed this step
    num_tokens: int  # rows fed this step
    is_prefill: bool
    sample: bool  # whether the last row's logits are sampled


@dataclass
class SchedulerOutput:
    scheduled: List[ScheduledSeq]
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    preempted: List[Sequence] = field(default_factory=list)
    cow_copies: List[Tuple[int, int]] = field(default_factory=list)  # (src, dst) block copies to perform

    @property
    def total_tokens(self) -> int:
        return self.num_prefill_tokens + self.num_decode_tokens

    @property
    def is_empty(self) -> bool:
        return not self.scheduled


class Scheduler:
    def __init__(self, config: SchedulerConfig, pool: BlockPool):
        self.config = config
        self.pool = pool
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.finished: List[Sequence] = []
        self.num_preemptions = 0

    # ---- queue management
    def add(self, seq: Sequence) -> None:
        if len(seq.prompt) == 0:
            raise ValueError("empty prompt")
        if len(seq.prompt) + seq.params.max_tokens > self.config.max_model_len:
            raise ValueError("prompt + max_tokens exceeds max_model_len")
        need = (len(seq.prompt) + self.pool.page_size) // self.pool.page_size
        if need > self.pool.num_blocks:
            raise OutOfBlocks(f"prompt needs {need} KV blocks, pool has {self.pool.num_blocks}")
        self.waiting.append(seq)

    def abort(self, request_id: str) -> bool:
        for s in list(self.running) + list(self.waiting):
            if s.request_id == request_id:
                self._finish(s, "abort")
                return True
        return False

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _finish(self, seq: Sequence, reason: str) -> None:
        if seq.is_finished:
            return
        seq.status = SeqStatus.FINISHED
        seq.finish_reason = reason
        self.pool.release_all(seq.blocks[seq._released:])
        seq.blocks, seq._released = [], 0
        if seq in self.running:
            self.running.remove(seq)
        try:
            self.waiting.remove(seq)
        except ValueError:
            pass
        self.finished.append(seq)

    def _preempt(self, seq: Sequence) -> None:
        self.pool.release_all(seq.blocks[seq._released:])
        seq.blocks, seq._released = [], 0
        seq.num_computed = 0
        seq._hash_state = FNV_OFFSET
        seq._published = 0
        seq.status = SeqStatus.WAITING
        # recompute-style preemption: generated tokens become part of the prompt to re-prefill
        seq.prompt = seq.prompt + seq.output
        seq._preempted_outputs = getattr(seq, "_preempted_outputs", []) + seq.output
        seq.output = []
        self.running.remove(seq)
        self.waiting.appendleft(seq)
        self.num_preemptions += 1

    # ---- block bookkeeping
    def _ensure_blocks(self, seq: Sequence, upto_tokens: int, out: SchedulerOutput) -> bool:
        """Make sure ``seq`` owns blocks for positions < upto_tokens; False when the pool is dry."""
        ps = self.pool.page_size
        need = (upto_tokens + ps - 1) // ps
        fresh = need - len(seq.blocks)
        # copy-on-write: the block that receives this step's first write may be shared.  Blocks are
        # shared only through the prefix cache, i.e. among the first ``_published`` blocks of a sequence
        # (those it matched at admission or published itself), so later blocks need no pool query.
        first_write_block = seq.num_computed // ps
        cow = (first_write_block < seq._published and first_write_block < len(seq.blocks)
               and self.pool.is_shared(seq.blocks[first_write_block]))
        if fresh <= 0 and not cow:
            return True
        if not self.pool.can_allocate(max(fresh, 0) + (1 if cow else 0)):
            return False
        if cow:
            old = seq.blocks[first_write_block]
            new = self.pool.allocate()
            out.cow_copies.append((old, new))
            self.pool.release(old)
            seq.blocks[first_write_block] = new
        for _ in range(max(fresh, 0)):
            seq.blocks.append(self.pool.allocate())
        return True

    def _publish_full_blocks(self, seq: Sequence) -> None:
        if not self.config.enable_prefix_cache or seq.input_embeds is not None:
            return
        ps = self.pool.page_size
        n_prompt_full = len(seq.prompt) // ps
        full = min(seq.num_computed // ps, n_prompt_full)
        while seq._published < full:
            i = seq._published
            seq._hash_state = block_hash(seq.prompt[i * ps : (i + 1) * ps], seq._hash_state)
            self.pool.publish(seq.blocks[i], seq._hash_state)
            seq._published += 1

    def _admit(self, seq: Sequence) -> None:
        """Attach cached prefix blocks to a sequence entering prefill."""
        if seq.num_computed == 0 and not seq.blocks and self.config.enable_prefix_cache and seq.input_embeds is None:
            blocks, covered = self.pool.match_prefix(seq.prompt)
            if blocks:
                seq.blocks = blocks
                seq.num_computed = covered
                seq.num_cached_tokens = covered
                ps = self.pool.page_size
                seq._hash_state = block_hash(seq.prompt[:covered])
                seq._published = covered // ps

    # ---- the step
    def schedule(self) -> SchedulerOutput:
        cfg = self.config
        out = SchedulerOutput([])
        budget = cfg.max_num_batched_tokens

        # Phase 1: decode for fully-prefilled running sequences (highest priority)
        RUNNING = SeqStatus.RUNNING
        partial = False  # some running sequence is still in prefill
        for seq in list(self.running):
            # (a sequence preempted earlier in this loop is WAITING again)
            if seq.status is not RUNNING:
                continue
            if not seq.output and seq.num_computed < len(seq.prompt):  # remaining_prefill > 0
                partial = True
                continue
            nd = len(seq.draft_tokens)
            n = 1 + nd
            if budget < n:
                partial = True  # the rest of the list was not looked at
                break
            ntok = len(seq.prompt) + len(seq.output)
            while not self._ensure_blocks(seq, ntok + nd, out):
                victim = self._pick_victim(exclude=seq)
                if victim is None:
                    break
                self._preempt(victim)
                out.preempted.append(victim)
                out.scheduled = [s for s in out.scheduled if s.seq is not victim]
            else:
                out.scheduled.append(ScheduledSeq(seq, ntok - 1, n, False, True))
                budget -= n
                out.num_decode_tokens += n
                continue
            # could not get a block even after preempting everyone else
            self._preempt(seq)
            out.preempted.append(seq)

        # Phase 2: continue partial prefills
        for seq in (list(self.running) if partial else ()):
            if seq.status is not RUNNING or seq.remaining_prefill == 0:
                continue
            chunk = min(seq.remaining_prefill, cfg.prefill_chunk_size, budget)
            if chunk <= 0:
                continue
            if not self._ensure_blocks(seq, seq.num_computed + chunk, out):
                continue
            last = seq.num_computed + chunk == len(seq.prompt)
            out.scheduled.append(ScheduledSeq(seq, seq.num_computed, chunk, True, last))
            budget -= chunk
            out.num_prefill_tokens += chunk

        # Phase 3: admit from the waiting queue
        if cfg.policy == "sjf" and len(self.waiting) > 1:
            self.waiting = deque(sorted(self.waiting, key=lambda s: (len(s.prompt) + s.params.max_tokens, s.seq_id)))
        still: Deque[Sequence] = deque()
        blocked = False
        while self.waiting:
            seq = self.waiting.popleft()
            if blocked or len(self.running) >= cfg.max_num_running_seqs or budget <= 0 or seq in out.preempted:
                still.append(seq)
                continue
            self._admit(seq)
            chunk = min(seq.remaining_prefill, cfg.prefill_chunk_size, budget)
            if chunk <= 0 or not self._ensure_blocks(seq, seq.num_computed + chunk, out):
                # FCFS: do not let later arrivals overtake a request that does not fit yet
                if seq.blocks and seq.num_cached_tokens and seq.num_computed == seq.num_cached_tokens:
                    self.pool.release_all(seq.blocks)
                    seq.blocks, seq.num_computed, seq.num_cached_tokens = [], 0, 0
                    seq._hash_state, seq._published = FNV_OFFSET, 0
                still.append(seq)
                blocked = True
                continue
            seq.status = SeqStatus.RUNNING
            self.running.append(seq)
            last = seq.num_computed + chunk == len(seq.prompt)
            out.scheduled.append(ScheduledSeq(seq, seq.num_computed, chunk, True, last))
            budget -= chunk
            out.num_prefill_tokens += chunk
        self.waiting = still
        return out

    def _pick_victim(self, exclude: Sequence) -> Optional[Sequence]:
        for s in reversed(self.running):
            if s is not exclude:
                return s
        return None

    # ---- after the forward pass
    def postprocess(self, out: SchedulerOutput, new_tokens: Dict[int, List[int]], eos_token_id: Optional[int] = None,
                    now: float = 0.0) -> List[Sequence]:
        """Advance every scheduled sequence; ``new_tokens[seq_id]`` holds the tokens sampled
        for it this step (one, or several after a speculative verify).  Returns the sequences
        that finished."""
        done: List[Sequence] = []
        ps = self.pool.page_size
        publish = self.config.enable_prefix_cache
        FINISHED = SeqStatus.FINISHED
        for ss in out.scheduled:
            seq = ss.seq
            if seq.status is FINISHED:
                continue
            toks = new_tokens.get(seq.seq_id, [])
            if ss.is_prefill:
                seq.num_computed += ss.num_tokens
            else:
                # rows fed: last token + drafts; accepted drafts = len(toks)-1
                seq.num_computed = len(seq.prompt) + len(seq.output) - 1 + max(len(toks), 1)
            if seq.draft_tokens:
                seq.draft_tokens = []
            if publish and seq._published < len(seq.prompt) // ps:
                self._publish_full_blocks(seq)
            if self.config.attention_window > 0:
                self._release_outside_window(seq)
            if not ss.sample:
                continue
            for t in toks:
                seq.output.append(int(t))
                if seq.first_token_time is None:
                    seq.first_token_time = now
                reason = self._stop_reason(seq, int(t), eos_token_id)
                if reason:
                    seq.finish_time = now
                    self._finish(seq, reason)
                    done.append(seq)
                    break
            if seq.status is not FINISHED and (len(seq.blocks) - 1) * ps >= len(seq.prompt) + len(seq.output):
                self._trim_blocks(seq)  # more pages than the tokens need (speculative rows that were rejected)
        return done

    def _release_outside_window(self, seq: Sequence) -> None:
        """Return the pages no later query of ``seq`` can see: the next query sits at position ``num_computed`` and sees
        keys at positions > num_computed - window, so a page whose last position is <= num_computed - window is dead."""
        ps = self.pool.page_size
        dead = min(max(0, (seq.num_computed - self.config.attention_window) // ps), len(seq.blocks) - 1)
        if dead <= seq._released:
            return
        keep = seq.blocks[dead]
        for i in range(seq._released, dead):
            self.pool.release(seq.blocks[i])  # a page published to the prefix cache stays findable there until evicted
        seq.blocks[:dead] = [keep] * dead  # every dead slot names a page this sequence still owns
        seq._released = dead

    def _trim_blocks(self, seq: Sequence) -> None:
        """Free tail pages past what the accepted tokens need (speculative rollback)."""
        ps = self.pool.page_size
        need = (seq.num_tokens + ps - 1) // ps
        while len(seq.blocks) > max(need, 1):
            self.pool.release(seq.blocks.pop())

    @staticmethod
    def _stop_reason(seq: Sequence, tok: int, eos: Optional[int]) -> Optional[str]:
        p = seq.params
        produced = len(seq.output) + len(getattr(seq, "_preempted_outputs", []))
        if not p.ignore_eos and eos is not None and tok == eos:
            return "stop"
        if tok in p.stop_token_ids:
            return "stop"
        for ss in p.stop_sequences:
            if ss and len(seq.output) >= len(ss) and tuple(seq.output[-len(ss):]) == tuple(ss):
                return "stop"
        if produced >= p.max_tokens:
            return "length"
        return None
