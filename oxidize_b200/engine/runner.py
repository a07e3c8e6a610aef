"""Model runner: turns a scheduler output into one flat device batch, runs the forward pass
(CUDA-graph replay for decode-only steps), samples, and hands tokens back to the host.

Per step the host writes ONE pinned int32 staging buffer laid out as
``[token_ids | positions | slot_mapping | query_start | seq_lens | logits_indices |
block_tables]`` plus a small float section with per-sequence sampling knobs and this step's
uniform draws; one async copy moves it to a device buffer of identical layout whose
sub-views have fixed addresses, so captured graphs stay valid (the role of the reference's
3-word ``{pos, context, token}`` device state, ``backends/cuda/cuda_decode_graph.rs:45-52``,
generalised to a whole batch).  The only device→host traffic is the sampled token ids.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..models.transformer import BatchMeta, Transformer
from .kv_pool import KVCache
from .sampler import SamplingParams, sample as host_sample
from .scheduler import ScheduledSeq, SchedulerOutput

DECODE_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def _bucket(n: int, buckets=DECODE_BUCKETS) -> int:
    for b in buckets:
        if n <= b:
            return b
    return n


class StagingBuffers:
    """Host (pinned on CUDA) + device mirror of the per-step integer/float inputs."""

    def __init__(self, max_tokens: int, max_seqs: int, max_blocks_per_seq: int, device: torch.device):
        self.max_tokens, self.max_seqs, self.max_blocks = max_tokens, max_seqs, max_blocks_per_seq
        T, B, M = max_tokens, max_seqs, max_blocks_per_seq
        sizes = [("token_ids", T), ("positions", T), ("slot_mapping", T), ("query_start", B + 1), ("seq_lens", B),
                 ("logits_indices", T), ("top_k", T), ("block_tables", B * M)]
        fsizes = [("temperature", T), ("top_p", T), ("min_p", T), ("random", T)]
        self.offsets: Dict[str, Tuple[int, int]] = {}
        off = 0
        for name, n in sizes + fsizes:
            n4 = (n + 3) // 4 * 4  # keep every section 16-byte aligned
            self.offsets[name] = (off, n)
            off += n4
        self.total = off
        pin = device.type == "cuda"
        # Two pinned host copies, used alternately: with one step running ahead of the host (LLM.step), the copy of
        # step k may not have been read by the copy engine yet when the host fills in step k + 1.
        self.hosts = [torch.zeros(self.total, dtype=torch.int32, pin_memory=pin) for _ in range(2 if pin else 1)]
        self._np = [h.numpy() for h in self.hosts]
        self._npf = [a.view(np.float32) for a in self._np]
        self.which = 0
        self.host = self.hosts[0]
        self.host_np = self._np[0]
        self.host_f = self._npf[0]
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device) if pin else self.host
        self.device = device
        self._float_names = {n for n, _ in fsizes}
        self.tokens_end = self.offsets["positions"][0]  # the token ids are the first section

    def flip(self) -> int:
        """Switch to the other host copy; returns its index."""
        self.which = (self.which + 1) % len(self.hosts)
        self.host, self.host_np, self.host_f = self.hosts[self.which], self._np[self.which], self._npf[self.which]
        return self.which

    def h(self, name: str) -> np.ndarray:
        o, n = self.offsets[name]
        return (self.host_f if name in self._float_names else self.host_np)[o : o + n]

    def d(self, name: str, n: Optional[int] = None) -> torch.Tensor:
        o, full = self.offsets[name]
        v = self.dev[o : o + (full if n is None else n)]
        return v.view(torch.float32) if name in self._float_names else v

    def upload(self, skip_tokens: bool = False) -> int:
        """Async H2D of the staging area (without the token ids when the device already holds them); returns bytes moved."""
        o = self.tokens_end if skip_tokens else 0
        if self.dev is not self.host:
            self.dev[o:].copy_(self.host[o:], non_blocking=True)
        return (self.total - o) * 4


@dataclass
class StepResult:
    tokens: Dict[int, List[int]]  # seq_id -> sampled tokens
    logits: Optional[torch.Tensor] = None
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    launches: int = 0


@dataclass
class Pending:
    """A launched step whose sampled tokens have not been read back yet."""

    rows: list
    n_out: int
    toks: Optional[torch.Tensor]
    host_buf: Optional[torch.Tensor]
    event: object
    logits: Optional[torch.Tensor]
    host_rows: list
    keep_logits: bool
    h2d_bytes: int
    bucket: int = 0  # decode-graph bucket the step replayed, 0 = eager
    seq_ids: tuple = ()  # row order of the step (decode-only steps)
    finished: bool = True  # the token copy to the host has been enqueued (pipeline stages do that in finish())


class ModelRunner:
    def __init__(self, model: Transformer, kv: KVCache, max_tokens: int, max_seqs: int, max_model_len: int,
                 use_cuda_graphs: bool = True):
        self.model = model
        self.kv = kv
        self.device = model.device
        self.page = kv.page_size
        self.max_blocks = (max_model_len + self.page - 1) // self.page
        self.buf = StagingBuffers(max_tokens, max_seqs, self.max_blocks, self.device)
        # (a pipeline stage exchanges activations with its neighbours inside the step: no graph capture)
        self.use_graphs = use_cuda_graphs and self.device.type == "cuda" and getattr(model, "pipe", None) is None
        self.graphs: Dict[int, "torch.cuda.CUDAGraph"] = {}
        self.graph_out: Dict[int, torch.Tensor] = {}
        self.out_hosts = [torch.zeros(max(max_tokens, max_seqs), dtype=torch.int32, pin_memory=self.device.type == "cuda")
                          for _ in range(2)]
        self._out_which = 0
        self.keep_logits = False
        self._bt_owners = [[None] * max_seqs for _ in self.buf.hosts]

    # ------------------------------------------------------------------ batch building
    def build(self, scheduled: Sequence[ScheduledSeq], pad_to: Optional[int] = None):
        """Fill the staging buffer; returns (T, B, n_logits, max_q, max_len, sample_rows)."""
        b = self.buf
        tok, pos, slot = b.h("token_ids"), b.h("positions"), b.h("slot_mapping")
        qs, sl, li, bt = b.h("query_start"), b.h("seq_lens"), b.h("logits_indices"), b.h("block_tables")
        M, ps = self.max_blocks, self.page
        t = 0
        nl = 0
        max_q = 0
        max_len = 0
        rows: List[Tuple[ScheduledSeq, int, int]] = []  # (ss, first logits row, n rows)
        qs[0] = 0
        self._bt_owners[b.which] = [None] * b.max_seqs  # this path rewrites block-table rows: the decode path's record is void
        for i, ss in enumerate(scheduled):
            seq = ss.seq
            n = ss.num_tokens
            if t + n > b.max_tokens or i >= b.max_seqs:
                raise RuntimeError("scheduled batch exceeds runner capacity")
            start = ss.start
            blist = seq.blocks
            nb = len(blist)
            # the block list changes once per page: keep its array form on the sequence
            cache = getattr(seq, "_blocks_np", None)
            if cache is None or cache[0] != nb or cache[1] != (blist[-1] if nb else -1):
                cache = (nb, blist[-1] if nb else -1, np.asarray(blist, dtype=np.int32))
                seq._blocks_np = cache
            bt[i * M : i * M + nb] = cache[2]
            if n == 1 and not ss.is_prefill:
                # decode row: plain integer arithmetic, no temporaries
                tok[t] = seq.token_at(start)
                pos[t] = start
                slot[t] = blist[start // ps] * ps + start % ps
                sl[i] = start + 1
                qs[i + 1] = t + 1
                if ss.sample:
                    li[nl] = t
                    rows.append((ss, nl, 1))
                    nl += 1
                if max_q < 1:
                    max_q = 1
                if start + 1 > max_len:
                    max_len = start + 1
                t += 1
                continue
            if ss.is_prefill:
                tok[t : t + n] = seq.prompt[start : start + n]
            else:
                tok[t] = seq.token_at(start)
                if n > 1:
                    tok[t + 1 : t + n] = seq.draft_tokens
            p = np.arange(start, start + n, dtype=np.int32)
            pos[t : t + n] = p
            slot[t : t + n] = cache[2][p // ps] * ps + p % ps
            sl[i] = start + n
            qs[i + 1] = t + n
            if ss.sample:
                k = n if (not ss.is_prefill and n > 1) else 1
                li[nl : nl + k] = np.arange(t + n - k, t + n, dtype=np.int32)
                rows.append((ss, nl, k))
                nl += k
            max_q = max(max_q, n)
            max_len = max(max_len, start + n)
            t += n
        B = len(scheduled)
        if pad_to is not None and pad_to > B:
            # dummy sequences: zero context, no KV write; their logits rows are ignored
            for i in range(B, pad_to):
                tok[t] = 0
                pos[t] = 0
                slot[t] = -1
                sl[i] = 0
                qs[i + 1] = t + 1
                li[nl] = t
                nl += 1
                t += 1
            B = pad_to
        return t, B, nl, max_q, max_len, rows

    def build_decode(self, scheduled: Sequence[ScheduledSeq], pad_to: Optional[int] = None, skip_tokens: bool = False):
        """``build`` for the steady state: every sequence feeds exactly one decode row.  Whole-column
        writes instead of per-row scalar stores, and a block-table row is rewritten only when its
        sequence or that sequence's block list changed since the previous step."""
        b = self.buf
        n = len(scheduled)
        if n > b.max_tokens or n > b.max_seqs:
            raise RuntimeError("scheduled batch exceeds runner capacity")
        tok, pos, slot = b.h("token_ids"), b.h("positions"), b.h("slot_mapping")
        qs, sl, li, bt = b.h("query_start"), b.h("seq_lens"), b.h("logits_indices"), b.h("block_tables")
        M, ps = self.max_blocks, self.page
        owner = self._bt_owners[b.which]
        ar = getattr(self, "_arange", None)
        if ar is None:
            ar = self._arange = np.arange(max(b.max_seqs, b.max_tokens) + 1, dtype=np.int32)
        seqs = [ss.seq for ss in scheduled]
        starts = [ss.start for ss in scheduled]
        for i, seq in enumerate(seqs):
            bl = seq.blocks
            nb = len(bl)
            key = (seq.seq_id, id(bl), nb, bl[-1] if nb else -1)
            if owner[i] != key:
                bt[i * M : i * M + nb] = bl
                owner[i] = key
        if not skip_tokens:  # (skipped: the previous step's kernel left the ids in the device copy)
            tok[:n] = [seq.token_at(st) for seq, st in zip(seqs, starts)]
        pos[:n] = starts
        slot[:n] = [seq.blocks[st // ps] * ps + st % ps for seq, st in zip(seqs, starts)]
        np.add(pos[:n], 1, out=sl[:n])
        qs[: n + 1] = ar[: n + 1]
        if all(ss.sample for ss in scheduled):
            rows = [(ss, i, 1) for i, ss in enumerate(scheduled)]
            nl = n
            li[:n] = ar[:n]
        else:
            rows, nl = [], 0
            for i, ss in enumerate(scheduled):
                if ss.sample:
                    li[nl] = i
                    rows.append((ss, nl, 1))
                    nl += 1
        t, B = n, n
        max_len = max(starts) + 1
        if pad_to is not None and pad_to > B:
            # dummy sequences: zero context, no KV write; their logits rows are ignored
            k = pad_to - B
            if not skip_tokens:
                tok[t : t + k] = 0
            pos[t : t + k] = 0
            slot[t : t + k] = -1
            sl[B:pad_to] = 0
            qs[B + 1 : pad_to + 1] = ar[t + 1 : t + k + 1]
            li[nl : nl + k] = ar[t : t + k]
            nl += k
            t += k
            B = pad_to
        return t, B, nl, 1, max_len, rows

    def _fill_sampling(self, rows, n_logits: int) -> bool:
        """Per-logits-row sampling knobs; returns True when every row is greedy."""
        b = self.buf
        temp, tp, mp, rnd, tk = b.h("temperature"), b.h("top_p"), b.h("min_p"), b.h("random"), b.h("top_k")
        all_greedy = True
        temp[:n_logits] = 0.0
        greedy: Dict[int, bool] = {}  # many requests share one params object
        for ss, r0, k in rows:
            p: SamplingParams = ss.seq.params
            g = greedy.get(id(p))
            if g is None:
                g = greedy[id(p)] = p.is_greedy
            if g:
                continue
            all_greedy = False
            for j in range(r0, r0 + k):
                temp[j] = p.temperature
                tp[j] = p.top_p if p.top_p is not None else 1.0
                mp[j] = p.min_p if p.min_p is not None else 0.0
                tk[j] = p.top_k if p.top_k is not None else 0
                rnd[j] = ss.seq.rng.next()
        return all_greedy

    def _meta(self, T: int, B: int, nl: int, max_q: int, max_len: int, logits_all: bool = False) -> BatchMeta:
        b = self.buf
        return BatchMeta(
            logits_all=logits_all,
            token_ids=b.d("token_ids", T), positions=b.d("positions", T), slot_mapping=b.d("slot_mapping", T),
            query_start=b.d("query_start", B + 1), seq_lens=b.d("seq_lens", B),
            block_tables=b.d("block_tables").view(b.max_seqs, self.max_blocks)[:B],
            logits_indices=b.d("logits_indices", nl), max_query_len=max_q, max_seq_len=max_len, num_seqs=B)

    def _embed_overrides(self, scheduled: Sequence[ScheduledSeq], meta: BatchMeta) -> None:
        """Prompt positions of this step's prefill rows whose embedding is given by the request (image tokens) instead of
        the token table: collected as (batch rows, embedding rows) for the model's embedding stage."""
        rows: List[int] = []
        vecs: List[torch.Tensor] = []
        t = 0
        for ss in scheduled:
            emb = getattr(ss.seq, "input_embeds", None)
            if emb is not None and ss.is_prefill:
                lo, hi = ss.start, ss.start + ss.num_tokens
                for j, p in enumerate(ss.seq.embed_positions):
                    if lo <= p < hi:
                        rows.append(t + p - lo)
                        vecs.append(emb[j])
            t += ss.num_tokens
        if rows:
            meta.extra["embed_overrides"] = (torch.tensor(rows, dtype=torch.int64, device=self.device),
                                             torch.stack(vecs).to(self.device))

    # ------------------------------------------------------------------ execution
    def _forward_sample(self, meta: BatchMeta, all_greedy: bool, tie: str, feed: Optional[torch.Tensor] = None):
        if all_greedy and not self.keep_logits:
            return self.model.greedy_tokens(meta, self.kv, tie, feed=feed), None
        logits = self.model.forward(meta, self.kv)
        if logits is None:
            return None, None  # not the last pipeline stage: the tokens come from there
        if all_greedy:
            return ops.argmax(logits, tie), logits
        from . import device_sampler

        nl = logits.shape[0]
        b = self.buf
        return device_sampler.sample(logits, b.d("temperature", nl), b.d("top_k", nl), b.d("top_p", nl),
                                     b.d("min_p", nl), b.d("random", nl), tie), logits

    def execute(self, out: SchedulerOutput, needs_host_logits: bool = False) -> StepResult:
        p = self.launch(out, needs_host_logits)
        return self.collect(p) if p is not None else StepResult({})

    def launch(self, out: SchedulerOutput, needs_host_logits: bool = False, tokens_on_device: bool = False) -> Optional[Pending]:
        """Build, upload and enqueue one step and the copy of its sampled tokens to the host, without waiting for it.
        ``tokens_on_device``: the step continues the decode step launched just before it with the same sequences in
        the same rows, whose kernel left each row's next input id in the device staging buffer."""
        p = self.launch_forward(out, needs_host_logits, tokens_on_device)
        return self.finish(p) if p is not None else None

    def finish(self, p: Pending) -> Pending:
        """Second half of a launch: every pipeline stage obtains the tokens the last stage sampled, and the copy of
        the tokens to the host is enqueued.  Separate from ``launch_forward`` so that a stage can push several
        micro-batches into the pipeline before it waits for the first one's tokens."""
        if p.finished:
            return p
        pipe = getattr(self.model, "pipe", None)
        if pipe is not None:
            pipe.broadcast_tokens(p.toks)
        if self.device.type == "cuda":
            self._out_which ^= 1
            hb = self.out_hosts[self._out_which]
            hb[: p.n_out].copy_(p.toks, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            p.host_buf, p.event = hb, ev
        p.finished = True
        return p

    def launch_forward(self, out: SchedulerOutput, needs_host_logits: bool = False,
                       tokens_on_device: bool = False) -> Optional[Pending]:
        scheduled = out.scheduled
        if not scheduled:
            return None
        for src, dst in out.cow_copies:
            self.kv.copy_block(src, dst)
        # the scheduler's own counts settle the common case without a scan of the rows
        decode_only = ((out.num_prefill_tokens == 0 and out.num_decode_tokens == len(scheduled))
                       or all((not s.is_prefill) and s.num_tokens == 1 for s in scheduled))
        # (a model that records layer outputs for a hidden-conditioned draft runs eagerly: the recorded tensors must be
        # this step's own, not a captured graph's private buffers)
        graphable = (self.use_graphs and decode_only and not needs_host_logits and not self.keep_logits
                     and not getattr(self.model, "capture_layers", None))
        pad_to = _bucket(len(scheduled)) if graphable else None
        if pad_to is not None and pad_to > self.buf.max_seqs:
            pad_to, graphable = None, False
        self.buf.flip()
        if decode_only:
            T, B, nl, max_q, max_len, rows = self.build_decode(scheduled, pad_to, skip_tokens=tokens_on_device)
        else:
            T, B, nl, max_q, max_len, rows = self.build(scheduled, pad_to)
        self.last_rows = rows
        on_host = {id(p): p.needs_host_sampler for p in {id(r[0].seq.params): r[0].seq.params for r in rows}.values()}
        host_rows = [r for r in rows if on_host[id(r[0].seq.params)]] if any(on_host.values()) else []
        needs_host_logits = needs_host_logits or bool(host_rows)
        graphable = graphable and not host_rows
        all_greedy = self._fill_sampling(rows, nl)
        tie = scheduled[0].seq.params.tie
        if tokens_on_device and not (decode_only and all_greedy and (graphable or self.device.type != "cuda")):
            raise RuntimeError("a step that takes its input ids from the device must be a greedy decode step")
        h2d = self.buf.upload(skip_tokens=tokens_on_device)
        logits = None
        bucket = 0
        feed = self.buf.d("token_ids", B) if decode_only and all_greedy and nl == T else None
        if graphable and all_greedy:
            toks = self._replay(B, tie)
            bucket = B
        else:
            meta = self._meta(T, B, nl, max_q, max_len, logits_all=decode_only and nl == T)
            if not decode_only:
                self._embed_overrides(scheduled, meta)
            toks, logits = self._forward_sample(meta, all_greedy and not needs_host_logits, tie,
                                                feed=feed if not needs_host_logits else None)
        if toks is None:  # not the last pipeline stage
            toks = torch.empty(nl, dtype=torch.int32, device=self.device)
        toks = toks.to(torch.int32) if toks.dtype != torch.int32 else toks
        return Pending(rows, toks.shape[0], toks, None, None, logits, host_rows, needs_host_logits or self.keep_logits, h2d,
                       bucket, tuple(ss.seq.seq_id for ss in scheduled) if decode_only else (), finished=False)

    def collect(self, p: Pending) -> StepResult:
        """Wait for a launched step and return its tokens."""
        if p.event is not None:
            p.event.synchronize()
            host = p.host_buf[: p.n_out].numpy()
        else:
            host = p.toks.numpy()
        hl = host.tolist()
        result: Dict[int, List[int]] = {ss.seq.seq_id: hl[r0 : r0 + k] for ss, r0, k in p.rows}
        pipe = getattr(self.model, "pipe", None)
        if p.host_rows:
            if pipe is None:
                self._host_sample(p.host_rows, p.logits, result)
            else:
                # only the last stage holds the logits: it draws, everybody gets the outcome
                if pipe.is_last:
                    self._host_sample(p.host_rows, p.logits, result)
                result = pipe.broadcast_object(result if pipe.is_last else None)
        return StepResult(result, p.logits if p.keep_logits else None, p.h2d_bytes, p.n_out * 4)

    def _host_sample(self, host_rows, logits: torch.Tensor, result: Dict[int, List[int]]) -> None:
        """Rows whose parameters the device kernel does not cover (penalties, typical / tail-free,
        Mirostat, grammar) are drawn on the host from their logits; the grammar state advances here."""
        idx = torch.tensor([r0 + j for _, r0, k in host_rows for j in range(k)], dtype=torch.long, device=logits.device)
        lg = logits.index_select(0, idx).float().cpu().numpy()
        n = 0
        for ss, r0, k in host_rows:
            seq = ss.seq
            state = seq.__dict__.setdefault("sampler_state", {})
            recent = seq.all_tokens
            toks = []
            for j in range(k):
                tok = host_sample(lg[n], seq.params, seq.rng.next(), recent, state=state)
                n += 1
                toks.append(tok)
                if j + 1 < k and tok != result[seq.seq_id][j]:
                    break  # a speculative row diverged from the draft: later rows are void
                recent = recent + [tok]
            if seq.params.grammar is not None:
                for t in toks:
                    seq.params.grammar.advance(state, t)
            result[seq.seq_id] = toks

    def _replay(self, B: int, tie: str) -> torch.Tensor:
        g = self.graphs.get(B)
        if g is None:
            g = self._capture(B, tie)
        g.replay()
        return self.graph_out[B]

    def _capture(self, B: int, tie: str):
        """Capture one decode step for bucket ``B`` (every sequence feeds exactly one row)."""
        meta = self._meta(B, B, B, 1, self.max_blocks * self.page, logits_all=True)
        feed = self.buf.d("token_ids", B)  # every row's next input id, left on the device for a step that runs ahead
        # warm up on a side stream so lazy initialisation does not land inside the capture
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                # (no token feed here: these runs execute for real and must leave the step's input ids alone)
                self.model.greedy_tokens(meta, self.kv, tie)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        from ..ops import cuda as opcuda

        n0 = opcuda.launch_count
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self.model.greedy_tokens(meta, self.kv, tie, feed=feed)
        if not hasattr(self, "launches_per_step"):
            self.launches_per_step = {}
        self.launches_per_step[B] = opcuda.launch_count - n0
        self.graphs[B] = g
        self.graph_out[B] = out
        return g
