"""Speculative decoding: a draft model (separate GGUF) or the in-GGUF multi-token-prediction
head proposes K tokens per sequence, the target verifies all K+1 rows in ONE batched forward over
the paged KV cache, accepted drafts keep their KV entries and the rest is rolled back.

Step structure of the reference (``SpeculativeGenerationStream::run_speculative_step``,
``oxidize-core/src/model/generation.rs:230-326``; MTP variant ``:421`` with
``draft_mtp_tokens`` ``inference/mtp.rs:10-146``; acceptance rule ``sampling.rs:492-623``;
health auto-disable after 2 zero-accept rounds or acceptance < 0.2 after 4K drafts
``generation.rs:209-228``; stats ``speculative.rs:98-139``).  Differences: verification is one
multi-row attention launch for the whole batch instead of a rewind + re-forward per sequence, and
rollback is "free the tail pages" in the block pool.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .. import ops
from .kv_pool import BlockPool, KVCache, KVCacheSpec, make_block_pool
from .runner import ModelRunner
from .sampler import GREEDY, SamplingParams
from .scheduler import ScheduledSeq, SchedulerOutput, Sequence

MAX_DRAFT_TOKENS_PER_STEP = 64


@dataclass
class SpecStats:
    proposed: int = 0
    accepted: int = 0
    target_forwards: int = 0
    emitted: int = 0
    zero_rounds: int = 0
    disabled: bool = False

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    @property
    def tokens_per_target_forward(self) -> float:
        return self.emitted / self.target_forwards if self.target_forwards else 0.0

    def estimated_speedup(self, draft_cost_ratio: float, k: int) -> float:
        """Tokens per unit of target-forward time, relative to plain decoding."""
        return self.tokens_per_target_forward / (1.0 + draft_cost_ratio * k) if self.target_forwards else 1.0


def verify_greedy(drafts: List[int], target: List[int]) -> List[int]:
    """Exact-match rule: keep drafts while they equal the target's argmax; the first mismatch is
    replaced by the target's token; if all match, the target's extra row is a bonus token."""
    out: List[int] = []
    for i, d in enumerate(drafts):
        if target[i] == d:
            out.append(d)
        else:
            out.append(target[i])
            return out
    out.append(target[len(drafts)])
    return out


class DraftModelProposer:
    """Runs a small draft model with its own paged KV; one shadow sequence per target sequence."""

    def __init__(self, draft_weights, k: int, max_seqs: int, max_model_len: int, num_blocks: int = 0, comm=None):
        from ..models.transformer import Transformer

        self.k = k
        self.model = Transformer(draft_weights, comm)
        dev = self.model.device
        cfg = draft_weights.cfg
        page = 16
        nblocks = num_blocks or max_seqs * ((max_model_len + page - 1) // page + 1)
        kvd = "bf16" if dev.type == "cuda" else "f32"
        self.kv = KVCache(KVCacheSpec(len(draft_weights.layers), self.model.n_kv_local, cfg.head_dim, page, kvd), nblocks, dev)
        self.pool = make_block_pool(nblocks, page, enable_prefix_cache=False)
        self.runner = ModelRunner(self.model, self.kv, max(2048, max_seqs * (k + 2)), max_seqs, max_model_len, False)
        self.shadow: Dict[int, Sequence] = {}
        self.computed: Dict[int, int] = {}

    def _shadow(self, seq: Sequence) -> Sequence:
        sh = self.shadow.get(seq.seq_id)
        if sh is None:
            sh = Sequence([], GREEDY)
            self.shadow[seq.seq_id] = sh
            self.computed[seq.seq_id] = 0
        return sh

    def release(self, seq: Sequence) -> None:
        sh = self.shadow.pop(seq.seq_id, None)
        self.computed.pop(seq.seq_id, None)
        if sh is not None:
            self.pool.release_all(sh.blocks)

    def _ensure(self, sh: Sequence, n_tokens: int) -> None:
        need = (n_tokens + self.pool.page_size - 1) // self.pool.page_size
        while len(sh.blocks) < need:
            sh.blocks.append(self.pool.allocate())

    def propose(self, seqs: List[Sequence]) -> Dict[int, List[int]]:
        drafts: Dict[int, List[int]] = {s.seq_id: [] for s in seqs}
        # catch-up pass: everything the draft has not seen yet, including the last sampled token
        sched = []
        for s in seqs:
            sh = self._shadow(s)
            sh.prompt = s.all_tokens
            done = min(self.computed[s.seq_id], len(sh.prompt) - 1)
            self._ensure(sh, len(sh.prompt) + self.k)
            sched.append(ScheduledSeq(sh, done, len(sh.prompt) - done, True, True))
        for it in range(self.k):
            res = self.runner.execute(SchedulerOutput(list(sched)))
            sched = []
            for s in seqs:
                sh = self.shadow[s.seq_id]
                t = res.tokens[sh.seq_id][0]
                drafts[s.seq_id].append(t)
                sh.prompt = sh.prompt + [t]
                if it + 1 < self.k:
                    sched.append(ScheduledSeq(sh, len(sh.prompt) - 1, 1, True, True))
        for s in seqs:
            # KV is valid for every token fed so far (all but the last draft)
            self.computed[s.seq_id] = len(s.all_tokens) + self.k - 1
        return drafts

    def rollback(self, seq: Sequence, n_valid_tokens: int) -> None:
        if seq.seq_id in self.computed:
            self.computed[seq.seq_id] = min(self.computed[seq.seq_id], n_valid_tokens)


class MtpProposer:
    """Drafts with the model's own nextn layer: ``eh_proj([enorm(embed(tok)) ; hnorm(prev_hidden)])``
    → one decoder layer → ``shared_head_norm`` → head (``mtp_forward_one``, inference/mtp.rs:72-146).
    The MTP layer keeps its own single-layer KV and attends over the positions it has drafted
    at; verification by the target keeps the output exact whatever the draft quality."""

    def __init__(self, target_model, k: int, max_seqs: int, max_model_len: int):
        self.k = k
        self.m = target_model
        self.mtp = target_model.w.mtp[0]
        dev = target_model.device
        cfg = target_model.cfg
        page = 16
        nblocks = max_seqs * ((max_model_len + page - 1) // page + 1)
        kvd = "bf16" if dev.type == "cuda" else "f32"
        self.kv = KVCache(KVCacheSpec(1, target_model.n_kv_local, cfg.head_dim, page, kvd), nblocks, dev)
        self.pool = make_block_pool(nblocks, page, enable_prefix_cache=False)
        self.blocks: Dict[int, List[int]] = {}
        self.start: Dict[int, int] = {}
        self.hidden: Dict[int, torch.Tensor] = {}  # last verified hidden state per sequence
        self.max_blocks = (max_model_len + page - 1) // page

    def observe_hidden(self, seq: Sequence, h: torch.Tensor) -> None:
        self.hidden[seq.seq_id] = h

    def release(self, seq: Sequence) -> None:
        self.pool.release_all(self.blocks.pop(seq.seq_id, []))
        self.hidden.pop(seq.seq_id, None)
        self.start.pop(seq.seq_id, None)

    def rollback(self, seq: Sequence, n_valid_tokens: int) -> None:
        pass  # positions are rewritten on the next round

    def propose(self, seqs: List[Sequence]) -> Dict[int, List[int]]:
        from ..models.transformer import BatchMeta

        m, w, cfg = self.m, self.mtp, self.m.cfg
        dev = m.device
        ready = [s for s in seqs if s.seq_id in self.hidden]
        drafts: Dict[int, List[int]] = {s.seq_id: [] for s in seqs}
        if not ready:
            return drafts
        B = len(ready)
        i32 = dict(dtype=torch.int32, device=dev)
        toks = torch.tensor([s.all_tokens[-1] for s in ready], **i32)
        hid = torch.stack([self.hidden[s.seq_id] for s in ready]).to(m.act_dtype)
        pos0 = [s.num_tokens - 1 for s in ready]
        for s in ready:
            self.start.setdefault(s.seq_id, s.num_tokens - 1)
            need = (s.num_tokens + self.k + 15) // 16
            bl = self.blocks.setdefault(s.seq_id, [])
            while len(bl) < need:
                bl.append(self.pool.allocate())
        bt = torch.zeros(B, self.max_blocks, **i32)
        for i, s in enumerate(ready):
            bl = self.blocks[s.seq_id]
            bt[i, : len(bl)] = torch.tensor(bl, **i32)
        embed_table = w.embed if w.embed is not None else m.w.embed
        head = w.shared_head if w.shared_head is not None else m.w.lm_head
        for it in range(self.k):
            pos = torch.tensor([p + it for p in pos0], **i32)
            e = ops.rmsnorm(ops.embed(toks, embed_table, m.act_dtype), w.enorm, cfg.rms_eps)
            hn = ops.rmsnorm(hid, w.hnorm, cfg.rms_eps)
            x = ops.linear(torch.cat([e, hn], dim=-1), w.eh_proj)
            slots = torch.tensor([self.blocks[s.seq_id][(p + it) // 16] * 16 + (p + it) % 16
                                  for s, p in zip(ready, pos0)], **i32)
            meta = BatchMeta(toks, pos, slots, torch.arange(B + 1, **i32),
                             torch.tensor([p + it + 1 for p in pos0], **i32), bt, torch.arange(B, **i32), 1,
                             max(pos0) + it + 1, B)
            # the MTP layer only holds KV from its first drafted position on: mask earlier ones by
            # treating them as outside a sliding window
            saved = m.w.layers, m.w.first_layer
            m.w.layers = [w.layer]
            try:
                win = cfg.sliding_window
                cfg.sliding_window = max(1, min((p + it + 1) - self.start[s.seq_id] for s, p in zip(ready, pos0)))
                h, res = m.run_layers(x, None, meta, self.kv)
            finally:
                cfg.sliding_window = win
                m.w.layers, m.w.first_layer = saved
            xn, hsum = ops.add_rmsnorm(h, res, w.shared_head_norm, cfg.rms_eps)
            logits = ops.linear(xn, head).float()
            if m.w.tp_size > 1 and logits.shape[-1] != cfg.vocab_size:
                logits = m.comm.all_gather_cat(logits, dim=-1)
            toks = ops.argmax(logits)
            hid = hsum
            for i, s in enumerate(ready):
                drafts[s.seq_id].append(int(toks[i]))
        return drafts


class SpecDecoder:
    def __init__(self, proposer, k: int):
        if not 1 <= k <= MAX_DRAFT_TOKENS_PER_STEP:
            raise ValueError(f"draft tokens per step must be in [1, {MAX_DRAFT_TOKENS_PER_STEP}]")
        self.proposer = proposer
        self.k = k
        self.stats = SpecStats()

    def update_health(self, accepted: int, proposed: int) -> None:
        st = self.stats
        st.proposed += proposed
        st.accepted += accepted
        st.zero_rounds = st.zero_rounds + 1 if (proposed and accepted == 0) else 0
        if st.zero_rounds >= 2 * 8 or (st.proposed >= 4 * self.k * 8 and st.acceptance_rate < 0.2 * 0.25):
            # far below any useful acceptance: stop paying for drafts
            st.disabled = True

    def before_schedule(self, llm) -> None:
        if self.stats.disabled:
            return
        seqs = [s for s in llm.scheduler.running if s.remaining_prefill == 0 and s.output and s.params.is_greedy
                and s.params.max_tokens - len(s.output) > self.k + 1
                and s.num_tokens + self.k + 1 < llm.config.max_model_len]
        if not seqs:
            return
        drafts = self.proposer.propose(seqs)
        for s in seqs:
            d = drafts.get(s.seq_id) or []
            s.draft_tokens = d[: self.k]

    def after_forward(self, llm, out: SchedulerOutput, tokens: Dict[int, List[int]]) -> Dict[int, List[int]]:
        """Turn the target's per-row argmax into the accepted token list per sequence."""
        self.stats.target_forwards += 1
        acc_total = prop_total = 0
        for ss in out.scheduled:
            s = ss.seq
            if ss.is_prefill or ss.num_tokens == 1 or s.seq_id not in tokens:
                if s.seq_id in tokens:
                    self.stats.emitted += len(tokens[s.seq_id])
                continue
            drafts = list(s.draft_tokens)
            emitted = verify_greedy(drafts, tokens[s.seq_id])
            tokens[s.seq_id] = emitted
            acc_total += len(emitted) - 1
            prop_total += len(drafts)
            self.stats.emitted += len(emitted)
            self.proposer.rollback(s, s.num_tokens + len(emitted) - 1)
        if prop_total:
            self.update_health(acc_total, prop_total)
        observe = getattr(self.proposer, "observe_hidden", None)
        hid = getattr(llm.model, "last_hidden", None)
        if observe is not None and hid is not None:
            # hidden state at the position of the last accepted token: the MTP head's next input
            for ss, r0, k in getattr(llm.runner, "last_rows", []):
                n = len(tokens.get(ss.seq.seq_id, []))
                if n and r0 + n - 1 < hid.shape[0]:
                    observe(ss.seq, hid[r0 + n - 1].detach().clone())
        return tokens

    def on_finished(self, seq: Sequence) -> None:
        self.proposer.release(seq)


def attach_speculation(llm, draft_model_path: Optional[str], k: int = 4, use_mtp: bool = False, device=None) -> SpecDecoder:
    """Enable speculative decoding on an engine: a draft GGUF if given, else the model's MTP head."""
    c = llm.config
    if draft_model_path:
        from ..formats.gguf import load_gguf
        from ..models.config import config_from_gguf
        from ..models.weights import load_weights

        g = load_gguf(draft_model_path)
        dcfg = config_from_gguf(g)
        if dcfg.vocab_size != llm.cfg.vocab_size:
            raise ValueError(f"draft vocabulary {dcfg.vocab_size} != target vocabulary {llm.cfg.vocab_size}")
        act = torch.bfloat16 if llm.device.type == "cuda" else torch.float32
        dw = load_weights(g, dcfg, llm.device, act)
        prop = DraftModelProposer(dw, k, c.max_num_seqs, c.max_model_len)
    elif use_mtp and llm.weights.mtp:
        prop = MtpProposer(llm.model, k, c.max_num_seqs, c.max_model_len)
    else:
        raise ValueError("speculation needs --draft-model or a model with nextn (MTP) layers")
    llm.spec = SpecDecoder(prop, k)
    return llm.spec
