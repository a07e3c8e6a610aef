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
from .sampler import GREEDY, SamplingParams, probs_from_logits, speculative_accept
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

    def __init__(self, draft_weights, k: int, max_seqs: int, max_model_len: int, num_blocks: int = 0, comm=None,
                 kv_dtype: Optional[str] = None):
        from ..models.transformer import Transformer

        self.k = k
        self.model = Transformer(draft_weights, comm)
        dev = self.model.device
        cfg = draft_weights.cfg
        page = 16
        nblocks = num_blocks or max_seqs * ((max_model_len + page - 1) // page + 1)
        kvd = kv_dtype or ("bf16" if dev.type == "cuda" else "f32")
        self.kv = self.model.new_cache(nblocks, page, kvd)
        self.pool = make_block_pool(nblocks, page, enable_prefix_cache=False)
        self.runner = ModelRunner(self.model, self.kv, max(2048, max_seqs * (k + 2)), max_seqs, max_model_len, False)
        self.shadow: Dict[int, Sequence] = {}
        self.computed: Dict[int, int] = {}
        self.draft_logits: Dict[int, torch.Tensor] = {}  # seq_id -> [k, V] fp32 logits behind the sampled drafts

    def _shadow(self, seq: Sequence) -> Sequence:
        sh = self.shadow.get(seq.seq_id)
        if sh is None:
            p = seq.params
            # a sampled request drafts by sampling from the draft model at the request's temperature (the acceptance
            # rule needs tokens drawn from the very distribution q it divides by); its own stream of uniforms
            sp = GREEDY if p.is_greedy else SamplingParams(temperature=p.temperature, max_tokens=1 << 30, ignore_eos=True,
                                                           seed=None if p.seed is None else p.seed + 7919, tie=p.tie)
            sh = Sequence([], sp)
            self.shadow[seq.seq_id] = sh
            self.computed[seq.seq_id] = 0
        return sh

    def release(self, seq: Sequence) -> None:
        sh = self.shadow.pop(seq.seq_id, None)
        self.computed.pop(seq.seq_id, None)
        self.draft_logits.pop(seq.seq_id, None)
        if sh is not None:
            self.pool.release_all(sh.blocks)

    def _ensure(self, sh: Sequence, n_tokens: int) -> None:
        need = (n_tokens + self.pool.page_size - 1) // self.pool.page_size
        while len(sh.blocks) < need:
            sh.blocks.append(self.pool.allocate())

    def propose(self, seqs: List[Sequence]) -> Dict[int, List[int]]:
        drafts: Dict[int, List[int]] = {s.seq_id: [] for s in seqs}
        # catch-up: everything the draft has not seen yet, including the last sampled token.  A whole prompt can be
        # pending (first round after the target's prefill), so what does not fit into one batch of the draft's runner
        # next to the other sequences is fed ahead in unsampled chunks.
        cap = self.runner.buf.max_tokens
        done_of = {}
        for s in seqs:
            sh = self._shadow(s)
            sh.prompt = s.all_tokens
            done_of[s.seq_id] = min(self.computed[s.seq_id], len(sh.prompt) - 1)
            self._ensure(sh, len(sh.prompt) + self.k)
        while sum(len(self.shadow[s.seq_id].prompt) - done_of[s.seq_id] for s in seqs) > cap:
            budget, batch = cap, []
            for s in seqs:
                sh = self.shadow[s.seq_id]
                n = min(len(sh.prompt) - done_of[s.seq_id] - 1, budget)  # the last pending token belongs to the sampled pass
                if n > 0:
                    batch.append(ScheduledSeq(sh, done_of[s.seq_id], n, True, False))
                    done_of[s.seq_id] += n
                    budget -= n
            if not batch:
                break
            self.runner.execute(SchedulerOutput(batch))
        sched = [ScheduledSeq(self.shadow[s.seq_id], done_of[s.seq_id], len(self.shadow[s.seq_id].prompt) - done_of[s.seq_id], True,
                              True) for s in seqs]
        sampled = [s for s in seqs if not s.params.is_greedy]
        rows_of: Dict[int, List[torch.Tensor]] = {s.seq_id: [] for s in sampled}
        keep, self.runner.keep_logits = self.runner.keep_logits, bool(sampled)
        try:
            for it in range(self.k):
                res = self.runner.execute(SchedulerOutput(list(sched)))
                if sampled:
                    row_of = {ss.seq.seq_id: r0 + n - 1 for ss, r0, n in self.runner.last_rows}
                sched = []
                for s in seqs:
                    sh = self.shadow[s.seq_id]
                    t = res.tokens[sh.seq_id][0]
                    drafts[s.seq_id].append(t)
                    if s.seq_id in rows_of:
                        rows_of[s.seq_id].append(res.logits[row_of[sh.seq_id]].float())
                    sh.prompt = sh.prompt + [t]
                    if it + 1 < self.k:
                        sched.append(ScheduledSeq(sh, len(sh.prompt) - 1, 1, True, True))
        finally:
            self.runner.keep_logits = keep
        for sid, rows in rows_of.items():
            self.draft_logits[sid] = torch.stack(rows)
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
        self.kv = KVCache(KVCacheSpec(1, target_model.n_kv_local, target_model.kv_head_dim, page, kvd), nblocks, dev)
        self.pool = make_block_pool(nblocks, page, enable_prefix_cache=False)
        self.blocks: Dict[int, List[int]] = {}
        self.start: Dict[int, int] = {}
        self.hidden: Dict[int, torch.Tensor] = {}  # last verified hidden state per sequence
        self.max_blocks = (max_model_len + page - 1) // page
        self.draft_logits: Dict[int, torch.Tensor] = {}  # seq_id -> [k, V] fp32 logits behind the sampled drafts
        self._rng: Dict[int, object] = {}

    def observe_hidden(self, seq: Sequence, h: torch.Tensor) -> None:
        self.hidden[seq.seq_id] = h

    def release(self, seq: Sequence) -> None:
        self.pool.release_all(self.blocks.pop(seq.seq_id, []))
        self.hidden.pop(seq.seq_id, None)
        self.start.pop(seq.seq_id, None)
        self.draft_logits.pop(seq.seq_id, None)
        self._rng.pop(seq.seq_id, None)

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
                win, pat = cfg.sliding_window, cfg.sliding_window_pattern
                cfg.sliding_window = max(1, min((p + it + 1) - self.start[s.seq_id] for s, p in zip(ready, pos0)))
                cfg.sliding_window_pattern = 0
                h, res = m.run_layers(x, None, meta, self.kv)
            finally:
                cfg.sliding_window, cfg.sliding_window_pattern = win, pat
                m.w.layers, m.w.first_layer = saved
            xn, hsum = ops.add_rmsnorm(h, res, w.shared_head_norm, cfg.rms_eps)
            logits = ops.linear(xn, head).float()
            if m.w.tp_size > 1 and logits.shape[-1] != cfg.vocab_size:
                logits = m.comm.all_gather_cat(logits, dim=-1)
            temps = [0.0 if s.params.is_greedy else float(s.params.temperature) for s in ready]
            if any(t > 0 for t in temps):
                # sampled requests draft by sampling at their own temperature; the logits are kept for the acceptance rule
                from . import device_sampler
                from .sampler import RequestRng

                f32 = dict(dtype=torch.float32, device=dev)
                rnd = [self._rng.setdefault(s.seq_id, RequestRng(None if s.params.seed is None else s.params.seed + 104729)).next()
                       if t > 0 else 0.0 for s, t in zip(ready, temps)]
                toks = device_sampler.sample(logits, torch.tensor(temps, **f32), torch.zeros(B, **i32), torch.ones(B, **f32),
                                             torch.zeros(B, **f32), torch.tensor(rnd, **f32))
                for i, s in enumerate(ready):
                    if temps[i] > 0:
                        prev = self.draft_logits.get(s.seq_id) if it > 0 else None
                        row = logits[i : i + 1].float()
                        self.draft_logits[s.seq_id] = row if prev is None else torch.cat([prev, row])
            else:
                toks = ops.argmax(logits)
            toks = toks.to(torch.int32)
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
        self.needs_logits = False  # this step verifies sampled drafts: the runner must hand back the target logits

    def update_health(self, accepted: int, proposed: int) -> None:
        st = self.stats
        st.proposed += proposed
        st.accepted += accepted
        st.zero_rounds = st.zero_rounds + 1 if (proposed and accepted == 0) else 0
        if st.zero_rounds >= 2 * 8 or (st.proposed >= 4 * self.k * 8 and st.acceptance_rate < 0.2 * 0.25):
            # far below any useful acceptance: stop paying for drafts
            st.disabled = True

    @staticmethod
    def drafts_for(p: SamplingParams) -> bool:
        """Greedy requests, and sampled ones whose distribution is the plain softmax at a temperature (the acceptance
        rule is exact for those; filters, penalties, Mirostat and grammars are drawn without drafts)."""
        return p.is_greedy or (p.temperature > 0 and not p.has_filters and not p.needs_host_sampler)

    def before_schedule(self, llm) -> None:
        self.needs_logits = False
        if self.stats.disabled:
            return
        seqs = [s for s in llm.scheduler.running if s.remaining_prefill == 0 and s.output and self.drafts_for(s.params)
                and s.params.max_tokens - len(s.output) > self.k + 1
                and s.num_tokens + self.k + 1 < llm.config.max_model_len]
        if not seqs:
            return
        drafts = self.proposer.propose(seqs)
        logits_of = getattr(self.proposer, "draft_logits", {})
        for s in seqs:
            d = drafts.get(s.seq_id) or []
            if not s.params.is_greedy and (s.seq_id not in logits_of or logits_of[s.seq_id].shape[0] < len(d[: self.k])):
                d = []  # a sampled draft without its distribution cannot be verified
            s.draft_tokens = d[: self.k]
            if s.draft_tokens and not s.params.is_greedy:
                self.needs_logits = True

    def _verify_sampled(self, llm, out: SchedulerOutput, logits: torch.Tensor) -> Dict[int, List[int]]:
        """min(1, p/q) acceptance with residual resampling for the sampled sequences of this step: one kernel launch
        on the GPU, the host statement of the same rule on CPU."""
        rows = {ss.seq.seq_id: (r0, n) for ss, r0, n in getattr(llm.runner, "last_rows", [])}
        todo = [ss.seq for ss in out.scheduled
                if not ss.is_prefill and ss.num_tokens > 1 and not ss.seq.params.is_greedy and ss.seq.seq_id in rows]
        if not todo:
            return {}
        K = self.k
        dl = self.proposer.draft_logits
        result: Dict[int, List[int]] = {}
        uni = [[s.rng.next() for _ in range(2 * K + 1)] for s in todo]
        if logits.is_cuda:
            from ..ops import cuda as opcuda

            dev = logits.device
            i32, f32 = dict(dtype=torch.int32, device=dev), dict(dtype=torch.float32, device=dev)
            V = logits.shape[1]
            dlog = torch.zeros(len(todo) * K, V, **f32)
            dtok = torch.zeros(len(todo), K, **i32)
            for i, s in enumerate(todo):
                n = len(s.draft_tokens)
                dlog[i * K : i * K + n] = dl[s.seq_id][:n]
                dtok[i, :n] = torch.tensor(s.draft_tokens, **i32)
            toks, cnt = opcuda.spec_verify(logits.float().contiguous(), dlog, dtok,
                                           torch.tensor([rows[s.seq_id][0] for s in todo], **i32),
                                           torch.tensor([len(s.draft_tokens) for s in todo], **i32),
                                           torch.tensor([s.params.temperature for s in todo], **f32),
                                           torch.tensor(uni, **f32), K, todo[0].params.tie)
            toks, cnt = toks.cpu().tolist(), cnt.cpu().tolist()
            for i, s in enumerate(todo):
                result[s.seq_id] = toks[i][: cnt[i]]
        else:
            lg = logits.float().numpy()
            for s, u in zip(todo, uni):
                r0, n = rows[s.seq_id]
                q = [probs_from_logits(dl[s.seq_id][i].numpy(), s.params.temperature) for i in range(len(s.draft_tokens))]
                # the bonus token is an inverse-CDF draw in index order from row K, like the kernel's
                emitted, _ = speculative_accept(s.draft_tokens, q, lg[r0 : r0 + n], s.params, u)
                result[s.seq_id] = emitted
        return result

    def after_forward(self, llm, out: SchedulerOutput, tokens: Dict[int, List[int]],
                      logits: Optional[torch.Tensor] = None) -> Dict[int, List[int]]:
        """Turn the target's rows into the accepted token list per sequence: exact match for greedy sequences (from the
        per-row argmax), the rejection-sampling rule for sampled ones (from the rows' logits)."""
        self.stats.target_forwards += 1
        acc_total = prop_total = 0
        sampled = self._verify_sampled(llm, out, logits) if (self.needs_logits and logits is not None) else {}
        for ss in out.scheduled:
            s = ss.seq
            if ss.is_prefill or ss.num_tokens == 1 or s.seq_id not in tokens:
                if s.seq_id in tokens:
                    self.stats.emitted += len(tokens[s.seq_id])
                continue
            drafts = list(s.draft_tokens)
            emitted = sampled[s.seq_id] if s.seq_id in sampled else verify_greedy(drafts, tokens[s.seq_id])
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
        observe_f = getattr(self.proposer, "observe_features", None)
        feats = getattr(llm.model, "last_features", None)
        if observe_f is not None and feats is not None:
            # the capture layers' hidden states at the same position: the context of a hidden-conditioned draft
            for ss, r0, k in getattr(llm.runner, "last_rows", []):
                n = len(tokens.get(ss.seq.seq_id, []))
                if n and r0 + n - 1 < feats.shape[0]:
                    observe_f(ss.seq, feats[r0 + n - 1].detach().clone())
        return tokens

    def on_finished(self, seq: Sequence) -> None:
        self.proposer.release(seq)


def attach_speculation(llm, draft_model_path: Optional[str], k: int = 4, use_mtp: bool = False, device=None,
                       quantspec: bool = False) -> SpecDecoder:
    """Enable speculative decoding on an engine: a draft GGUF if given, else the model's MTP head; with ``quantspec`` the
    model drafts for itself over a 4-bit copy of its KV cache (the reference's ``--quantspec``,
    ``SpeculativeGenerationConfig::quantspec_draft_kv``): the draft reads a quarter of the cache bytes, which is what a
    long-context decode step is bound by, and the target's verification keeps the output exact."""
    c = llm.config
    if quantspec and not draft_model_path:
        if llm.cfg.is_ssm or llm.cfg.is_mla:
            raise ValueError("self-speculation over a 4-bit cache needs ordinary attention layers")
        if llm.model.kv_head_dim % 32:
            raise ValueError("a 4-bit cache needs a head width that is a multiple of 32")
        prop = DraftModelProposer(llm.weights, k, c.max_num_seqs, c.max_model_len, comm=llm.model.comm, kv_dtype="q4")
        llm.spec = SpecDecoder(prop, k)
        return llm.spec
    if llm.cfg.is_ssm:
        raise ValueError("speculative decoding needs a cache that can be rolled back: not available for state-space models")
    if draft_model_path:
        from ..formats.gguf import load_gguf
        from ..models.config import config_from_gguf
        from ..models.weights import load_weights

        g = load_gguf(draft_model_path)
        if "fc.weight" in g.tensors and "blk.0.attn_norm_2.weight" in g.tensors:
            # an EAGLE-3 head: one block fed with [embedding ; fused target features]
            from .feature_draft import Eagle3Proposer, load_eagle3

            if llm.config.tp_size > 1 or llm.config.pp_size > 1:
                raise ValueError("hidden-conditioned drafts run with single-rank engines")
            act = torch.bfloat16 if llm.device.type == "cuda" else torch.float32
            ew = load_eagle3(draft_model_path, llm.device, act, llm.cfg.n_layers, llm.cfg.hidden_size)
            llm.spec = SpecDecoder(Eagle3Proposer(ew, llm.model, k, c.max_num_seqs, c.max_model_len), k)
            return llm.spec
        if any(n in g.tensors for n in ("fc.weight", "dflash_fc.weight", "model.fc.weight")):
            # a hidden-conditioned draft (DFlash-style): it reads the target's hidden states besides the tokens
            from .feature_draft import FeatureDraftProposer, load_feature_draft

            if llm.config.tp_size > 1 or llm.config.pp_size > 1:
                raise ValueError("hidden-conditioned drafts run with single-rank engines")
            act = torch.bfloat16 if llm.device.type == "cuda" else torch.float32
            fw = load_feature_draft(draft_model_path, llm.device, act, llm.cfg.n_layers)
            llm.spec = SpecDecoder(FeatureDraftProposer(fw, llm.model, k, c.max_num_seqs, c.max_model_len), k)
            return llm.spec
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
