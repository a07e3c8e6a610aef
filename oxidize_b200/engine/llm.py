"""``LLM``: the public engine object — load (or synthesise) a model, then ``generate`` or
drive ``add_request`` / ``step`` yourself.

It plays the role of the reference's ``ContinuousBatchEngine::{submit, step, cancel}``
(``oxidize-core/src/model/inference/batch_engine.rs:128,180,157``) and of
``GenerationStream`` (``model/generation.rs:1057``) for one-shot use, on top of a real paged
KV pool.  Under tensor parallelism every rank constructs the same ``LLM`` and calls the same
methods in lock step (SPMD): scheduling is deterministic and the sampled tokens are identical
on all ranks, so no control-plane broadcast sits on the step path.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence as Seq, Union

import torch

from ..formats.gguf import GGUFFile, load_gguf
from ..models.config import ModelConfig, config_from_gguf
from ..models.transformer import Transformer
from ..models.weights import ModelWeights, load_weights
from ..utils import profiler as _profiler
from .kv_pool import BlockPool, KVCache, KVCacheSpec, make_block_pool
from .runner import ModelRunner, StepResult
from .sampler import SamplingParams
from .scheduler import ScheduledSeq, Scheduler, SchedulerConfig, SchedulerOutput, Sequence


@dataclass
class EngineConfig:
    """Typed engine configuration (CLI flags and YAML map onto these fields)."""

    kv_cache_dtype: str = "auto"  # auto | f32 | f16 | bf16 | q8 | q4
    kv_page_size: int = 16
    num_kv_blocks: int = 0  # 0 = size from gpu_memory_utilization / max_model_len
    gpu_memory_utilization: float = 0.90
    max_model_len: int = 4096
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048  # tokens per step (prefill chunks + decode rows); 0 = pick by tile waves (autotune)
    prefill_chunk_size: int = 512
    policy: str = "fcfs"
    enable_prefix_cache: bool = True
    cuda_graphs: bool = True
    tp_size: int = 1
    ep_size: int = 0  # experts partitioned over this many ranks; 0 = tp_size, 1 = replicated on every rank
    pp_size: int = 1
    fused_comm: bool = True
    # dense bf16 layers: RMSNorm folded into the GEMM epilogues around it (GPU only).  Two launches fewer per layer, but the
    # epilogues it lengthens sit on the critical path of the fused all-reduce: measured 2.6 % slower at 8 GPUs, even on one.
    fold_norms: bool = False
    # Steady-state greedy decode: launch step k+1 (input ids taken from step k's kernel on the device) before
    # reading step k's tokens, so that the host's scheduling and batch building overlap the GPU's work.
    async_decode: bool = True
    fuse_qkv_rope: bool = True  # RoPE + KV write as the qkv GEMM's epilogue where the shapes allow
    fuse_swiglu: bool = True  # SiLU(gate) * up as the gate_up GEMM's epilogue for dense bf16 FFNs
    kernel_options: Optional[object] = None  # ops.cuda.KernelOptions; None = the library's defaults
    eos_token_id: Optional[int] = None
    # > 0: keep only this many decoder layers loaded, streaming the others from the file mapping as the forward pass
    # reaches them (for checkpoints larger than the memory left beside the KV cache)
    resident_layers: int = 0
    # "Q8_0" / "Q4_0": float weight matrices are re-encoded in that block format while loading (the reference's
    # --turboquant: block-wise int8 / int4 weights with per-block scales); "" = keep the checkpoint's encodings
    weight_transcode: str = ""


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: List[int]
    token_ids: List[int]
    finished: bool
    finish_reason: Optional[str] = None
    ttft: Optional[float] = None
    latency: Optional[float] = None
    num_cached_tokens: int = 0
    text: Optional[str] = None


class LLM:
    def __init__(self, weights: ModelWeights, config: Optional[EngineConfig] = None, comm=None, tokenizer=None, pipe=None):
        self.config = config or EngineConfig()
        c = self.config
        self.pipe = pipe  # parallel.pp.StageIO: this process holds one pipeline stage (all stages run this same engine)
        if (pipe is not None) != (c.pp_size > 1) or (pipe is not None and pipe.world != c.pp_size):
            raise ValueError("pp_size > 1 needs the stage's StageIO (parallel.pp.make_pipeline_groups) and vice versa")
        self.weights = weights
        self.cfg: ModelConfig = weights.cfg
        if c.max_num_batched_tokens <= 0:
            from ..utils.autotune import prefill_token_budget

            c.max_num_batched_tokens = max(prefill_token_budget(self.cfg, max(c.tp_size, 1)), c.max_num_seqs)
        if weights.embed.device.type == "cuda" and c.kernel_options is not None:
            from ..ops import cuda as _opcuda

            _opcuda.configure(c.kernel_options)
        self.model = Transformer(weights, comm, fold_norms=c.fold_norms, fuse_qkv_rope=c.fuse_qkv_rope,
                                 fuse_swiglu=c.fuse_swiglu, pipe=pipe, max_context=c.max_model_len)
        self.device = self.model.device
        self.tokenizer = tokenizer
        kv_dtype = c.kv_cache_dtype
        if kv_dtype == "auto":
            kv_dtype = "bf16" if self.device.type == "cuda" else "f32"
        spec = KVCacheSpec(max(1, self.model.n_kv_layers), self.model.n_kv_local, self.model.kv_head_dim, c.kv_page_size, kv_dtype)
        # (a hybrid model's convolution layers keep one hidden-sized row per token as well)
        conv_bytes = self.model.n_conv_layers * c.kv_page_size * self.cfg.hidden_size * (2 if self.device.type == "cuda" else 4)
        nblocks = c.num_kv_blocks or self._auto_blocks(spec, conv_bytes)
        self.kv = self.model.new_cache(nblocks, c.kv_page_size, kv_dtype)
        # a recurrent state cannot be rebuilt from shared pages: state-space models run without the prefix cache
        prefix_cache = c.enable_prefix_cache and not self.cfg.is_ssm
        self.pool = make_block_pool(nblocks, c.kv_page_size, prefix_cache)
        # a window that applies to every layer lets the scheduler hand pages back as they fall out of it
        uniform_window = self.cfg.sliding_window if (self.cfg.sliding_window > 0 and self.cfg.sliding_window_pattern == 0) else 0
        self.scheduler = Scheduler(SchedulerConfig(c.max_num_batched_tokens, c.prefill_chunk_size, c.max_num_seqs,
                                                   c.policy, prefix_cache, c.max_model_len, uniform_window), self.pool)
        self.runner = ModelRunner(self.model, self.kv, max(c.max_num_batched_tokens, c.max_num_seqs), c.max_num_seqs,
                                  c.max_model_len, c.cuda_graphs and not _profiler.PROFILE and not _profiler.TRACE_FWD
                                  and isinstance(weights.layers, list)  # a captured graph would pin evicted layers' addresses
                                  and not self.cfg.is_mla  # latent attention's device step sizes its gather on the host
                                  and not self.model.n_conv_layers  # so does the convolution layers' row gather
                                  and not self.cfg.is_ssm)  # the recurrence runs from the host, token by token
        self.eos_token_id = c.eos_token_id
        if self.eos_token_id is None and tokenizer is not None:
            self.eos_token_id = tokenizer.special_tokens.eos
        self._seqs: Dict[str, Sequence] = {}
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "h2d_bytes": 0, "d2h_bytes": 0}

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_gguf(cls, path: Union[str, GGUFFile], config: Optional[EngineConfig] = None, device=None, comm=None,
                  tp_rank: int = 0, ep_rank: int = 0, rope_pairing: Optional[str] = None, pipe=None,
                  experts_per_token: int = 0) -> "LLM":
        from ..formats.tokenizer import TokenizerError, load_tokenizer_from_metadata

        config = config or EngineConfig()
        g = path if isinstance(path, GGUFFile) else load_gguf(path)
        cfg = config_from_gguf(g)
        if rope_pairing:
            cfg.rope_pairing = rope_pairing
        if experts_per_token:
            # route every token to this many experts instead of the checkpoint's count (the C port's --experts-per-tok)
            if not cfg.is_moe or not 1 <= experts_per_token <= cfg.n_experts:
                raise ValueError(f"experts_per_token must be between 1 and the model's {cfg.n_experts} experts")
            cfg.n_experts_used = experts_per_token
        device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        act = torch.bfloat16 if device.type == "cuda" else torch.float32
        ep_size = config.ep_size or config.tp_size
        if ep_size == config.tp_size and ep_rank == 0:
            ep_rank = tp_rank  # the expert partition follows the tensor-parallel rank
        if ep_size == 1:
            ep_rank = 0
        layer_range = None
        if config.pp_size > 1:
            from ..parallel.pp import split_layers

            if pipe is None:
                raise ValueError("pp_size > 1 needs the stage's StageIO")
            layer_range = split_layers(cfg.n_layers, config.pp_size)[pipe.rank]
        w = load_weights(g, cfg, device, act, tp_rank, config.tp_size, ep_rank, ep_size, layer_range=layer_range,
                         resident_layers=config.resident_layers, transcode=config.weight_transcode)
        try:
            tok = load_tokenizer_from_metadata(g.metadata)
        except TokenizerError:
            tok = None
        llm = cls(w, config, comm, tok, pipe)
        from ..formats.tokenizer import chat_template_from_metadata

        llm.chat_template = chat_template_from_metadata(g.metadata)  # None when the file carries none
        return llm

    def _auto_blocks(self, spec: KVCacheSpec, extra_bytes_per_block: int = 0) -> int:
        c = self.config
        want = c.max_num_seqs * ((c.max_model_len + spec.page_size - 1) // spec.page_size + 1)
        if self.device.type != "cuda":
            return max(16, min(want, 4096))
        free, total = torch.cuda.mem_get_info(self.device)
        budget = int(free - (1.0 - c.gpu_memory_utilization) * total)
        fit = max(16, budget // max(spec.bytes_per_block() + extra_bytes_per_block, 1))
        return int(min(want, fit))

    # ------------------------------------------------------------------ request API
    def add_request(self, prompt: Union[str, Seq[int]], params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, input_embeds: Optional[torch.Tensor] = None,
                    embed_positions: Optional[Seq[int]] = None) -> str:
        """Queue a request.  ``input_embeds`` [n, hidden] with ``embed_positions`` (n ascending prompt positions) replaces
        the token embeddings at those positions: image tokens of a multimodal prompt (see ``vision.MultimodalPrompt``)."""
        params = params or SamplingParams()
        params.validate()
        if isinstance(prompt, tuple):  # (token ids, embedding positions, embedding rows), as vision.MultimodalPrompt builds
            prompt, embed_positions, input_embeds = prompt
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("text prompt given but the model has no tokenizer; pass token ids")
            ids = self.tokenizer.encode_with_special_tokens(prompt)
        else:
            ids = [int(t) for t in prompt]
        bad = [t for t in ids if not 0 <= t < self.cfg.vocab_size]
        if bad:
            raise ValueError(f"token id {bad[0]} outside vocabulary of {self.cfg.vocab_size}")
        seq = Sequence(ids, params, request_id, arrival=time.perf_counter())
        if input_embeds is not None:
            pos = [int(p) for p in (embed_positions or [])]
            if input_embeds.ndim != 2 or input_embeds.shape[0] != len(pos) or input_embeds.shape[1] != self.cfg.hidden_size:
                raise ValueError(f"input_embeds must be [len(embed_positions), {self.cfg.hidden_size}]")
            if any(b <= a for a, b in zip(pos, pos[1:])) or (pos and not 0 <= pos[0] <= pos[-1] < len(ids)):
                raise ValueError("embed_positions must be ascending positions inside the prompt")
            if getattr(self, "spec", None) is not None:
                raise ValueError("requests with input embeddings are not drafted for: run them on an engine without speculation")
            seq.input_embeds, seq.embed_positions = input_embeds.to(self.device), pos
        self.scheduler.add(seq)
        self._seqs[seq.request_id] = seq
        return seq.request_id

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort(request_id)

    @property
    def has_unfinished(self) -> bool:
        return self.scheduler.has_work or getattr(self, "_inflight", None) is not None

    def step(self) -> List[RequestOutput]:
        """One engine iteration (see ``_step``); with ``KernelOptions.checked`` the scratch buffers' canary bands are
        verified after it."""
        out = self._step()
        if self.device.type == "cuda":
            from ..ops import cuda as _opcuda

            if _opcuda.checked:
                _opcuda.verify_guards()
        return out

    def _step(self) -> List[RequestOutput]:
        """One engine iteration: schedule → forward → sample → postprocess.

        In the steady state of greedy decoding the engine keeps one step in flight: before it waits for the tokens
        of step k it has already launched step k+1 for the same sequences, whose input ids never leave the device
        (the role of the reference's device-resident ``{token, pos, step}`` state,
        ``oxidize-c/src/backends/cuda_fast.cu:58-63,495``).  A call then returns the results of the step launched
        one call earlier.  A sequence that turns out to have ended on step k (EOS, stop sequence, abort) has one
        surplus row in step k+1, whose token is dropped."""
        spec = getattr(self, "spec", None)
        inflight = getattr(self, "_inflight", None)
        if inflight is not None:
            out, pending = inflight
            self._inflight = None
        else:
            if spec is not None:
                spec.before_schedule(self)
            out = self.scheduler.schedule()
            if out.is_empty:
                if self.scheduler.has_work and not out.preempted:
                    raise RuntimeError("scheduler made no progress: KV pool too small for the waiting request")
                return []
            if self.pipe is not None:
                return self._step_pipelined(out)
            pending = self.runner.launch(out, needs_host_logits=bool(spec is not None and spec.needs_logits))
        if self.config.async_decode and spec is None and self.pipe is None:
            nxt = self._schedule_ahead(out, pending)
            if nxt is not None:
                self._inflight = (nxt, self.runner.launch(nxt, tokens_on_device=True))
        was_finished = [ss.seq.is_finished for ss in out.scheduled]
        res = self.runner.collect(pending)
        if spec is not None:
            res.tokens = spec.after_forward(self, out, res.tokens, res.logits)
        now = time.perf_counter()
        done = self.scheduler.postprocess(out, res.tokens, self.eos_token_id, now)
        if spec is not None:
            for s in done:
                spec.on_finished(s)
        st = self.stats
        st["steps"] += 1
        st["prefill_tokens"] += out.num_prefill_tokens
        st["decode_tokens"] += out.num_decode_tokens
        st["h2d_bytes"] += res.h2d_bytes
        st["d2h_bytes"] += res.d2h_bytes
        self.last_step = (out, res)
        outs = []
        for ss, gone in zip(out.scheduled, was_finished):
            if gone:
                continue  # ended on the step before: this row ran ahead for nothing
            if ss.sample or ss.seq.is_finished:
                outs.append(self._output(ss.seq))
        return outs

    def _step_pipelined(self, out: SchedulerOutput) -> List[RequestOutput]:
        """One step on a pipeline stage.  The scheduled sequences are cut into as many micro-batches as there are
        stages (at most two are in flight on the staging buffers); every stage pushes all of them through its layers
        before it waits for the first one's tokens, so stage i works on micro-batch j+1 while stage i+1 works on j
        (the reference's pipeline streams positions the same way, ``oxidize-cli/src/pipeline.rs:17-21,302``)."""
        n = len(out.scheduled)
        parts = min(2, self.config.pp_size, n)
        cuts = [n * i // parts for i in range(parts + 1)]
        subs = []
        for i in range(parts):
            sch = out.scheduled[cuts[i] : cuts[i + 1]]
            so = SchedulerOutput(sch, sum(s.num_tokens for s in sch if s.is_prefill),
                                 sum(s.num_tokens for s in sch if not s.is_prefill), [], out.cow_copies if i == 0 else [])
            subs.append(so)
        pend = [self.runner.launch_forward(so) for so in subs]
        for p in pend:
            self.runner.finish(p)
        tokens: Dict[int, List[int]] = {}
        h2d = d2h = 0
        for p in pend:
            r = self.runner.collect(p)
            tokens.update(r.tokens)
            h2d += r.h2d_bytes
            d2h += r.d2h_bytes
        res = StepResult(tokens, None, h2d, d2h)
        now = time.perf_counter()
        self.scheduler.postprocess(out, res.tokens, self.eos_token_id, now)
        st = self.stats
        st["steps"] += 1
        st["prefill_tokens"] += out.num_prefill_tokens
        st["decode_tokens"] += out.num_decode_tokens
        st["h2d_bytes"] += h2d
        st["d2h_bytes"] += d2h
        self.last_step = (out, res)
        return [self._output(ss.seq) for ss in out.scheduled if ss.sample or ss.seq.is_finished]

    def close(self) -> None:
        """Release what must go before the process group does: the step in flight, then the captured CUDA graphs.
        A graph keeps the kernels, buffers and (on the NCCL baseline path) the communicator it captured alive;
        tearing the communicator down while a graph still refers to it blocks, so the graphs are dropped first and
        the device is idle when the caller destroys the process group."""
        try:
            self.drain()
        except Exception:
            self._inflight = None
        self.runner.graphs.clear()
        self.runner.graph_out.clear()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def drain(self) -> List[RequestOutput]:
        """Finish the step that is in flight, if any, without launching another one ahead of it."""
        if getattr(self, "_inflight", None) is None:
            return []
        keep, self.config.async_decode = self.config.async_decode, False
        try:
            return self.step()
        finally:
            self.config.async_decode = keep

    def _schedule_ahead(self, out: SchedulerOutput, pending) -> Optional[SchedulerOutput]:
        """The decode step that follows ``out`` if nothing unexpected happens, or None when the next step needs the
        scheduler proper: anything but a pure greedy graph-replayed decode step, requests waiting, a sequence about
        to reach its token limit, or a KV pool that cannot give every sequence its next slot."""
        sch = self.scheduler
        if pending is None or pending.bucket == 0 and self.device.type == "cuda":
            return None
        if pending.host_rows or pending.keep_logits or not pending.seq_ids:
            return None
        if sch.waiting or len(out.scheduled) != len(sch.running) or out.cow_copies or out.preempted:
            return None
        ps = self.pool.page_size
        nxt = SchedulerOutput([])
        max_len = self.config.max_model_len
        for ss in out.scheduled:
            seq = ss.seq
            if ss.is_prefill or ss.num_tokens != 1 or not ss.sample or seq.is_finished or seq.draft_tokens:
                return None
            p = seq.params
            if not p.is_greedy or p.needs_host_sampler:
                return None
            # after the step in flight the sequence holds one more token; the step after it must still be wanted
            produced = len(seq.output) + len(getattr(seq, "_preempted_outputs", ())) + 1
            if produced >= p.max_tokens:
                return None
            start = ss.start + 1
            if start + 1 > max_len:
                return None
            nxt.scheduled.append(ScheduledSeq(seq, start, 1, False, True))
        # every sequence needs a slot for position `start`; nothing is taken unless all of them can have one
        need = sum(1 for s2 in nxt.scheduled if (s2.start + ps) // ps > len(s2.seq.blocks))
        if need and not self.pool.can_allocate(need):
            return None
        for s2 in nxt.scheduled:
            while (s2.start + ps) // ps > len(s2.seq.blocks):
                s2.seq.blocks.append(self.pool.allocate())
        nxt.num_decode_tokens = len(nxt.scheduled)
        return nxt

    def _output(self, seq: Sequence) -> RequestOutput:
        # A running request's output references the sequence's own lists (no per-step copies of the
        # prompt and of everything generated so far); a finished one gets its own copy.
        pre = getattr(seq, "_preempted_outputs", None)
        if pre:
            gen = pre + seq.output
            prompt = seq.prompt[: len(seq.prompt) - len(pre)]
        else:
            gen = list(seq.output) if seq.is_finished else seq.output
            prompt = seq.prompt
        ro = RequestOutput(seq.request_id, prompt, gen, seq.is_finished, seq.finish_reason,
                           None if seq.first_token_time is None else seq.first_token_time - seq.arrival,
                           None if seq.finish_time is None else seq.finish_time - seq.arrival, seq.num_cached_tokens)
        if seq.is_finished:
            self._seqs.pop(seq.request_id, None)
        return ro

    def next_token_logits(self, token_lists: Seq[Seq[int]]) -> "np.ndarray":
        """Logits of the token that would follow each sequence, [n, vocab] float32 (scored as one-token
        requests through the normal scheduler, so shared prefixes are served by the prefix cache)."""
        import numpy as np

        sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
        ids = [self.add_request(list(t), sp) for t in token_lists]
        want = set(ids)
        got = {}
        keep, self.runner.keep_logits = self.runner.keep_logits, True
        try:
            while len(got) < len(ids):
                if not self.step() and not self.has_unfinished:
                    break
                _, res = self.last_step
                for ss, r0, k in self.runner.last_rows:
                    rid = ss.seq.request_id
                    if rid in want and ss.sample and res.logits is not None:
                        got[rid] = res.logits[r0 + k - 1].float().cpu().numpy()
        finally:
            self.runner.keep_logits = keep
        return np.stack([got[i] for i in ids])

    def embed(self, prompts: Iterable[Union[str, Seq[int]]], pooling: str = "mean", normalize: bool = True) -> "np.ndarray":
        """Text embeddings [n, hidden] float32: the final-norm hidden states of each prompt, pooled over its tokens
        (``mean``) or taken at its last token (``last``), L2-normalised.  Runs outside the scheduler on a cache of its own
        that lives for the call, so it neither takes blocks from nor waits for running requests; single-rank engines only
        (the other ranks of a tensor- or pipeline-parallel group would have to run the same forward)."""
        import numpy as np

        from ..models.transformer import BatchMeta

        if self.model.w.tp_size > 1 or self.pipe is not None:
            raise NotImplementedError("embeddings are served by single-rank engines")
        if pooling not in ("mean", "last"):
            raise ValueError("pooling must be 'mean' or 'last'")
        dev, m = self.device, self.model
        i32 = dict(dtype=torch.int32, device=dev)
        page = self.config.kv_page_size
        out = []
        for p in prompts:
            ids = self.tokenizer.encode(p) if isinstance(p, str) else list(p)
            if not ids:
                raise ValueError("cannot embed an empty prompt")
            ids = ids[: self.config.max_model_len]
            n = len(ids)
            nblk = (n + page - 1) // page
            kv = m.new_cache(nblk, page, self.kv.spec.dtype_name)
            pos = torch.arange(n, **i32)
            meta = BatchMeta(torch.tensor(ids, **i32), pos, pos.clone(), torch.tensor([0, n], **i32), torch.tensor([n], **i32),
                             torch.arange(nblk, **i32)[None, :], torch.arange(n, **i32), n, n, 1, logits_all=True)
            h, residual = m.run_layers(m.embed(meta.token_ids), None, meta, kv)
            from .. import ops

            m.release_state(kv)
            x = ops.add_rmsnorm(h, residual, m.w.out_norm, m.cfg.rms_eps)[0].float()
            v = x.mean(dim=0) if pooling == "mean" else x[-1]
            if normalize:
                v = v / v.norm().clamp_min(1e-12)
            out.append(v.cpu().numpy())
        return np.stack(out)

    def token_logprobs(self, tokens: Seq[int], chunk: int = 256) -> "np.ndarray":
        """log p(tokens[i] | tokens[:i]) for i = 1 .. n-1, float64 [n - 1]: one pass over the text in chunks of ``chunk`` rows
        on a cache of its own, the head applied to every row (the quantity behind perplexity; single-rank engines)."""
        import numpy as np

        from ..models.transformer import BatchMeta

        if self.model.w.tp_size > 1 or self.pipe is not None:
            raise NotImplementedError("scoring runs on single-rank engines")
        ids = [int(t) for t in tokens]
        if len(ids) < 2:
            raise ValueError("need at least two tokens to score")
        dev, m = self.device, self.model
        i32 = dict(dtype=torch.int32, device=dev)
        page = self.config.kv_page_size
        n = len(ids)
        nblk = (n + page - 1) // page
        kv = m.new_cache(nblk, page, self.kv.spec.dtype_name)
        bt = torch.arange(nblk, **i32)[None, :]
        out = np.empty(n - 1, dtype=np.float64)
        for lo in range(0, n - 1, chunk):
            hi = min(lo + chunk, n - 1)  # rows lo .. hi-1 predict tokens lo+1 .. hi
            pos = torch.arange(lo, hi, **i32)
            meta = BatchMeta(torch.tensor(ids[lo:hi], **i32), pos, pos.clone(), torch.tensor([0, hi - lo], **i32),
                             torch.tensor([hi], **i32), bt, torch.arange(hi - lo, **i32), hi - lo, hi, 1, logits_all=True)
            lp = torch.log_softmax(m.forward(meta, kv).float(), dim=-1)
            tgt = torch.tensor(ids[lo + 1 : hi + 1], dtype=torch.int64, device=dev)
            out[lo:hi] = lp.gather(1, tgt[:, None]).squeeze(1).double().cpu().numpy()
        m.release_state(kv)
        return out

    def perplexity(self, text: Union[str, Seq[int]], chunk: int = 256) -> float:
        """exp(-mean log p) of a text under the model (``max_model_len`` tokens at most)."""
        import numpy as np

        ids = self.tokenizer.encode_with_special_tokens(text) if isinstance(text, str) else list(text)
        return float(np.exp(-self.token_logprobs(ids[: self.config.max_model_len], chunk).mean()))

    def beam_search(self, prompt: Union[str, Seq[int]], beam_width: int = 4, max_tokens: int = 32,
                    length_penalty: float = 1.0):
        """Width-``beam_width`` search; returns [(generated token ids, normalised log-probability)], best first."""
        from .constrained import beam_search

        toks = self.tokenizer.encode(prompt) if isinstance(prompt, str) else list(prompt)
        return beam_search(self.next_token_logits, toks, beam_width, max_tokens, self.eos_token_id, length_penalty)

    def generate(self, prompts: Iterable[Union[str, Seq[int]]], params: Union[SamplingParams, Seq[SamplingParams], None] = None,
                 on_token: Optional[Callable[[RequestOutput], None]] = None) -> List[RequestOutput]:
        """Run a set of prompts to completion with continuous batching; results in input order."""
        prompts = list(prompts)
        if params is None or isinstance(params, SamplingParams):
            plist = [params or SamplingParams()] * len(prompts)
        else:
            plist = list(params)
        # a prompt may also be (token ids, embedding positions, embedding rows): see add_request / vision.MultimodalPrompt
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        final: Dict[str, RequestOutput] = {}
        while self.has_unfinished:
            for ro in self.step():
                if on_token is not None:
                    on_token(ro)
                if ro.finished:
                    final[ro.request_id] = ro
        outs = [final[i] for i in ids]
        if self.tokenizer is not None:
            for ro in outs:
                ro.text = self.tokenizer.decode_without_special_tokens(ro.token_ids)
        return outs
