"""Decoder-only transformer forward over a flat token batch and a paged KV cache.

One code path serves decode (1 query row per sequence), chunked prefill and speculative
verification (several rows per sequence) for Llama / Mistral / Qwen3 (per-head QK-norm)
and the MoE families Mixtral / Qwen3-MoE / DeepSeek-MoE (shared expert, sigmoid+bias
routing).  Layer semantics follow the reference's per-token layer loop
(``oxidize-core/src/model/inference/layers.rs``: attention :893+, MoE + shared expert
:1420-1475) and MoE math ``moe_ffn_forward_weights`` (``model/inference.rs:1662-1935``); the
batching, paging and sharding are this framework's own.

Tensor parallelism is Megatron-style: qkv / gate_up are column-parallel, attn_output /
ffn_down are row-parallel and end in an all-reduce supplied by ``comm`` (fused into the
GEMM kernel on the GPU path), the lm_head is vocabulary-parallel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from .. import ops
from ..utils import profiler as _profiler
from ..ops import ref as opref
from .config import ModelConfig
from .weights import LayerWeights, ModelWeights


@dataclass
class RopeState:
    inv_freq: torch.Tensor
    pairing: str
    mscale: float
    n_heads: int  # local (this rank's) head counts
    n_kv_heads: int
    head_dim: int


@dataclass
class BatchMeta:
    """Flat description of one engine step (all int32 tensors on the model's device)."""

    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T]
    slot_mapping: torch.Tensor  # [T]  block*page + offset, -1 = do not write
    query_start: torch.Tensor  # [B+1]
    seq_lens: torch.Tensor  # [B] context length including this step's rows
    block_tables: torch.Tensor  # [B, max_blocks]
    logits_indices: torch.Tensor  # [L] rows that need logits
    max_query_len: int = 1
    max_seq_len: int = 0
    num_seqs: int = 0
    # host copies for CPU-side loops (reference path); optional on the GPU path
    extra: dict = field(default_factory=dict)


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class SingleRankComm:
    """Communication facade for tp=ep=1 (every collective is the identity)."""

    rank = 0
    size = 1

    def all_reduce(self, x):
        return x

    def all_gather_cat(self, x, dim=-1):
        return x

    def linear_allreduce(self, x, w, residual=None):
        out = ops.linear(x, w)
        return out if residual is None else out + residual


class Transformer:
    def __init__(self, weights: ModelWeights, comm=None, act_dtype: Optional[torch.dtype] = None):
        self.w = weights
        self.cfg: ModelConfig = weights.cfg
        self.comm = comm or SingleRankComm()
        dev = weights.embed.device
        self.device = dev
        self.act_dtype = act_dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        cfg = self.cfg
        tp = weights.tp_size
        group = getattr(self.comm, "size", 1)
        if tp != group:
            raise ValueError(f"weights are sharded {tp}-way (tp_size) but the communication group has {group} ranks")
        if cfg.is_moe and weights.ep_size not in (1, group):
            raise ValueError(f"expert parallelism must span the whole group: ep_size={weights.ep_size}, group size={group} "
                             "(use ep_size=1 to replicate the experts)")
        if cfg.is_moe and weights.ep_size > 1 and weights.ep_rank != getattr(self.comm, "rank", 0):
            raise ValueError(f"ep_rank={weights.ep_rank} does not match this rank ({getattr(self.comm, 'rank', 0)})")
        self.n_heads_local = cfg.n_heads // tp
        self.n_kv_local = max(1, cfg.n_kv_heads // tp)
        self.rope = RopeState(
            inv_freq=opref.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta, cfg.rope_scaling, device=dev),
            pairing=cfg.rope_pairing, mscale=opref.rope_mscale(cfg.rope_scaling),
            n_heads=self.n_heads_local, n_kv_heads=self.n_kv_local, head_dim=cfg.head_dim)
        self.attn_scale = cfg.head_dim ** -0.5
        # The qkv and gate_up GEMMs run right behind the all-reduce of the previous row-parallel
        # projection (plus one small norm kernel).  With more than one rank that wait leaves HBM
        # idle, so those two GEMMs ask for the head of their weight stream into the L2 meanwhile.
        import os

        self._post_collective_prefetch_kb = 0
        if dev.type == "cuda" and getattr(self.comm, "size", 1) > 1:
            # measured at 2 and 8 GPUs: no effect on the step (10.42 vs 10.43 ms at 8), so it is off by default
            self._post_collective_prefetch_kb = int(os.environ.get("OXB_L2_PREFETCH_KB", "0"))
        # per-projection override "qkv:o:gate_up:down" in weight k-blocks per CTA (experiments)
        pf = os.environ.get("OXB_PF", "")
        self._pf = [int(v) for v in pf.split(":")] if pf and dev.type == "cuda" else None
        self._fuse_qkv_rope = dev.type == "cuda" and os.environ.get("OXB_FUSED_QKV_ROPE", "1") != "0"
        if dev.type == "cuda" and os.environ.get("OXB_FUSED_SWIGLU", "1") != "0":
            self._interleave_gate_up()

    def _interleave_gate_up(self) -> None:
        """Dense bf16 gate|up projections are re-laid out once so that SiLU(gate) * up becomes the
        epilogue of the gate_up GEMM (one kernel and one activation round trip less per layer)."""
        from ..ops import cuda as opcuda

        for lw in self.w.layers:
            w = lw.w_gate_up
            if w is None or w.swiglu_interleaved or len(w.parts) != 1 or w.bias is not None:
                continue
            p = w.parts[0]
            if p.qtype != "BF16" or p.shape[0] % 128 != 0:
                continue
            p.data = opcuda.interleave_gate_up(p.data)
            w.swiglu_interleaved = True

    # ------------------------------------------------------------------ blocks
    def _attention(self, lw: LayerWeights, layer: int, x: torch.Tensor, meta: BatchMeta, kv) -> torch.Tensor:
        cfg = self.cfg
        if self._fuse_qkv_rope and x.is_cuda and lw.wqkv.bias is None:
            from ..ops import cuda as opcuda

            if opcuda.qkv_rope_fusable(lw.wqkv.parts, kv, self.rope, lw.q_norm, lw.k_norm):
                with self._prefetch(0, self._post_collective_prefetch_kb):
                    q = opcuda.linear_qkv_rope(x, lw.wqkv.parts[0].data, meta.positions, meta.slot_mapping, kv, layer,
                                               self.rope)
                attn = ops.paged_attention(q, kv, layer, meta, self.attn_scale, cfg.sliding_window)
                with self._prefetch(1, 0):
                    return self.comm.linear_allreduce(attn.reshape(attn.shape[0], -1), lw.wo)
        qkv = self._linear_after_collective(x, lw.wqkv, 0)
        q = ops.qk_rope_kv_write(qkv, meta.positions, meta.slot_mapping, kv, layer, self.rope,
                                 lw.q_norm, lw.k_norm, cfg.rms_eps)
        attn = ops.paged_attention(q, kv, layer, meta, self.attn_scale, cfg.sliding_window)
        with self._prefetch(1, 0):
            return self.comm.linear_allreduce(attn.reshape(attn.shape[0], -1), lw.wo)

    def _prefetch(self, which: int, default_kb: int):
        from ..ops import cuda as opcuda

        kb = self._pf[which] if self._pf is not None else default_kb
        return opcuda.l2_prefetch(kb) if self.device.type == "cuda" else _NullCtx()

    def _dense_ffn(self, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        if lw.w_gate_up.swiglu_interleaved:
            from ..ops import cuda as opcuda

            with self._prefetch(2, self._post_collective_prefetch_kb):
                act = opcuda.linear_swiglu(x, lw.w_gate_up.parts[0].data)
        else:
            act = ops.silu_mul(self._linear_after_collective(x, lw.w_gate_up, 2))
        with self._prefetch(3, 0):
            return self.comm.linear_allreduce(act, lw.w_down)

    def _linear_after_collective(self, x: torch.Tensor, w, which: int) -> torch.Tensor:
        with self._prefetch(which, self._post_collective_prefetch_kb):
            return ops.linear(x, w)

    def _moe_ffn(self, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        """Routed experts + optional shared expert.

        With expert parallelism (``ep_size`` = group size) the experts are partitioned across ranks;
        tokens are replicated after the attention all-reduce, so each rank runs its local experts on
        the rows routed to them and the combine is the weighted sum + all-reduce (the shared expert,
        sharded by ``tp_rank``, rides in the same all-reduce).  With ``ep_size`` = 1 every rank holds
        all experts and computes the whole routed sum itself; only the tensor-parallel shared expert
        is all-reduced.  Any other combination is rejected when the model is built."""
        cfg = self.cfg
        logits = ops.linear(x, lw.router).float()
        ep_sharded = self.w.ep_size > 1
        sh = None
        if lw.shared_gate_up is not None:
            sh = ops.linear(ops.silu_mul(ops.linear(x, lw.shared_gate_up)), lw.shared_down)
            if not ep_sharded and self.w.tp_size > 1:
                sh = self.comm.all_reduce(sh)
            if lw.shared_gate is not None:
                sh = (sh.float() * torch.sigmoid(ops.linear(x, lw.shared_gate).float())).to(sh.dtype)
        if x.is_cuda:
            from ..ops import cuda_moe

            out = cuda_moe.moe_layer(x, logits, cfg, lw.router_bias, lw.experts, sh)
            return self.comm.all_reduce(out) if ep_sharded else out
        ids, wts = ops.moe_route(logits, cfg, lw.router_bias)
        out = moe_experts_forward(x, ids, wts, lw.experts)
        if sh is not None:
            out = out + sh
        return self.comm.all_reduce(out) if ep_sharded else out

    def run_layers(self, h: torch.Tensor, residual: Optional[torch.Tensor], meta: BatchMeta, kv,
                   layers: Optional[Tuple[int, int]] = None, capture: Optional[dict] = None):
        """Run local layers; returns (h, residual) where the true hidden is h + residual."""
        cfg = self.cfg
        lo, hi = layers if layers is not None else (0, len(self.w.layers))
        for li in range(lo, hi):
            lw = self.w.layers[li]
            gl = self.w.first_layer + li
            x, residual = ops.add_rmsnorm(h, residual, lw.attn_norm, cfg.rms_eps)
            h = self._attention(lw, li, x, meta, kv)
            x, residual = ops.add_rmsnorm(h, residual, lw.ffn_norm, cfg.rms_eps)
            h = self._moe_ffn(lw, x) if lw.router is not None else self._dense_ffn(lw, x)
            if capture is not None and gl in capture.get("layers", ()):
                capture.setdefault("hidden", {})[gl] = (h.float() + residual.float())
            if _profiler.TRACE_FWD:
                _profiler.trace_hidden(gl, h, residual)
        return h, residual

    def embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embed(token_ids, self.w.embed, self.act_dtype)

    def head(self, h: torch.Tensor, residual: Optional[torch.Tensor], logits_indices: torch.Tensor,
             return_hidden: bool = False):
        """Final norm + vocabulary-parallel lm_head on the selected rows; logits float32."""
        if logits_indices is not None:
            idx = logits_indices.long()
            h = h.index_select(0, idx)
            residual = residual.index_select(0, idx) if residual is not None else None
        x, hidden = ops.add_rmsnorm(h, residual, self.w.out_norm, self.cfg.rms_eps)
        logits = ops.linear(x, self.w.lm_head).float()
        if self.w.tp_size > 1 and self.w.lm_head.out_features != self.cfg.vocab_size:
            logits = self.comm.all_gather_cat(logits, dim=-1)
        return (logits, hidden) if return_hidden else logits

    def greedy_tokens(self, meta: BatchMeta, kv, tie: str = "lowest") -> torch.Tensor:
        """Forward + argmax without ever materialising full-vocabulary logits across ranks:
        each rank takes the argmax of its vocabulary shard and only (value, index) pairs are
        all-gathered (vocabulary-parallel head, distributed argmax)."""
        h = self.embed(meta.token_ids)
        h, residual = self.run_layers(h, None, meta, kv)
        idx = meta.logits_indices.long()
        h = h.index_select(0, idx)
        residual = residual.index_select(0, idx) if residual is not None else None
        x, hid = ops.add_rmsnorm(h, residual, self.w.out_norm, self.cfg.rms_eps)
        self.last_hidden = hid  # pre-norm hidden of the logits rows (input of an MTP head)
        logits = ops.linear(x, self.w.lm_head).float()
        sharded = self.w.tp_size > 1 and self.w.lm_head.out_features != self.cfg.vocab_size
        if not sharded:
            return ops.argmax(logits, tie)
        if logits.is_cuda:
            from ..ops import cuda as opcuda

            val = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
            loc = opcuda.argmax(logits, tie, out_val=val, index_offset=self.w.vocab_start)
        else:
            loc = ops.argmax(logits, tie) + self.w.vocab_start
            val = logits.gather(1, (loc - self.w.vocab_start).long()[:, None]).squeeze(1)
        pair = torch.stack([val, loc.view(torch.float32) if loc.dtype == torch.int32 else loc.float()], dim=1)
        allp = self.comm.all_gather_cat(pair.contiguous(), dim=0).reshape(self.w.tp_size, -1, 2)
        vals = allp[:, :, 0]
        ids = allp[:, :, 1].contiguous().view(torch.int32)
        # shards are in ascending vocabulary order: first max = lowest index, last max = highest
        if tie == "highest":
            win = self.w.tp_size - 1 - torch.flip(vals, dims=[0]).argmax(dim=0)
        else:
            win = vals.argmax(dim=0)
        return ids.gather(0, win[None, :]).squeeze(0)

    def forward(self, meta: BatchMeta, kv, return_hidden: bool = False, capture: Optional[dict] = None):
        h = self.embed(meta.token_ids)
        h, residual = self.run_layers(h, None, meta, kv, capture=capture)
        return self.head(h, residual, meta.logits_indices, return_hidden)


def moe_experts_forward(x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, experts) -> torch.Tensor:
    """Σ_k w[t,k] · down_e(silu(gate_e x) ⊙ up_e x) over the experts held locally."""
    if x.is_cuda:
        from ..ops import cuda as opcuda

        return opcuda.moe_experts_forward(x, ids, wts, experts)
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    n_local = len(experts.gate_up)
    for le in range(n_local):
        e = experts.first_expert + le
        sel = (ids == e)
        rows = sel.any(dim=1).nonzero(as_tuple=True)[0]
        if rows.numel() == 0:
            continue
        w = (wts * sel).sum(dim=1)[rows]
        xe = x.index_select(0, rows)
        y = ops.linear(ops.silu_mul(ops.linear(xe, experts.gate_up[le])), experts.down[le])
        out.index_add_(0, rows, y.float() * w[:, None])
    return out.to(x.dtype)
