"""Decoder-only transformer forward over a flat token batch and a paged KV cache.

One code path serves decode (1 query row per sequence), chunked prefill and speculative
verification (several rows per sequence) for Llama / Mistral / Qwen3 (per-head QK-norm),
Gemma 1-3 (GeGLU, scaled embeddings, norms on the branch outputs, soft-capped logits, local / global
layers with two rotary bases; the reference's ``layers.rs:293-304,1323,1515``), DeepSeek-V2/V3 latent
attention (``deepseek_mla_layer`` ``layers.rs:1547``; here with the latent itself in the cache) and the MoE families Mixtral / Qwen3-MoE / DeepSeek-MoE (shared expert, sigmoid+bias
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
    logits_all: bool = False  # logits_indices is the identity (every row is a logits row): no row gather needed
    # host copies for CPU-side loops (reference path); optional on the GPU path
    extra: dict = field(default_factory=dict)


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
    def __init__(self, weights: ModelWeights, comm=None, act_dtype: Optional[torch.dtype] = None, fold_norms: bool = False,
                 fuse_qkv_rope: bool = True, fuse_swiglu: bool = True, pipe=None, max_context: int = 0):
        self.w = weights
        self.pipe = pipe  # parallel.pp.StageIO when this model holds one pipeline stage's layers
        # layers whose outputs (hidden states of the logits rows, concatenated) are kept in ``last_features`` after every
        # forward: the input of a hidden-conditioned draft model
        self.capture_layers: Optional[List[int]] = None
        self.last_features: Optional[torch.Tensor] = None
        self._sends: list = []  # activation sends still on the link
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
        # frequency factors stored in the checkpoint; LongRoPE switches to its long set (and its magnitude factor) when
        # the serving context exceeds the one the model was trained with
        ff, mscale = weights.rope_freq_factors, opref.rope_mscale(cfg.rope_scaling)
        orig_ctx = cfg.rope_scaling.original_context_length if cfg.rope_scaling is not None else 0
        if weights.rope_freq_factors_long is not None and orig_ctx > 0 and (max_context or cfg.context_length) > orig_ctx:
            ff, mscale = weights.rope_freq_factors_long, mscale * cfg.rope_attn_factor
        self.rope = RopeState(
            inv_freq=opref.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta, cfg.rope_scaling, device=dev, freq_factors=ff),
            pairing=cfg.rope_pairing, mscale=mscale,
            n_heads=self.n_heads_local, n_kv_heads=self.n_kv_local, head_dim=cfg.head_dim)
        # windowed layers with a rotary base of their own (Gemma-3): that base, and no context scaling
        self.rope_swa = None
        if cfg.rope_theta_swa > 0 and cfg.sliding_window > 0:
            self.rope_swa = RopeState(
                inv_freq=opref.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta_swa, None, device=dev),
                pairing=cfg.rope_pairing, mscale=1.0,
                n_heads=self.n_heads_local, n_kv_heads=self.n_kv_local, head_dim=cfg.head_dim)
        self.attn_scale = cfg.attn_scale if cfg.attn_scale > 0 else cfg.head_dim ** -0.5
        self.kv_head_dim = cfg.head_dim  # width of one cached key / value row
        # which cache layer a decoder layer writes: attention layers count through the KV cache, convolution layers (hybrid
        # models) through a second cache that holds their gated inputs; the reference's ``kv_layer_map`` (load.rs:470-480)
        conv = set(i - weights.first_layer for i in cfg.conv_layers)
        gdn = set(i - weights.first_layer for i in cfg.gdn_layers)
        self.kv_index, self.conv_index = [], []
        for li in range(len(weights.layers)):
            is_conv = li in conv
            self.kv_index.append(-1 if (is_conv or li in gdn) else sum(1 for j in range(li) if j not in conv and j not in gdn))
            self.conv_index.append(sum(1 for j in range(li) if j in conv) if is_conv else -1)
        self.n_kv_layers = sum(1 for i in self.kv_index if i >= 0)
        self.n_conv_layers = sum(1 for i in self.conv_index if i >= 0)
        # layers with a recurrent state, numbered among themselves
        rec = sorted(gdn) if gdn else (list(range(len(weights.layers))) if cfg.ssm_d_inner > 0 else [])
        self.rec_index = {li: n for n, li in enumerate(rec)}
        # state-space layers: per-sequence recurrent state (convolution window + [d_inner, d_state] state per layer), in
        # slots found through the sequence's first page (see _ssm_slot)
        self._ssm_slots: dict = {}
        self._ssm_conv = self._ssm_state = None
        self._ssm_clock = 0
        if cfg.ssm_d_inner > 0:
            self.n_kv_layers = 0
        if cfg.is_mla:
            # One cached row per token, shared by all heads: the normalised latent followed by the rotary key.
            self.n_kv_local = 1
            self.kv_head_dim = cfg.kv_lora_rank + cfg.rotary_dim
            self.latent_statement = dev.type == "cuda"  # attention over latent rows as batched torch products
            self.rope.n_kv_heads = 1
            if cfg.rope_scaling.type == "yarn" and cfg.rope_scaling.factor > 1:
                # DeepSeek's YaRN: the magnitude correction goes into the softmax scale (squared: it would have
                # multiplied queries and keys), not into the rotary table
                import math

                m = 1.0 + cfg.yarn_log_multiplier * math.log(cfg.rope_scaling.factor)
                self.rope.mscale = 1.0
                self.attn_scale *= m * m
        self._fuse_qkv_rope = dev.type == "cuda" and fuse_qkv_rope
        # (load-time re-layouts walk every layer: not for a model that streams its layers from the file)
        streamed = not isinstance(weights.layers, list)
        if dev.type == "cuda" and fuse_swiglu and not streamed:
            self._interleave_gate_up()
        if dev.type == "cuda" and fold_norms and not streamed:
            self._fold_norm_weights()

    def _fold_norm_weights(self) -> None:
        """Fold the two RMSNorm weight vectors of a dense bf16 layer into the columns of the projections that
        consume them (qkv, gate_up).  What is left of a norm is one scalar per token, which the consuming GEMM
        applies in its epilogue from sums of squares that the epilogue writing the residual stream leaves behind
        (``run_layers``): two kernels per layer disappear.  The norm vectors become all-ones, so the unfused
        kernels still compute the same function on these weights."""
        cfg = self.cfg
        if cfg.hidden_size % 8:
            return

        def bf16_single(w) -> bool:
            return (w is not None and len(w.parts) == 1 and w.parts[0].qtype == "BF16" and w.bias is None
                    and w.parts[0].data.is_contiguous())

        for lw in self.w.layers:
            if (lw.router is not None or lw.post_attn_norm is not None or lw.post_ffn_norm is not None or cfg.qk_norm_after_rope
                    or cfg.attn_out_gate or cfg.qk_norm_full
                    or not (bf16_single(lw.wqkv) and bf16_single(lw.wo) and bf16_single(lw.w_gate_up)
                            and bf16_single(lw.w_down) and lw.w_gate_up.swiglu_interleaved)):
                continue
            if lw.wo.parts[0].shape[0] % 8 or lw.w_down.parts[0].shape[0] % 8:
                continue
            for w, norm in ((lw.wqkv, lw.attn_norm), (lw.w_gate_up, lw.ffn_norm)):
                d = w.parts[0].data
                step = max(1, (1 << 27) // d.shape[1])
                nv = norm.float()[None, :]
                for r in range(0, d.shape[0], step):  # in row chunks: no second copy of a large matrix
                    d[r : r + step] = (d[r : r + step].float() * nv).to(d.dtype)
            lw.attn_norm = torch.ones_like(lw.attn_norm)
            lw.ffn_norm = torch.ones_like(lw.ffn_norm)
            lw.norms_folded = True  # on the layer object: layer lists are swapped in and out (MTP head)

    def _row_parallel_into(self, x: torch.Tensor, w, r: torch.Tensor, acc: torch.Tensor) -> None:
        """r += all_reduce(x @ w^T) in place; ``acc`` (cleared by the preceding consumer) receives the sums of squares
        of the new rows of r."""
        from ..ops import cuda as opcuda

        comm = self.comm
        if getattr(comm, "size", 1) == 1:
            xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
            opcuda.gemm_bf16(xb.contiguous(), w.parts[0].data, out=r, add_into=True, sumsq_out=acc)
            return
        into = getattr(comm, "linear_allreduce_into", None)
        if into is None or not into(x, w, r, acc):  # prefill-sized calls, or a comm without the fused kernels
            r.add_(comm.linear_allreduce(x, w))
            opcuda.row_sumsq(r, acc)

    def _layer_folded(self, lw: LayerWeights, layer: int, r: torch.Tensor, acc: torch.Tensor, cur: int, meta: BatchMeta,
                      kv) -> int:
        """One dense layer on the residual stream ``r`` (updated in place) with both norms folded: five kernels.
        ``acc`` is the pair of per-token sum-of-squares accumulators, ``acc[cur]`` describes r; returns the new ``cur``."""
        from ..ops import cuda as opcuda

        cfg = self.cfg
        eps = cfg.rms_eps
        wq = lw.wqkv.parts[0].data
        window = cfg.layer_sliding_window(self.w.first_layer + layer)
        rope = self._layer_rope(window)
        if self._fuse_qkv_rope and opcuda.qkv_rope_fusable(lw.wqkv.parts, kv, rope, lw.q_norm, lw.k_norm):
            q = opcuda.linear_qkv_rope(r, wq, meta.positions, meta.slot_mapping, kv, layer, rope, sumsq_in=acc[cur],
                                       eps=eps, clear=acc[1 - cur])
        else:
            qkv = opcuda.gemm_bf16(r, wq, sumsq_in=acc[cur], eps=eps, clear=acc[1 - cur])
            q = ops.qk_rope_kv_write(qkv, meta.positions, meta.slot_mapping, kv, layer, rope, lw.q_norm, lw.k_norm, eps)
        attn = ops.paged_attention(q, kv, layer, meta, self.attn_scale, window, cfg.attn_softcap)
        cur = 1 - cur
        self._row_parallel_into(attn.reshape(attn.shape[0], -1), lw.wo, r, acc[cur])
        act = opcuda.linear_swiglu(r, lw.w_gate_up.parts[0].data, sumsq_in=acc[cur], eps=eps, clear=acc[1 - cur],
                                   gelu=cfg.ffn_act == "gelu_tanh")
        cur = 1 - cur
        self._row_parallel_into(act, lw.w_down, r, acc[cur])
        return cur

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
    def new_cache(self, num_blocks: int, page_size: int, dtype_name: str):
        """A paged cache shaped for this model: KV rows for the attention layers and, for a hybrid model, a second cache
        (same pages, same block ids) whose rows are the convolution layers' gated inputs, split over its K and V halves."""
        from ..engine.kv_pool import KVCache, KVCacheSpec

        kv = KVCache(KVCacheSpec(max(1, self.n_kv_layers), self.n_kv_local, self.kv_head_dim, page_size, dtype_name),
                     num_blocks, self.device)
        if self.n_conv_layers:
            if self.cfg.hidden_size % 2:
                raise ValueError("convolution layers need an even hidden size")
            plain = "bf16" if self.device.type == "cuda" else "f32"  # never quantized: the rows are convolved, not attended
            kv.conv = KVCache(KVCacheSpec(self.n_conv_layers, 1, self.cfg.hidden_size // 2, page_size, plain), num_blocks,
                              self.device)
        return kv

    def _ssm_slot(self, kv, first_block: int, position: int) -> int:
        """State slot of the sequence whose first page is ``first_block`` in cache ``kv``.  A sequence keeps its first page
        for as long as it runs (prefix sharing is off for these models), a new or restarted sequence shows up at position 0
        and gets a cleared slot; slots not touched for many steps are handed to newcomers."""
        cfg = self.cfg
        key = (id(kv), first_block)
        ent = self._ssm_slots.get(key)
        if ent is None and position != 0:
            raise RuntimeError("the recurrent state of a running sequence is gone (its slot was handed on after "
                               "thousands of steps without a row of that sequence)")
        if ent is None or position == 0:
            if ent is None:
                used = {v[0] for v in self._ssm_slots.values()}
                n = 0 if self._ssm_state is None else self._ssm_state.shape[0]
                slot = next((i for i in range(n) if i not in used), None)
                if slot is None:
                    stale = [k for k, v in self._ssm_slots.items() if self._ssm_clock - v[1] > 4096]
                    if stale:
                        slot = self._ssm_slots.pop(stale[0])[0]
                    else:  # grow by one block of slots
                        L = len(self.rec_index)
                        if cfg.gdn_layers:  # convolution window over q / k / v rows, one [key, value] matrix per value head
                            rows = 2 * cfg.gdn_k_heads * cfg.gdn_k_dim + cfg.gdn_v_heads * cfg.gdn_v_dim
                            c_shape, s_shape = (rows, max(1, cfg.gdn_conv - 1)), (cfg.gdn_v_heads, cfg.gdn_k_dim, cfg.gdn_v_dim)
                        else:
                            c_shape, s_shape = (cfg.ssm_d_inner, max(1, cfg.ssm_d_conv - 1)), (cfg.ssm_d_inner, cfg.ssm_d_state)
                        add_c = torch.zeros(16, L, *c_shape, dtype=torch.float32, device=self.device)
                        add_s = torch.zeros(16, L, *s_shape, dtype=torch.float32, device=self.device)
                        self._ssm_conv = add_c if self._ssm_conv is None else torch.cat([self._ssm_conv, add_c])
                        self._ssm_state = add_s if self._ssm_state is None else torch.cat([self._ssm_state, add_s])
                        slot = n
                ent = [slot, self._ssm_clock]
                self._ssm_slots[key] = ent
            if position == 0:
                self._ssm_conv[ent[0]].zero_()
                self._ssm_state[ent[0]].zero_()
        ent[1] = self._ssm_clock
        return ent[0]

    def release_state(self, kv) -> None:
        """Forget the state slots of every sequence of cache ``kv`` (a cache that lived for one call)."""
        for key in [k for k in self._ssm_slots if k[0] == id(kv)]:
            del self._ssm_slots[key]

    def _mamba(self, lw: LayerWeights, layer: int, x: torch.Tensor, meta: BatchMeta, kv) -> torch.Tensor:
        """Selective state-space mixer, sequence by sequence and token by token (the recurrence is sequential):
        (u, z) = in_proj(x); u = silu(conv(u)); (dt, B, C) = x_proj(u); dt = softplus(dt_proj(dt) + b);
        h = exp(A dt) h + dt B u; y = (h C + D u) silu(z); out_proj(y)."""
        cfg, m = self.cfg, lw.ssm
        di, N, K, R = cfg.ssm_d_inner, cfg.ssm_d_state, cfg.ssm_d_conv, cfg.ssm_dt_rank
        xz = ops.linear(x, m.in_proj).float()
        u_all, z_all = xz[:, :di], xz[:, di:]
        qs, first = meta.query_start.tolist(), meta.block_tables[:, 0].tolist()
        pos0 = meta.positions.tolist()
        w, A, D = m.conv_kernel.float(), m.a.float(), m.d.float()
        y = torch.empty_like(u_all)
        if layer == 0:
            self._ssm_clock += 1
        for b in range(len(qs) - 1):
            t0, t1 = qs[b], qs[b + 1]
            if t1 == t0:
                continue
            slot = self._ssm_slot(kv, first[b], pos0[t0] if layer == 0 else -1)
            win = torch.cat([self._ssm_conv[slot, layer], u_all[t0:t1].t()], dim=1)  # [di, K-1 + n]
            conv = sum(w[:, j : j + 1] * win[:, j : j + (t1 - t0)] for j in range(K))
            if m.conv_bias is not None:
                conv = conv + m.conv_bias.float()[:, None]
            uc = torch.nn.functional.silu(conv).t().contiguous()  # [n, di]
            self._ssm_conv[slot, layer] = win[:, -(K - 1):] if K > 1 else win[:, :0]
            # step size, B and C steer an exponential recurrence: these two narrow projections stay in float32 (plain
            # products on the decoded matrices) instead of going through the bf16 GEMM
            par = uc @ m.x_proj.dense_cache().float().t()
            dt = torch.nn.functional.softplus(par[:, :R] @ m.dt_proj.dense_cache().float().t() + m.dt_bias.float())
            Bm, Cm = par[:, R : R + N], par[:, R + N :]
            h = self._ssm_state[slot, layer]
            for i in range(t1 - t0):
                h = torch.exp(A * dt[i][:, None]) * h + (dt[i] * uc[i])[:, None] * Bm[i][None, :]
                y[t0 + i] = h @ Cm[i] + D * uc[i]
            self._ssm_state[slot, layer] = h
        return ops.linear((y * torch.nn.functional.silu(z_all)).to(x.dtype), m.out_proj)

    def _gated_delta(self, lw: LayerWeights, layer: int, x: torch.Tensor, meta: BatchMeta, kv) -> torch.Tensor:
        """Gated delta rule (Qwen3.5's linear attention), sequence by sequence and token by token:
        (q, k, v) = silu(conv(in_qkv(x))), q and k scaled to unit length per head; per value head a [key, value] matrix S:
        S = exp(g) S; S += k (beta (v - S^T k))^T; o = S^T q / sqrt(d_k), with g = A softplus(in_a(x) + dt_bias) and
        beta = sigmoid(in_b(x)); out_proj(rmsnorm(o) * silu(in_z(x))).  The reference's run_mamba_layer
        (model/layer_wise/ssm.rs:82) is the same recurrence on one token."""
        cfg, m = self.cfg, lw.gdn
        Hk, Hv, dk, dv, K = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_k_dim, cfg.gdn_v_dim, cfg.gdn_conv
        kdim = Hk * dk
        F = torch.nn.functional
        T = x.shape[0]
        mixed = ops.linear(x, m.in_qkv).float()
        z = ops.linear(x, m.in_z).float().reshape(T, Hv, dv)
        # decay and write strength steer an exponential recurrence: these two narrow projections stay in float32
        xf = x.float()
        beta_all = torch.sigmoid(xf @ m.in_b.dense_cache().float().t())
        g_all = m.a.float() * F.softplus(xf @ m.in_a.dense_cache().float().t() + m.dt_bias.float())
        qs, first = meta.query_start.tolist(), meta.block_tables[:, 0].tolist()
        pos0 = meta.positions.tolist()
        w = m.conv_kernel.float()
        ri = self.rec_index[layer]
        if ri == 0:
            self._ssm_clock += 1
        out = torch.empty(T, Hv, dv, dtype=torch.float32, device=x.device)
        for b in range(len(qs) - 1):
            t0, t1 = qs[b], qs[b + 1]
            if t1 == t0:
                continue
            n = t1 - t0
            slot = self._ssm_slot(kv, first[b], pos0[t0] if ri == 0 else -1)
            win = torch.cat([self._ssm_conv[slot, ri], mixed[t0:t1].t()], dim=1)  # [rows, K-1 + n]
            qkv = F.silu(sum(w[:, j : j + 1] * win[:, j : j + n] for j in range(K))).t()  # [n, rows]
            self._ssm_conv[slot, ri] = win[:, -(K - 1):] if K > 1 else win[:, :0]
            q = qkv[:, :kdim].reshape(n, Hk, dk)
            k = qkv[:, kdim : 2 * kdim].reshape(n, Hk, dk)
            v = qkv[:, 2 * kdim :].reshape(n, Hv, dv)
            q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
            k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            if Hv != Hk:  # consecutive value heads share a key head
                q, k = q.repeat_interleave(Hv // Hk, dim=1), k.repeat_interleave(Hv // Hk, dim=1)
            decay, beta = torch.exp(g_all[t0:t1]), beta_all[t0:t1]
            S = self._ssm_state[slot, ri]  # [Hv, dk, dv]
            for i in range(n):
                S = S * decay[i][:, None, None]
                delta = (v[i] - (S * k[i][:, :, None]).sum(1)) * beta[i][:, None]
                S = S + k[i][:, :, None] * delta[:, None, :]
                out[t0 + i] = (S * q[i][:, :, None]).sum(1)
            self._ssm_state[slot, ri] = S
        y = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * m.norm.float() * F.silu(z)
        return ops.linear(y.reshape(T, Hv * dv).to(x.dtype), m.out_proj)

    def _short_conv(self, lw: LayerWeights, layer: int, x: torch.Tensor, meta: BatchMeta, kv) -> torch.Tensor:
        """LFM2 mixer: (B, C, v) = in_proj(x); u = B * v; y_t = C_t * sum_j w[:, j] u_{t - (L-1) + j}; out_proj(y).  The rows u
        go into the convolution cache at the token's slot, and the L-1 earlier rows a token needs are read back through
        its sequence's block table: earlier chunks, cached prefixes and rows of this very step alike."""
        cfg = self.cfg
        h, L = cfg.hidden_size, cfg.conv_l_cache
        cache, idx = kv.conv, self.conv_index[layer]
        bcx = ops.linear(x, lw.conv_in).float()
        gate_b, gate_c, v = bcx[:, :h], bcx[:, h : 2 * h], bcx[:, 2 * h :]
        u = gate_b * v
        opref.kv_write(cache, idx, u[:, None, : h // 2], u[:, None, h // 2 :], meta.slot_mapping)
        qs = meta.query_start.long()
        row_seq = torch.repeat_interleave(torch.arange(qs.numel() - 1, device=x.device), qs[1:] - qs[:-1])
        pos = meta.positions.long()
        page = cache.page_size
        w = lw.conv_kernel.float()
        acc = w[:, L - 1] * u
        data = cache.data[idx]
        for j in range(1, L):
            q = pos - j
            ok = q >= 0
            qc = q.clamp(min=0)
            blk = meta.block_tables[row_seq, qc // page].long()
            prev = torch.cat([data[blk, 0, 0, qc % page], data[blk, 0, 1, qc % page]], dim=-1).float()
            acc = acc + w[:, L - 1 - j] * prev * ok[:, None]
        return ops.linear((gate_c * acc).to(x.dtype), lw.conv_out)

    def _layer_rope(self, window: int) -> RopeState:
        """Rotary state of a layer: windowed layers use their own base when the model has one."""
        return self.rope_swa if (window > 0 and self.rope_swa is not None) else self.rope

    def _mla_attention(self, lw: LayerWeights, layer: int, x: torch.Tensor, meta: BatchMeta, kv) -> torch.Tensor:
        """Latent attention in its "absorbed" form.  Per token the cache holds ONE row shared by all heads:
        [norm(latent) (kv_lora), rope(k_pe) (rope)].  A head's key would be [W_uk latent, k_pe] and its value W_uv latent;
        instead of rebuilding them for every cached token, the query's position-free part is multiplied by W_uk once
        (q_nope . (W_uk c) = (W_uk^T q_nope) . c), attention runs as multi-query attention over the latent rows, and the
        attended latent is multiplied by W_uv afterwards.  Same function, kv_lora + rope cached values per token instead of
        heads * (nope + rope + v)."""
        cfg, m = self.cfg, lw.mla
        T, H = x.shape[0], self.n_heads_local
        nope, rot, c = cfg.qk_nope_dim, cfg.rotary_dim, cfg.kv_lora_rank
        if m.q_a is not None:
            q = ops.linear(ops.rmsnorm(ops.linear(x, m.q_a), m.q_a_norm, cfg.rms_eps), m.q_b)
        else:
            q = ops.linear(x, m.q)
        q = q.reshape(T, H, nope + rot)
        ckv = ops.linear(x, m.kv_a)
        latent = ops.rmsnorm(ckv[:, :c].contiguous(), m.kv_a_norm, cfg.rms_eps)
        rope = self.rope
        k_pe = opref.apply_rope(ckv[:, c:].reshape(T, 1, rot), meta.positions, rope.inv_freq, rope.pairing, rope.mscale)
        q_pe = opref.apply_rope(q[:, :, nope:], meta.positions, rope.inv_freq, rope.pairing, rope.mscale)
        q_lat = torch.einsum("thn,hnc->thc", q[:, :, :nope].float(), m.w_uk.float()).to(x.dtype)
        row = torch.cat([latent[:, None, :], k_pe], dim=-1)  # [T, 1, c + rot]
        opref.kv_write(kv, layer, row, row, meta.slot_mapping)
        qq = torch.cat([q_lat, q_pe], dim=-1)
        if self.latent_statement:
            # the attention kernel has 64- and 128-wide heads; over the (kv_lora + rope)-wide latent rows the attention
            # step runs as batched matrix products (torch) on the device
            o = opref.latent_attention(qq, kv, layer, meta, self.attn_scale, c)
        else:
            o = ops.paged_attention(qq, kv, layer, meta, self.attn_scale, 0)[:, :, :c]
        out = torch.einsum("thc,hvc->thv", o.float(), m.w_uv.float()).to(x.dtype)
        return self.comm.linear_allreduce(out.reshape(T, -1), lw.wo)

    def _attention(self, lw: LayerWeights, layer: int, x: torch.Tensor, meta: BatchMeta, kv) -> torch.Tensor:
        cfg = self.cfg
        if lw.conv_in is not None:
            return self._short_conv(lw, layer, x, meta, kv)
        if lw.gdn is not None:
            return self._gated_delta(lw, layer, x, meta, kv)
        window_of = self.w.first_layer + layer  # the window pattern counts decoder layers, the cache counts attention layers
        layer = self.kv_index[layer]
        if lw.mla is not None:
            return self._mla_attention(lw, layer, x, meta, kv)
        window = cfg.layer_sliding_window(window_of)
        rope = self._layer_rope(window)
        if (self._fuse_qkv_rope and x.is_cuda and lw.wqkv.bias is None and not cfg.qk_norm_after_rope and not cfg.attn_out_gate
                and not cfg.qk_norm_full):
            from ..ops import cuda as opcuda

            if opcuda.qkv_rope_fusable(lw.wqkv.parts, kv, rope, lw.q_norm, lw.k_norm):
                q = opcuda.linear_qkv_rope(x, lw.wqkv.parts[0].data, meta.positions, meta.slot_mapping, kv, layer, rope)
                attn = ops.paged_attention(q, kv, layer, meta, self.attn_scale, window, cfg.attn_softcap)
                return self.comm.linear_allreduce(attn.reshape(attn.shape[0], -1), lw.wo)
        qkv = ops.linear(x, lw.wqkv)
        gate = None
        if cfg.attn_out_gate:
            # the query block holds, per head, the query and then that head's output gate: pull the gates out
            nq, hd = self.n_heads_local, cfg.head_dim
            qg = qkv[:, : nq * 2 * hd].reshape(-1, nq, 2 * hd)
            gate = qg[:, :, hd:].reshape(-1, nq * hd)
            qkv = torch.cat([qg[:, :, :hd].reshape(-1, nq * hd), qkv[:, nq * 2 * hd :]], dim=-1)
        q_norm, k_norm = lw.q_norm, lw.k_norm
        if cfg.qk_norm_full and q_norm is not None:
            # one norm over all heads of q and one over all heads of k, ahead of the head split
            if self.w.tp_size > 1:
                raise ValueError("a norm over all heads is not sharded: run this model with tp_size = 1")
            nq, nk = self.n_heads_local * cfg.head_dim, self.n_kv_local * cfg.head_dim
            qkv = torch.cat([opref.rmsnorm(qkv[:, :nq], q_norm, cfg.rms_eps).to(qkv.dtype),
                             opref.rmsnorm(qkv[:, nq : nq + nk], k_norm, cfg.rms_eps).to(qkv.dtype), qkv[:, nq + nk :]], dim=-1)
            q_norm = k_norm = None
        q = ops.qk_rope_kv_write(qkv, meta.positions, meta.slot_mapping, kv, layer, rope, q_norm, k_norm, cfg.rms_eps,
                                 norm_after=cfg.qk_norm_after_rope)
        attn = ops.paged_attention(q, kv, layer, meta, self.attn_scale, window, cfg.attn_softcap)
        if gate is not None:
            attn = (attn.reshape(attn.shape[0], -1) * torch.sigmoid(gate.float())).to(attn.dtype)
        return self.comm.linear_allreduce(attn.reshape(attn.shape[0], -1), lw.wo)

    def _dense_ffn(self, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        if lw.w_gate_up.swiglu_interleaved:
            from ..ops import cuda as opcuda

            act = opcuda.linear_swiglu(x, lw.w_gate_up.parts[0].data, gelu=self.cfg.ffn_act == "gelu_tanh")
        elif self.cfg.ffn_act == "gelu_tanh":
            act = ops.gelu_mul(ops.linear(x, lw.w_gate_up))
        else:
            act = ops.silu_mul(ops.linear(x, lw.w_gate_up))
        return self.comm.linear_allreduce(act, lw.w_down)

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

            out, reduced = cuda_moe.moe_layer(x, logits, cfg, lw.router_bias, lw.experts, sh,
                                              self.comm if ep_sharded else None)
            return self.comm.all_reduce(out) if (ep_sharded and not reduced) else out
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
        acc, cur = None, 0  # per-token sum-of-squares accumulators of the residual stream while it is in folded form
        for li in range(lo, hi):
            lw = self.w.layers[li]
            gl = self.w.first_layer + li
            if getattr(lw, "norms_folded", False) and (h if h is not None else residual).dtype == torch.bfloat16:
                from ..ops import cuda as opcuda

                if acc is None:
                    # enter the folded form: the residual stream becomes one tensor, updated in place from here on
                    # (a stream that arrives as h alone, e.g. the embedding output, is taken over as it is)
                    if residual is not None:
                        residual.add_(h)
                    else:
                        residual = h.contiguous()
                    h = None
                    # two accumulator arrays, one 128-byte line per token (ops.cuda.SUMSQ_STRIDE words)
                    acc = torch.empty(2, residual.shape[0] * opcuda.SUMSQ_STRIDE, dtype=torch.int64, device=residual.device)
                    cur = 0
                    opcuda.row_sumsq(residual, acc[0])
                cur = self._layer_folded(lw, li, residual, acc, cur, meta, kv)
                if capture is not None and gl in capture.get("layers", ()):
                    capture.setdefault("hidden", {})[gl] = residual.float()
                if _profiler.TRACE_FWD:
                    _profiler.trace_hidden(gl, residual, None)
                continue
            if acc is not None:
                # leave the folded form: h + residual must again be the hidden state
                h, acc = torch.zeros_like(residual), None
            x, residual = ops.add_rmsnorm(h, residual, lw.attn_norm, cfg.rms_eps)
            if lw.ssm is not None:  # norm -> mixer -> residual; no feed-forward block
                h = self._mamba(lw, li, x, meta, kv)
                if capture is not None and gl in capture.get("layers", ()):
                    capture.setdefault("hidden", {})[gl] = (h.float() + residual.float())
                continue
            h = self._attention(lw, li, x, meta, kv)
            if lw.post_attn_norm is not None:
                h = ops.rmsnorm(h, lw.post_attn_norm, cfg.rms_eps)
            x, residual = ops.add_rmsnorm(h, residual, lw.ffn_norm, cfg.rms_eps)
            h = self._moe_ffn(lw, x) if lw.router is not None else self._dense_ffn(lw, x)
            if lw.post_ffn_norm is not None:
                h = ops.rmsnorm(h, lw.post_ffn_norm, cfg.rms_eps)
            if capture is not None and gl in capture.get("layers", ()):
                capture.setdefault("hidden", {})[gl] = (h.float() + residual.float())
            if _profiler.TRACE_FWD:
                _profiler.trace_hidden(gl, h, residual)
        if acc is not None:
            return residual, None
        return h, residual

    def _keep_features(self, capture: Optional[dict], idx: Optional[torch.Tensor]) -> None:
        if not self.capture_layers or capture is None or "hidden" not in capture:
            return
        hs = [capture["hidden"][l] for l in self.capture_layers if l in capture["hidden"]]
        if len(hs) == len(self.capture_layers):
            self.last_features = torch.cat([h if idx is None else h.index_select(0, idx) for h in hs], dim=-1)

    def embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embed(token_ids, self.w.embed, self.act_dtype, self.cfg.embedding_scale)

    # ------------------------------------------------------------------ pipeline stages
    def _stage_input(self, meta: BatchMeta):
        """(h, residual) entering this stage's layers: the embedding on the first stage, the previous stage's
        activations otherwise (one [2, T, H] message: h and the residual stream)."""
        if self.pipe is None or self.pipe.is_first:
            h = self.embed(meta.token_ids)
            ov = meta.extra.get("embed_overrides")
            if ov is not None:  # rows whose embedding the request supplied (image tokens)
                h.index_copy_(0, ov[0], ov[1].to(h.dtype))
            return h, None
        both = self.pipe.recv_prev((2, int(meta.token_ids.shape[0]), self.cfg.hidden_size), self.act_dtype, self.device)
        return both[0], both[1]

    def _stage_output(self, h: torch.Tensor, residual: Optional[torch.Tensor]) -> bool:
        """Hand (h, residual) to the next stage without waiting for the link; True when this was not the last stage."""
        if self.pipe is None or self.pipe.is_last:
            return False
        self._sends = [w for w in self._sends if not w.is_completed()]
        msg = torch.stack([h, residual if residual is not None else torch.zeros_like(h)])
        self._sends.append(self.pipe.send_next(msg))
        return True

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
        cap = self.cfg.final_softcap
        if cap > 0:
            logits = torch.tanh(logits / cap) * cap
        return (logits, hidden) if return_hidden else logits

    def greedy_tokens(self, meta: BatchMeta, kv, tie: str = "lowest", feed: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Forward + argmax without ever materialising full-vocabulary logits across ranks:
        each rank takes the argmax of its vocabulary shard and only (value, index) pairs are
        exchanged (vocabulary-parallel head, distributed argmax).  ``feed`` (int32, one entry per logits
        row) also receives the tokens: the next decode step's input ids, written where its kernels read them."""
        h, residual = self._stage_input(meta)
        cap = {"layers": set(self.capture_layers)} if self.capture_layers else None
        h, residual = self.run_layers(h, residual, meta, kv, capture=cap)
        if self._stage_output(h, residual):
            return None  # the tokens arrive from the last stage
        idx = None
        if not meta.logits_all:
            idx = meta.logits_indices.long()
            h = h.index_select(0, idx)
            residual = residual.index_select(0, idx) if residual is not None else None
        self._keep_features(cap, idx)
        x, hid = ops.add_rmsnorm(h, residual, self.w.out_norm, self.cfg.rms_eps)
        self.last_hidden = hid  # pre-norm hidden of the logits rows (input of an MTP head)
        logits = ops.linear(x, self.w.lm_head)
        sharded = self.w.tp_size > 1 and self.w.lm_head.out_features != self.cfg.vocab_size
        if logits.is_cuda:
            from ..ops import cuda as opcuda

            xchg = getattr(self.comm, "argmax_exchange", None) if sharded else None
            if not sharded or (xchg is not None and logits.shape[0] <= getattr(self.comm, "argmax_rows", 0)):
                # one kernel: shard argmax, pair exchange over peer memory, winner, token fed to the next step
                return opcuda.argmax_tp(logits, tie, self.w.vocab_start if sharded else 0, self.comm if sharded else None, feed)
        logits = logits.float()
        if not sharded:
            toks = ops.argmax(logits, tie)
        else:
            if logits.is_cuda:
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
            toks = ids.gather(0, win[None, :]).squeeze(0)
        if feed is not None:
            feed[: toks.shape[0]].copy_(toks.to(feed.dtype))
        return toks

    def forward(self, meta: BatchMeta, kv, return_hidden: bool = False, capture: Optional[dict] = None):
        h, residual = self._stage_input(meta)
        if capture is None and self.capture_layers:
            capture = {"layers": set(self.capture_layers)}
        h, residual = self.run_layers(h, residual, meta, kv, capture=capture)
        if self._stage_output(h, residual):
            return None
        self._keep_features(capture, None if meta.logits_indices is None else meta.logits_indices.long())
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
