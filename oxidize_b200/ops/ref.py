"""Plain-PyTorch fp32 statement of every operator: the CPU execution path and the oracle
that each sm_100a kernel is tested against.

Semantics follow the reference's CPU kernels: RMSNorm ``y = x * rsqrt(mean(x^2)+eps) * w``
(``compute/tensor/kernels/activation.rs:357``), NeoX split-half *partial* RoPE on the first
``rope_dim`` channels of each head (``activation.rs:98-198``; YaRN scaling included), online
softmax GQA attention (``compute/flash_attention.rs:596,745``), SwiGLU, and the symmetric
per-32-channel KV quantizers (``compute/kv_cache/storage.rs:90-138``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from ..quant import ref as qref

KV_QBLOCK = 32  # channels per KV quantization block


# --------------------------------------------------------------------------- weights


def dequantize_weight(w) -> torch.Tensor:
    """QTensor -> dense float32 [out, in] (host decode through the NumPy oracle)."""
    if w.qtype in ("F32", "F16", "BF16"):
        return w.data.float()
    if w.qtype == "FP8B":
        codes = w.data.cpu().numpy().reshape(-1)
        scales = w.scales.float().cpu().numpy().reshape(-1)
        out = qref.dequantize_fp8_block(codes, scales, w.block)
        return torch.from_numpy(out).reshape(w.shape).to(w.data.device)
    raw = w.data.cpu().numpy()
    n = w.shape[0] * w.shape[1]
    return torch.from_numpy(qref.dequantize(w.qtype, raw, n).copy()).reshape(w.shape).to(w.data.device)


def linear(x: torch.Tensor, w, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    dense = w.dense_cache()
    y = x.float() @ dense.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def embed(tokens: torch.Tensor, table, scale: float = 1.0) -> torch.Tensor:
    dense = table.dense_cache()
    out = dense[tokens.long()]
    return out * scale if scale != 1.0 else out


# --------------------------------------------------------------------------- norms / act


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], w: torch.Tensor, eps: float):
    """(normed, new_residual) with new_residual = x + residual (residual kept in x.dtype)."""
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(x, w, eps), x


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)


def gelu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    return (torch.nn.functional.gelu(g, approximate="tanh") * u).to(gate_up.dtype)


# --------------------------------------------------------------------------- rope


def rope_inv_freq(rotary_dim: int, theta: float, scaling=None, device=None, freq_factors=None) -> torch.Tensor:
    """Per-pair inverse frequencies [rotary_dim/2] with optional linear / YaRN scaling.  ``freq_factors``
    ([rotary_dim/2], from a ``rope_freqs.weight`` / ``rope_factors_*.weight`` tensor of the checkpoint) divides each
    frequency: that is how Llama-3.1-style and LongRoPE context extensions are stored in GGUF files."""
    half = rotary_dim // 2
    idx = torch.arange(half, dtype=torch.float64, device=device)
    inv = theta ** (-2.0 * idx / rotary_dim)
    if scaling is not None and scaling.type == "linear" and scaling.factor > 0:
        inv = inv / scaling.factor
    elif scaling is not None and scaling.type == "yarn" and scaling.factor > 1 and scaling.original_context_length > 0:
        orig = scaling.original_context_length

        def corr_dim(n_rot):
            return rotary_dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

        lo = max(math.floor(corr_dim(scaling.beta_fast)), 0)
        hi = min(math.ceil(corr_dim(scaling.beta_slow)), half - 1)
        ramp = ((idx - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        mix = 1.0 - ramp  # 1 => extrapolate (keep), 0 => interpolate
        inv = inv / scaling.factor * (1 - mix) + inv * mix
    if freq_factors is not None:
        ff = torch.as_tensor(freq_factors, dtype=torch.float64, device=inv.device).reshape(-1)
        if ff.numel() < half:
            raise ValueError(f"rope frequency factors have {ff.numel()} entries, the rotary half dimension is {half}")
        inv = inv / ff[:half]
    return inv.float()


def rope_mscale(scaling) -> float:
    if scaling is not None and scaling.type == "yarn" and scaling.factor > 1:
        return 0.1 * math.log(scaling.factor) + 1.0
    return 1.0


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, pairing: str = "split_half",
               mscale: float = 1.0) -> torch.Tensor:
    """x: [T, n_heads, head_dim]; rotates the first 2*len(inv_freq) channels of each head."""
    half = inv_freq.numel()
    rot = 2 * half
    ang = positions.double()[:, None] * inv_freq.double()[None, :]
    cos = (ang.cos() * mscale).float()[:, None, :]
    sin = (ang.sin() * mscale).float()[:, None, :]
    xf = x.float()
    xr = xf[..., :rot]
    if pairing == "split_half":
        a, b = xr[..., :half], xr[..., half:]
        out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    else:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    return torch.cat([out, xf[..., rot:]], dim=-1).to(x.dtype)


# --------------------------------------------------------------------------- KV cache


def kv_quantize(x: torch.Tensor, bits: int):
    """Symmetric per-32-channel quantization: returns (codes uint8, scales f32).

    q8: code = q + 127 with q in [-127,127]; q4: code = q + 7 with q in [-7,7], two codes per
    byte, low nibble first (storage.rs:90-138)."""
    xf = x.float().reshape(*x.shape[:-1], -1, KV_QBLOCK)
    qmax = 127.0 if bits == 8 else 7.0
    amax = xf.abs().amax(-1, keepdim=True)
    scale = amax / qmax
    inv = torch.where(scale > 0, 1.0 / scale, torch.zeros_like(scale))
    q = torch.round(xf * inv).clamp(-qmax, qmax) + qmax
    q = q.to(torch.uint8).reshape(*x.shape)
    if bits == 4:
        q = q[..., 0::2] | (q[..., 1::2] << 4)
    return q, scale.squeeze(-1)


def kv_dequantize(codes: torch.Tensor, scales: torch.Tensor, bits: int) -> torch.Tensor:
    if bits == 4:
        lo = (codes & 0xF).float() - 7.0
        hi = (codes >> 4).float() - 7.0
        q = torch.stack([lo, hi], dim=-1).flatten(-2)
    else:
        q = codes.float() - 127.0
    q = q.reshape(*q.shape[:-1], -1, KV_QBLOCK) * scales.unsqueeze(-1)
    return q.flatten(-2)


def kv_write(kv, layer: int, k: torch.Tensor, v: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Scatter post-RoPE K/V rows [T, n_kv, hd] into the paged cache at flat slots."""
    page = kv.page_size
    slots = slot_mapping.long()
    valid = slots >= 0
    if not bool(valid.all()):
        k, v, slots = k[valid], v[valid], slots[valid]
    blk, off = slots // page, slots % page
    data = kv.data[layer]
    if kv.dtype_name in ("f16", "bf16", "f32"):
        data[blk, :, 0, off] = k.to(data.dtype)
        data[blk, :, 1, off] = v.to(data.dtype)
    else:
        bits = 8 if kv.dtype_name == "q8" else 4
        kc, ks = kv_quantize(k, bits)
        vc, vs = kv_quantize(v, bits)
        data[blk, :, 0, off] = kc
        data[blk, :, 1, off] = vc
        kv.scales[layer][blk, :, 0, off] = ks
        kv.scales[layer][blk, :, 1, off] = vs


def kv_gather(kv, layer: int, block_table: torch.Tensor, seq_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense (K, V) [seq_len, n_kv, hd] float32 of one sequence, through its block table."""
    page = kv.page_size
    nb = (seq_len + page - 1) // page
    blocks = block_table[:nb].long()
    d = kv.data[layer][blocks]  # [nb, n_kv, 2, page, hd or packed]
    if kv.dtype_name in ("q8", "q4"):
        bits = 8 if kv.dtype_name == "q8" else 4
        d = kv_dequantize(d, kv.scales[layer][blocks], bits)
    d = d.float().permute(2, 0, 3, 1, 4).reshape(2, nb * page, d.shape[1], -1)[:, :seq_len]
    return d[0], d[1]


def paged_attention(q: torch.Tensor, kv, layer: int, meta, scale: float, sliding_window: int = 0,
                    softcap: float = 0.0) -> torch.Tensor:
    """Causal GQA attention of packed query rows against the paged cache.

    q: [T, n_heads, hd].  For sequence b the rows ``query_start[b]:query_start[b+1]`` are its
    last ``qlen`` positions (context length ``seq_lens[b]`` already includes them), so one
    code path covers decode (qlen 1), chunked prefill and speculative verify (qlen K+1).
    ``softcap`` > 0 replaces the scaled scores by ``softcap * tanh(scores / softcap)`` before masking (Gemma-2)."""
    T, nh, hd = q.shape
    out = torch.zeros(T, nh, hd, dtype=torch.float32, device=q.device)
    qs = meta.query_start.tolist()
    sl = meta.seq_lens.tolist()
    for b in range(len(sl)):
        t0, t1 = qs[b], qs[b + 1]
        qlen = t1 - t0
        if qlen == 0:
            continue
        L = sl[b]
        K, V = kv_gather(kv, layer, meta.block_tables[b], L)
        nkv = K.shape[1]
        g = nh // nkv
        qb = q[t0:t1].float().reshape(qlen, nkv, g, hd)
        s = torch.einsum("qkgd,lkd->kgql", qb, K) * scale
        if softcap > 0:
            s = torch.tanh(s / softcap) * softcap
        qpos = torch.arange(L - qlen, L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        mask = kpos <= qpos
        if sliding_window > 0:
            mask &= kpos > qpos - sliding_window
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("kgql,lkd->qkgd", p, V)
        out[t0:t1] = o.reshape(qlen, nh, hd)
    return out.to(q.dtype)


def latent_attention(q: torch.Tensor, kv, layer: int, meta, scale: float, latent_dim: int) -> torch.Tensor:
    """Multi-query attention over latent cache rows (DeepSeek latent attention in absorbed form).

    q: [T, H, latent_dim + rope]; the cache holds one row of that width per token, shared by all heads, and the value of
    a row is its first ``latent_dim`` entries.  Returns [T, H, latent_dim].  A decode step (one row per sequence) is one
    batched gather + two batched matrix products over all sequences; other steps go sequence by sequence.  Device-agnostic
    torch: this is what runs on a GPU too, where the attention kernel has no 576-wide head."""
    T, H, D = q.shape
    B = int(meta.seq_lens.shape[0])
    page = kv.page_size
    quant = kv.dtype_name in ("q8", "q4")

    def rows_of(blocks: torch.Tensor) -> torch.Tensor:  # [..., nb] block ids -> [..., nb * page, D] float32 key rows
        d = kv.data[layer][blocks]  # [..., nb, 1, 2, page, D or packed]
        if quant:
            d = kv_dequantize(d, kv.scales[layer][blocks], 8 if kv.dtype_name == "q8" else 4)
        d = d[..., 0, 0, :, :].float()
        return d.reshape(*d.shape[:-3], d.shape[-3] * page, d.shape[-1])

    if T == B and meta.max_query_len == 1:
        max_len = int(meta.max_seq_len) or int(meta.seq_lens.max())
        nb = (max_len + page - 1) // page
        K = rows_of(meta.block_tables[:, :nb].long())[:, :max_len]  # [B, L, D]
        s = torch.einsum("bhd,bld->bhl", q.float(), K) * scale
        live = torch.arange(max_len, device=q.device)[None, :] < meta.seq_lens.long()[:, None]
        s = s.masked_fill(~live[:, None, :], float("-inf"))
        return torch.einsum("bhl,blc->bhc", torch.softmax(s, dim=-1), K[..., :latent_dim]).to(q.dtype)
    out = torch.zeros(T, H, latent_dim, dtype=torch.float32, device=q.device)
    qs, sl = meta.query_start.tolist(), meta.seq_lens.tolist()
    for b in range(B):
        t0, t1 = qs[b], qs[b + 1]
        n, L = t1 - t0, sl[b]
        if n == 0:
            continue
        K = rows_of(meta.block_tables[b, : (L + page - 1) // page].long())[:L]  # [L, D]
        s = torch.einsum("qhd,ld->hql", q[t0:t1].float(), K) * scale
        causal = torch.arange(L, device=q.device)[None, :] <= torch.arange(L - n, L, device=q.device)[:, None]
        s = s.masked_fill(~causal[None], float("-inf"))
        out[t0:t1] = torch.einsum("hql,lc->qhc", torch.softmax(s, dim=-1), K[:, :latent_dim])
    return out.to(q.dtype)


# --------------------------------------------------------------------------- MoE routing


def moe_route(logits: torch.Tensor, cfg, bias: Optional[torch.Tensor] = None):
    """Router: returns (expert_ids [T,k] int32, weights [T,k] float32).

    softmax → top-k → renormalise (Mixtral/Qwen), or sigmoid(+bias for *selection* only)
    → optional group-limited top-k → unbiased weights → renorm → scale (DeepSeek), as in
    ``moe_ffn_forward_weights`` (model/inference.rs:1690-1804)."""
    lf = logits.float()
    k = cfg.n_experts_used
    if cfg.expert_gating == "sigmoid":
        scores = torch.sigmoid(lf)
    else:
        scores = torch.softmax(lf, dim=-1)
    sel = scores + bias.float() if bias is not None else scores
    if cfg.expert_group_count > 1 and cfg.expert_group_used_count > 0:
        T, E = sel.shape
        gs = E // cfg.expert_group_count
        grp = sel.reshape(T, cfg.expert_group_count, gs)
        if bias is not None:
            gscore = grp.topk(min(2, gs), dim=-1).values.sum(-1)
        else:
            gscore = grp.amax(-1)
        keep = gscore.topk(cfg.expert_group_used_count, dim=-1).indices
        gmask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, keep, True)
        sel = sel.masked_fill(~gmask[:, :, None].expand(T, cfg.expert_group_count, gs).reshape(T, E), float("-inf"))
    # stable tie rule: lowest expert index first
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :k]
    w = torch.gather(scores, 1, order)
    if cfg.expert_weights_norm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    w = w * cfg.expert_weights_scale
    return order.to(torch.int32), w


# --------------------------------------------------------------------------- sampling


def argmax(logits: torch.Tensor, tie: str = "lowest") -> torch.Tensor:
    """Row argmax; ``tie='highest'`` reproduces the Rust engine's ``max_by`` (last maximal
    element, sampling.rs:236-246), ``'lowest'`` the C port's rule (cuda_fast.cu:506-513)."""
    lf = logits.float()
    if tie == "highest":
        V = lf.shape[-1]
        return (V - 1 - torch.flip(lf, dims=[-1]).argmax(-1)).to(torch.int32)
    return lf.argmax(-1).to(torch.int32)
