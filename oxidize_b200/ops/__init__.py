"""Operator front door.

CPU tensors run the plain-PyTorch statements in :mod:`oxidize_b200.ops.ref` (the oracle and
the no-GPU execution path).  CUDA tensors always run the hand-written sm_100a kernels in
:mod:`oxidize_b200.ops.cuda`; there is no silent fallback — if the native library is missing
on a GPU machine the call raises.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ref
from ..utils.profiler import instrument


def _cuda():
    from . import cuda as _c

    return _c


@instrument("linear")
def linear(x: torch.Tensor, w, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ W^T (+bias) for a :class:`LinearWeight` (row segments concatenated) or a QTensor."""
    parts = getattr(w, "parts", None)
    if parts is None:
        parts = [w]
    else:
        bias = w.bias if bias is None else bias
    if x.is_cuda:
        return _cuda().linear(x, parts, bias, out)
    ys = [ref.linear(x, p) for p in parts]
    y = ys[0] if len(ys) == 1 else torch.cat(ys, dim=-1)
    if bias is not None:
        y = (y.float() + bias.float()).to(y.dtype)
    return y


@instrument("embed")
def embed(tokens: torch.Tensor, table, dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    if tokens.is_cuda:
        return _cuda().embed(tokens, table, dtype, scale)
    return ref.embed(tokens, table, scale).to(dtype)


@instrument("rmsnorm")
def rmsnorm(x, w, eps):
    if x.is_cuda:
        return _cuda().add_rmsnorm(x, None, w, eps)[0]
    return ref.rmsnorm(x, w, eps)


@instrument("add_rmsnorm")
def add_rmsnorm(x, residual, w, eps):
    if x.is_cuda:
        return _cuda().add_rmsnorm(x, residual, w, eps)
    return ref.add_rmsnorm(x, residual, w, eps)


@instrument("silu_mul")
def silu_mul(gate_up):
    if gate_up.is_cuda:
        return _cuda().silu_mul(gate_up)
    return ref.silu_mul(gate_up)


@instrument("gelu_mul")
def gelu_mul(gate_up):
    """tanh-GELU(gate) * up on the halves of a fused [T, 2F] projection (GeGLU)."""
    if gate_up.is_cuda:
        return _cuda().gelu_mul(gate_up)
    return ref.gelu_mul(gate_up)


@instrument("qk_rope_kv_write")
def qk_rope_kv_write(qkv, positions, slot_mapping, kv, layer, rope, q_norm=None, k_norm=None, eps=1e-6, norm_after=False):
    """Split fused qkv [T, (nq+2nkv)*hd], optional per-head QK RMSNorm, RoPE on q and k,
    write K/V into the paged cache.  Returns rotated q as [T, nq, hd].  ``norm_after``: the norms act on the rotated
    vectors (Hunyuan); that order runs as torch operations on either device."""
    norm_after = norm_after and q_norm is not None
    if qkv.is_cuda and not norm_after:
        return _cuda().qk_rope_kv_write(qkv, positions, slot_mapping, kv, layer, rope, q_norm, k_norm, eps)
    nq, nkv, hd = rope.n_heads, rope.n_kv_heads, rope.head_dim
    T = qkv.shape[0]
    q = qkv[:, : nq * hd].reshape(T, nq, hd)
    k = qkv[:, nq * hd : (nq + nkv) * hd].reshape(T, nkv, hd)
    v = qkv[:, (nq + nkv) * hd :].reshape(T, nkv, hd)
    if q_norm is not None and not norm_after:
        q = ref.rmsnorm(q, q_norm, eps)
        k = ref.rmsnorm(k, k_norm, eps)
    q = ref.apply_rope(q, positions, rope.inv_freq, rope.pairing, rope.mscale)
    k = ref.apply_rope(k, positions, rope.inv_freq, rope.pairing, rope.mscale)
    if norm_after:
        q = ref.rmsnorm(q, q_norm, eps).to(qkv.dtype)
        k = ref.rmsnorm(k, k_norm, eps).to(qkv.dtype)
    ref.kv_write(kv, layer, k, v, slot_mapping)
    return q


@instrument("paged_attention")
def paged_attention(q, kv, layer, meta, scale, sliding_window=0, softcap=0.0):
    if q.is_cuda:
        return _cuda().paged_attention(q, kv, layer, meta, scale, sliding_window, softcap=softcap)
    return ref.paged_attention(q, kv, layer, meta, scale, sliding_window, softcap)


@instrument("moe_route")
def moe_route(logits, cfg, bias=None):
    if logits.is_cuda:
        return _cuda().moe_route(logits, cfg, bias)
    return ref.moe_route(logits, cfg, bias)


@instrument("argmax")
def argmax(logits, tie="lowest"):
    if logits.is_cuda:
        return _cuda().argmax(logits, tie)
    return ref.argmax(logits, tie)
