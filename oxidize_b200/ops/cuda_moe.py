"""Mixture-of-experts on the GPU: device routing, grouped expert GEMMs, fused combine.

Up to 256 tokens per call (decode, speculative verify, small prefill chunks) the whole layer is
five launches and needs no host round trip, so it can sit inside a CUDA graph:

    moe_route_kernel      router logits → (ids, weights) + per-local-expert weight rows
    gemm_grouped          x → gate_up of ALL local experts (idle experts skipped on the device)
    silu_mul              over the stacked [E*T, 2F] activations
    gemm_grouped          per-expert down projection
    moe_combine_kernel    Σ_e scale[e, t] · y[e, t]  (+ shared expert)

Larger calls (long prefill chunks) gather each expert's rows and run ordinary GEMMs, which avoids
multiplying every token with every local expert.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import cuda as C

GROUPED_MAX_TOKENS = 256


def _declare(L):
    import ctypes

    if getattr(L, "_moe_declared", False):
        return
    vp, i32, f32, sz, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_longlong
    L.oxb_moe_route.argtypes = [vp, i32, i32, i32, i32, i32, vp, i32, f32, vp, vp, vp, i32, i32, i32, i32, i32, vp]
    L.oxb_moe_combine.argtypes = [vp, vp, i32, vp, vp, i32, i32, i32, vp]
    L.oxb_gemm_grouped.argtypes = [vp, i32, vp, i32, sz, vp, ll, vp, i32, i32, i32, i32, i32, i32, vp, sz, vp, i32, vp]
    L._moe_declared = True


def moe_route(logits: torch.Tensor, cfg, bias: Optional[torch.Tensor] = None, scale_out: Optional[torch.Tensor] = None,
              first_local: int = 0, n_local: int = 0):
    """(ids [T,k] int32, weights [T,k] f32); shapes beyond the kernel's limits use the torch statement
    (no host synchronisation either way, so both can be captured in a CUDA graph)."""
    grouped = cfg.expert_group_count > 1 and cfg.expert_group_used_count > 0
    if (cfg.n_experts > 256 or cfg.n_experts_used > 16
            or grouped and (cfg.expert_group_count > 32 or cfg.n_experts % cfg.expert_group_count)):
        from . import ref

        ids, w = ref.moe_route(logits, cfg, bias)
        if scale_out is not None:
            T = ids.shape[0]
            full = torch.zeros(T, cfg.n_experts, dtype=torch.float32, device=ids.device)
            full.scatter_add_(1, ids.long(), w.float())
            scale_out[:, :T].copy_(full[:, first_local:first_local + n_local].t())
        return ids, w
    L = C.lib()
    _declare(L)
    logits = logits.float().contiguous()
    T, E = logits.shape
    k = cfg.n_experts_used
    ids = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    C._check(L.oxb_moe_route(logits.data_ptr(), T, E, logits.stride(0), k, 1 if cfg.expert_gating == "sigmoid" else 0,
                             C._p(bias), 1 if cfg.expert_weights_norm else 0, float(cfg.expert_weights_scale),
                             ids.data_ptr(), w.data_ptr(), C._p(scale_out),
                             0 if scale_out is None else scale_out.stride(0), first_local, n_local,
                             cfg.expert_group_count if grouped else 1, cfg.expert_group_used_count if grouped else 0,
                             C._stream()),
             "oxb_moe_route")
    return ids, w


def gemm_grouped(x: torch.Tensor, x_rows: int, w, groups: int, T: int, scale: Optional[torch.Tensor]) -> torch.Tensor:
    """y[g] = x_g @ W_g^T for the stacked weight ``w`` ([(groups*N), K]); returns [groups, T, N] bf16."""
    L = C.lib()
    _declare(L)
    N = w.shape[0] // groups
    K = w.shape[1]
    y = torch.empty(groups, T, N, dtype=torch.bfloat16, device=x.device)
    s = C.scratch(x.device)
    qt = C.QTYPE_CODE[w.qtype]
    row_bytes = w.data.stride(0) * w.data.element_size()
    C._check(L.oxb_gemm_grouped(x.data_ptr(), x_rows, w.data.data_ptr(), qt, row_bytes, y.data_ptr(), T * N, C._p(scale),
                                0 if scale is None else scale.stride(0), groups, T, N, K, N, s.gemm_ws.data_ptr(),
                                s.gemm_ws.numel() * 4, s.gemm_counters.data_ptr(), s.gemm_counters.numel(), C._stream()),
             "oxb_gemm_grouped")
    return y


def moe_combine(y: torch.Tensor, scale: torch.Tensor, shared: Optional[torch.Tensor]) -> torch.Tensor:
    L = C.lib()
    _declare(L)
    E, T, H = y.shape
    out = torch.empty(T, H, dtype=torch.bfloat16, device=y.device)
    C._check(L.oxb_moe_combine(y.data_ptr(), scale.data_ptr(), scale.stride(0), C._p(shared), out.data_ptr(), E, T, H,
                               C._stream()), "oxb_moe_combine")
    return out


def moe_layer(x: torch.Tensor, router_logits: torch.Tensor, cfg, router_bias, experts,
              shared: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Whole routed-expert block for the experts held locally (+ optional shared-expert output)."""
    T = x.shape[0]
    E = len(experts.gate_up)
    if T <= GROUPED_MAX_TOKENS and experts.stack() and experts.gate_up_stack.shape[1] % 64 == 0 \
            and experts.down_stack.shape[1] % 64 == 0:
        scale = torch.empty(E, max(T, 1), dtype=torch.float32, device=x.device)
        moe_route(router_logits, cfg, router_bias, scale, experts.first_expert, E)
        x = x.contiguous()
        h = gemm_grouped(x, 0, experts.gate_up_stack, E, T, scale)  # [E, T, 2F]
        act = C.silu_mul(h.view(E * T, -1))  # [E*T, F]
        y = gemm_grouped(act, T, experts.down_stack, E, T, scale)  # [E, T, H]
        return moe_combine(y, scale, shared)
    ids, wts = moe_route(router_logits, cfg, router_bias)
    out = moe_experts_forward(x, ids, wts, experts)
    return out if shared is None else out + shared


def moe_experts_forward(x, ids, wts, experts):
    """Gather path: each local expert runs on the rows routed to it (host-visible row counts)."""
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    for le in range(len(experts.gate_up)):
        e = experts.first_expert + le
        sel = ids == e
        rows = sel.any(dim=1).nonzero(as_tuple=True)[0]
        if rows.numel() == 0:
            continue
        w = (wts * sel).sum(dim=1)[rows]
        xe = x.index_select(0, rows)
        y = C.linear(C.silu_mul(C.linear(xe, [experts.gate_up[le]])), [experts.down[le]])
        out.index_add_(0, rows, y.float() * w[:, None])
    return out.to(x.dtype)
