"""Mixture-of-experts on the GPU: device routing, token dispatch, grouped expert GEMMs, fused combine.

The whole layer runs on the device for any token count (no host round trip, so it sits inside CUDA graphs), and
every local expert multiplies exactly the tokens routed to it:

    moe_route_kernel            router logits → (ids, weights)
    moe_permute_kernel          per-local-expert token lists: row offsets, permutation, inverse map
    moe_gather_kernel           rows gathered expert by expert
    gemm_grouped_rows           gate_up of every local expert over its own rows (tcgen05, one launch)
    silu_mul_rows
    gemm_grouped_rows           down projection, same rows
    moe_combine_(exchange)      Σ_k w[t, k] · y[row(t, k)] (+ shared expert); with expert parallelism the all-reduce
                                over the ranks happens inside the same kernel, over NVLink peer memory

The older dense formulation (every active local expert multiplies all tokens, ``gemm_grouped`` + per-expert weight
rows) is kept for A/B measurements (``moe_layer(..., gathered=False)``).
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
    L.oxb_moe_permute.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    L.oxb_moe_gather.argtypes = [vp, i32, vp, vp, i32, vp, vp]
    L.oxb_silu_mul_rows.argtypes = [vp, vp, vp, i32, i32, vp]
    L.oxb_gemm_grouped_rows.argtypes = [vp, i32, vp, i32, sz, vp, vp, i32, i32, i32, i32, i32, vp]
    u64p = ctypes.POINTER(ctypes.c_uint64)
    L.oxb_moe_combine_gathered.argtypes = [vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, u64p, u64p, vp, i32, i32, i32,
                                           ctypes.c_ulonglong, vp]
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


def gemm_grouped_rows(xg: torch.Tensor, w, offsets: torch.Tensor, groups: int, max_rows: int) -> torch.Tensor:
    """y[r] = xg[r] @ W_g^T for every gathered row r of group g (rows [offsets[g], offsets[g+1])); [rows_cap, N] bf16."""
    L = C.lib()
    _declare(L)
    N = w.shape[0] // groups
    K = w.shape[1]
    y = torch.empty(xg.shape[0], N, dtype=torch.bfloat16, device=xg.device)
    row_bytes = w.data.stride(0) * w.data.element_size()
    C._check(L.oxb_gemm_grouped_rows(xg.data_ptr(), xg.shape[0], w.data.data_ptr(), C.QTYPE_CODE[w.qtype], row_bytes,
                                     y.data_ptr(), offsets.data_ptr(), groups, max_rows, N, K, N, C._stream()),
             "oxb_gemm_grouped_rows")
    return y


def moe_dispatch(ids: torch.Tensor, first_local: int, n_local: int):
    """Token lists of the local experts: (offsets [n_local+1], perm [T*k], inv [T, k]) int32, built on the device."""
    L = C.lib()
    _declare(L)
    T, k = ids.shape
    dev = ids.device
    offsets = torch.empty(n_local + 1, dtype=torch.int32, device=dev)
    perm = torch.empty(T * k, dtype=torch.int32, device=dev)
    inv = torch.empty(T, k, dtype=torch.int32, device=dev)
    C._check(L.oxb_moe_permute(ids.data_ptr(), T, k, first_local, n_local, offsets.data_ptr(), perm.data_ptr(),
                               inv.data_ptr(), C._stream()), "oxb_moe_permute")
    return offsets, perm, inv


def moe_combine_gathered(y: torch.Tensor, inv: torch.Tensor, wts: torch.Tensor, shared: Optional[torch.Tensor], T: int,
                         comm=None):
    """out[t] = Σ_k w[t,k] · y[inv[t,k]] (+ shared).  With ``comm`` (a FusedComm whose buffers hold T tokens) the partial
    sums of the expert-parallel ranks are all-reduced inside the same kernel; returns (out, reduced)."""
    L = C.lib()
    _declare(L)
    H = y.shape[1]
    k = inv.shape[1]
    out = torch.empty(T, H, dtype=torch.bfloat16, device=y.device)
    fused = (comm is not None and getattr(comm, "size", 1) > 1 and hasattr(comm, "_data_ptrs") and T <= comm.t_max
             and H <= comm.n_max and H % 8 == 0 and ((H + 127) // 128) * ((T + 15) // 16) <= C.sm_count(y.device) * 8
             and comm.size >= L.oxb_set_ar_ll_min_world(-1))
    if fused:
        import ctypes

        C._check(L.oxb_moe_combine_gathered(y.data_ptr(), inv.data_ptr(), wts.data_ptr(), k, C._p(shared), out.data_ptr(), T, H,
                                            comm.size, comm.rank, comm._data_ptrs, comm._flag_ptrs, comm.ctrl.data_ptr(),
                                            comm.t_max, comm.n_max, comm.max_tiles, ctypes.c_ulonglong(comm.timeout_ns),
                                            C._stream()), "oxb_moe_combine_gathered")
        comm.fused_calls += 1
        return out, True
    C._check(L.oxb_moe_combine_gathered(y.data_ptr(), inv.data_ptr(), wts.data_ptr(), k, C._p(shared), out.data_ptr(), T, H,
                                        1, 0, None, None, None, 0, 0, 0, 0, C._stream()), "oxb_moe_combine_gathered")
    return out, False


MAX_DISPATCH_ENTRIES = 1 << 17  # token x top-k entries one permute launch (a single CTA) is asked to place


def moe_layer(x: torch.Tensor, router_logits: torch.Tensor, cfg, router_bias, experts,
              shared: Optional[torch.Tensor] = None, comm=None, gathered: bool = True):
    """Whole routed-expert block for the experts held locally (+ optional shared-expert output).
    Returns (out, reduced): ``reduced`` says that the expert-parallel all-reduce already happened (fused combine)."""
    T = x.shape[0]
    E = len(experts.gate_up)
    k = cfg.n_experts_used
    stacked = experts.stack() and experts.gate_up_stack.shape[1] % 64 == 0 and experts.down_stack.shape[1] % 64 == 0
    kernel_route = cfg.n_experts <= 256 and k <= 16
    if gathered and stacked and kernel_route and T * k <= MAX_DISPATCH_ENTRIES and x.shape[1] % 8 == 0:
        L = C.lib()
        ids, wts = moe_route(router_logits, cfg, router_bias)
        offsets, perm, inv = moe_dispatch(ids, experts.first_expert, E)
        n_rows = offsets[E:]
        x = x.contiguous()
        xg = torch.empty(T * k, x.shape[1], dtype=torch.bfloat16, device=x.device)
        C._check(L.oxb_moe_gather(x.data_ptr(), x.shape[1], perm.data_ptr(), n_rows.data_ptr(), T * k, xg.data_ptr(),
                                  C._stream()), "oxb_moe_gather")
        h = gemm_grouped_rows(xg, experts.gate_up_stack, offsets, E, T)  # [T*k, 2F]
        F = h.shape[1] // 2
        act = torch.empty(T * k, F, dtype=torch.bfloat16, device=x.device)
        C._check(L.oxb_silu_mul_rows(h.data_ptr(), act.data_ptr(), n_rows.data_ptr(), T * k, F, C._stream()),
                 "oxb_silu_mul_rows")
        y = gemm_grouped_rows(act, experts.down_stack, offsets, E, T)  # [T*k, H]
        return moe_combine_gathered(y, inv, wts, shared, T, comm)
    # the dense form runs one token tile per expert: 256 tokens with bf16 experts, 128 with packed ones
    if stacked and T <= (GROUPED_MAX_TOKENS if experts.gate_up_stack.qtype == "BF16" else GROUPED_MAX_TOKENS // 2):
        scale = torch.empty(E, max(T, 1), dtype=torch.float32, device=x.device)
        moe_route(router_logits, cfg, router_bias, scale, experts.first_expert, E)
        x = x.contiguous()
        h = gemm_grouped(x, 0, experts.gate_up_stack, E, T, scale)  # [E, T, 2F]
        act = C.silu_mul(h.view(E * T, -1))  # [E*T, F]
        y = gemm_grouped(act, T, experts.down_stack, E, T, scale)  # [E, T, H]
        return moe_combine(y, scale, shared), False
    ids, wts = moe_route(router_logits, cfg, router_bias)
    out = moe_experts_forward(x, ids, wts, experts)
    return (out if shared is None else out + shared), False


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
