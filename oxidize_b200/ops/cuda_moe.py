"""Mixture-of-experts routing and expert FFN on the GPU."""
from __future__ import annotations

import torch

from . import cuda as C
from . import ref


def moe_route(logits, cfg, bias=None):
    return ref.moe_route(logits, cfg, bias)


def moe_experts_forward(x, ids, wts, experts):
    """Local experts on the rows routed to them, weighted sum into the output."""
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
