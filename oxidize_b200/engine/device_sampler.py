"""Batched sampler operating on device logits with per-row knobs and host-supplied uniforms.

Row r draws with ``temperature[r]`` (0 = greedy), ``top_k[r]`` (0 = off), ``top_p[r]``,
``min_p[r]`` and the uniform ``random[r]`` using the same order of filters as the host oracle
(:func:`oxidize_b200.engine.sampler.sample`): softmax over the full vocabulary, sort
descending, top-k, top-p, min-p, inverse CDF with ``target = random * sum(kept)``.  On CUDA
the work is done by the sm_100a sampling kernels; on CPU by the torch statement below.
"""
from __future__ import annotations

import torch

from .. import ops


def sample_torch(logits, temperature, top_k, top_p, min_p, random, tie="lowest"):
    lf = logits.float()
    R, V = lf.shape
    greedy = ops.ref.argmax(lf, tie).long()
    t = temperature.float().clamp_min(1e-6)[:, None]
    probs = torch.softmax((lf - lf.amax(-1, keepdim=True)) / t, dim=-1)
    sp, order = torch.sort(probs, dim=-1, descending=True, stable=True)
    rank = torch.arange(V, device=lf.device)[None, :]
    keep = torch.ones_like(sp, dtype=torch.bool)
    k = top_k.long()[:, None]
    keep &= (k <= 0) | (rank < k)
    csum = torch.cumsum(sp, dim=-1)
    # keep through the first index whose cumulative mass reaches top_p
    keep &= (csum - sp) < top_p.float()[:, None]
    keep &= sp >= min_p.float()[:, None] * sp[:, :1]
    keep[:, 0] = True
    kept = sp * keep
    c = torch.cumsum(kept, dim=-1)
    target = random.float()[:, None] * c[:, -1:]
    j = torch.searchsorted(c, target, right=True).clamp_max(V - 1)
    # never land on a filtered slot
    nkeep = keep.sum(-1, keepdim=True)
    j = torch.minimum(j, nkeep - 1)
    tok = torch.gather(order, 1, j).squeeze(1)
    return torch.where(temperature <= 0, greedy, tok).to(torch.int32)


def sample(logits, temperature, top_k, top_p, min_p, random, tie="lowest"):
    if logits.is_cuda:
        from ..ops import cuda as opcuda

        return opcuda.sample(logits, temperature, top_k, top_p, min_p, random, tie)
    return sample_torch(logits, temperature, top_k, top_p, min_p, random, tie)
