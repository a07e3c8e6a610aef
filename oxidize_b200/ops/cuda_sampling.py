"""Device sampling entry point for CUDA logits (``sample_kernel``; there is no host or torch fallback)."""
from __future__ import annotations

import torch

from . import cuda as C


def sample(logits, temperature, top_k, top_p, min_p, random, tie="lowest"):
    L = C.lib()
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    C._check(L.oxb_sample(logits.data_ptr(), R, V, logits.stride(0), temperature.data_ptr(), top_k.data_ptr(),
                          top_p.data_ptr(), min_p.data_ptr(), random.data_ptr(), 1 if tie == "highest" else 0,
                          out.data_ptr(), C._stream()), "oxb_sample")
    return out
