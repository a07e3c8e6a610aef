"""Linear layers over packed weights (Q4_K / Q6_K / Q8_0 / Q4_0 / NVFP4 GGUF blocks and
block-scaled fp8) on the GPU.

Everything goes through ``oxb_gemm_quant``.  Calls with one or two tokens take the dp4a GEMV
(``csrc/gemv_quant.cuh``: int8 activations, the packed bytes go straight into the arithmetic); larger
batches the tcgen05 GEMM whose producer warps decode the blocks into the swizzled shared-memory
operand tile.  Either way the weights are read from HBM once, in their packed form.  Formats without a
fused decoder (Q5_K, Q4_1 …), or a K that is not a multiple of 64, are decoded to a bf16 staging
buffer first.
"""
from __future__ import annotations

import torch

from . import cuda as C

FUSED_TYPES = {"Q4_K": 5, "Q6_K": 7, "Q8_0": 3, "Q4_0": 4, "NVFP4": 8}
QT_FP8B = 9


def _launch(x, data_ptr, qt, row_bytes, scales_ptr, scale_ld, out_view, bias, ld_out, N, K):
    s = C.scratch(x.device)
    C._check(C.lib().oxb_gemm_quant(x.data_ptr(), data_ptr, qt, row_bytes, scales_ptr, scale_ld, out_view.data_ptr(),
                                    C._p(bias), x.shape[0], N, K, ld_out, 0, 0, s.gemm_ws.data_ptr(),
                                    s.gemm_ws.numel() * 4, s.gemm_counters.data_ptr(), s.gemm_counters.numel(),
                                    C._stream()), "oxb_gemm_quant")
    return out_view


def linear_quant(x, p, out_view, bias, ld_out):
    n, k = p.shape
    staged_ok = C.mmq_max_tokens > 0 and x.shape[0] > C.mmq_max_tokens and n * k <= (1 << 28)
    if p.qtype in FUSED_TYPES and k % 64 == 0 and not staged_ok:
        row_bytes = p.data.stride(0) * p.data.element_size()
        return _launch(x, p.data.data_ptr(), FUSED_TYPES[p.qtype], row_bytes, None, 0, out_view, bias, ld_out, n, k)
    buf = C.scratch(x.device).dequant_buf(n * k)[: n * k].view(n, k)
    C.dequant_rows(p, buf, fast=True)
    # The GEMM requests its first weight tiles before it waits for the upstream kernel, which is only safe
    # for weights that no kernel writes.  Here the "weights" were written by the launch just before, so this
    # GEMM is launched without programmatic stream serialization (plain stream order).
    L = C.lib()
    old = L.oxb_set_pdl(0)
    try:
        C.gemm_bf16(x, buf, out_view, bias, ld_out=ld_out)
    finally:
        L.oxb_set_pdl(old)
    return out_view


def linear_fp8(x, p, out_view, bias, ld_out):
    n, k = p.shape
    if p.block != 128 or k % 128 != 0:
        raise ValueError("block-scaled fp8 weights need 128-channel blocks and K % 128 == 0")
    return _launch(x, p.data.data_ptr(), QT_FP8B, k, p.scales.data_ptr(), p.scales.shape[1], out_view, bias, ld_out, n, k)
