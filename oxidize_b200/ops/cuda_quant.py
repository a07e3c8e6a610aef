"""Linear layers over block-quantized weights on the GPU.

Small batches (the bandwidth-bound decode regime) run the fused dequant GEMV kernels that read
the packed blocks once; larger batches decode the blocks to a bf16 staging buffer and run the
tcgen05 GEMM on it.
"""
from __future__ import annotations

import torch

from . import cuda as C

GEMV_MAX_TOKENS = 8


def linear_quant(x, p, out_view, bias, ld_out):
    T = x.shape[0]
    if T <= GEMV_MAX_TOKENS and hasattr(C.lib(), "oxb_gemv_quant") and C.QTYPE_CODE.get(p.qtype) is not None:
        row_bytes = p.data.stride(0) * p.data.element_size()
        C._check(C.lib().oxb_gemv_quant(x.data_ptr(), p.data.data_ptr(), C.QTYPE_CODE[p.qtype], row_bytes,
                                        out_view.data_ptr(), C._p(bias), T, p.shape[0], p.shape[1], ld_out,
                                        C._stream()), "oxb_gemv_quant")
        return out_view
    n, k = p.shape
    buf = C.scratch(x.device).dequant_buf(n * k)[: n * k].view(n, k)
    C.dequant_rows(p, buf)
    C.gemm_bf16(x, buf, out_view, bias, ld_out=ld_out)
    return out_view


def linear_fp8(x, p, out_view, bias, ld_out):
    raise NotImplementedError("block-scaled fp8 linear is not built yet")
