"""Block quantizers written with torch ops so that large random-init models can be encoded
on the device they will run on (a 70B-shape Q4_K model never exists as floats on the host).

Same block layouts as :mod:`oxidize_b200.quant.ref`; the NumPy decoders there remain the
oracle (tests decode these encoders' output with them).
"""
from __future__ import annotations

import torch

from ..formats.gguf import ggml_type


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2) if x.dim() else x


def _safe_inv(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 0, 1.0 / torch.where(x > 0, x, torch.ones_like(x)), torch.zeros_like(x))


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    xb = x.float().reshape(-1, 32)
    d = xb.abs().amax(1, keepdim=True) / 127.0
    q = torch.round(xb * _safe_inv(d)).clamp(-127, 127).to(torch.int8)
    out = torch.empty(xb.shape[0], 34, dtype=torch.uint8, device=x.device)
    out[:, :2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(torch.uint8)
    return out


def _pack_scales_k4(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    sc = sc.to(torch.uint8)
    mn = mn.to(torch.uint8)
    out = torch.zeros(sc.shape[0], 12, dtype=torch.uint8, device=sc.device)
    out[:, 0:4] = (sc[:, :4] & 63) | ((sc[:, 4:] >> 4) << 6)
    out[:, 4:8] = (mn[:, :4] & 63) | ((mn[:, 4:] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:] & 0xF) | ((mn[:, 4:] & 0xF) << 4)
    return out


def quantize_q4_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.float().reshape(-1, 8, 32)
    lo = xb.amin(-1).clamp_max(0.0)
    hi = xb.amax(-1)
    scale = (hi - lo) / 15.0
    mn = -lo
    d = (scale.amax(1, keepdim=True) / 63.0).to(torch.float16).float()
    dmin = (mn.amax(1, keepdim=True) / 63.0).to(torch.float16).float()
    sc = torch.round(scale * _safe_inv(d)).clamp(0, 63)
    mq = torch.round(mn * _safe_inv(dmin)).clamp(0, 63)
    eff = (d * sc).unsqueeze(-1)
    effm = (dmin * mq).unsqueeze(-1)
    q = torch.round((xb + effm) * _safe_inv(eff)).clamp(0, 15).to(torch.uint8).reshape(-1, 4, 2, 32)
    out = torch.empty(xb.shape[0], 144, dtype=torch.uint8, device=x.device)
    out[:, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 4:16] = _pack_scales_k4(sc, mq)
    out[:, 16:] = (q[:, :, 0] | (q[:, :, 1] << 4)).reshape(-1, 128)
    return out


def quantize_q6_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.float().reshape(-1, 16, 16)
    amax = xb.abs().amax(2)
    sub = amax / 31.0
    d = (sub.amax(1, keepdim=True) / 127.0).to(torch.float16).float()
    sc = torch.round(sub * _safe_inv(d)).clamp(-128, 127)
    sc = torch.where((sc == 0) & (amax > 0), torch.ones_like(sc), sc)
    eff = (d * sc).unsqueeze(-1)
    inv = torch.where(eff != 0, 1.0 / torch.where(eff != 0, eff, torch.ones_like(eff)), torch.zeros_like(eff))
    q = (torch.round(xb * inv).clamp(-32, 31) + 32).to(torch.uint8).reshape(-1, 2, 4, 32)
    lo, hi = q & 0xF, q >> 4
    out = torch.empty(xb.shape[0], 210, dtype=torch.uint8, device=x.device)
    ql = torch.empty(xb.shape[0], 2, 64, dtype=torch.uint8, device=x.device)
    ql[:, :, :32] = lo[:, :, 0] | (lo[:, :, 2] << 4)
    ql[:, :, 32:] = lo[:, :, 1] | (lo[:, :, 3] << 4)
    qh = hi[:, :, 0] | (hi[:, :, 1] << 2) | (hi[:, :, 2] << 4) | (hi[:, :, 3] << 6)
    out[:, 0:128] = ql.reshape(-1, 128)
    out[:, 128:192] = qh.reshape(-1, 64)
    out[:, 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[:, 208:210] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    return out


_E2M1_POS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e4m3_encode_pos(x: torch.Tensor) -> torch.Tensor:
    """positive f32 -> e4m3 magnitude byte via torch's float8 cast (round-to-nearest-even)."""
    return x.clamp(0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8) & 0x7F


def quantize_nvfp4(x: torch.Tensor) -> torch.Tensor:
    xb = x.float().reshape(-1, 4, 16)
    amax = xb.abs().amax(2, keepdim=True)
    sb = _e4m3_encode_pos(amax / 6.0)
    s_dec = sb.view(torch.float8_e4m3fn).float()
    bump = (s_dec * 6.0 < amax) & (sb < 0x7E)
    sb = torch.where(bump, sb + 1, sb).to(torch.uint8)
    s_dec = sb.view(torch.float8_e4m3fn).float()
    y = xb * _safe_inv(s_dec)
    grid = torch.tensor(_E2M1_POS, device=x.device)
    code = (y.abs().unsqueeze(-1) - grid).abs().argmin(-1).to(torch.uint8)
    code = code | ((y < 0) | ((y == 0) & torch.signbit(y))).to(torch.uint8) << 3
    out = torch.empty(xb.shape[0], 36, dtype=torch.uint8, device=x.device)
    out[:, 0:4] = sb.reshape(-1, 4)
    out[:, 4:] = (code[:, :, :8] | (code[:, :, 8:] << 4)).reshape(-1, 32)
    return out


_ENC = {"Q8_0": quantize_q8_0, "Q4_K": quantize_q4_k, "Q6_K": quantize_q6_k, "NVFP4": quantize_nvfp4}


def quantize(qtype: str, w: torch.Tensor) -> torch.Tensor:
    """dense [out, in] -> uint8 [out, row_bytes]."""
    qtype = qtype.upper()
    if qtype not in _ENC:
        raise ValueError(f"no torch encoder for {qtype}")
    t = ggml_type(qtype)
    out_f, in_f = w.shape
    if in_f % t.block_size:
        raise ValueError(f"{qtype}: in_features {in_f} not a multiple of {t.block_size}")
    return _ENC[qtype](w.reshape(-1)).reshape(out_f, in_f // t.block_size * t.type_size)


def quantize_fp8_block(w: torch.Tensor, block: int = 128):
    out_f, in_f = w.shape
    xb = w.float().reshape(out_f, in_f // block, block)
    amax = xb.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    codes = (xb / scale).to(torch.float8_e4m3fn).view(torch.uint8).reshape(out_f, in_f)
    return codes, scale.squeeze(-1).contiguous()


def random_quantized(out_f: int, in_f: int, qtype: str, device, gen: torch.Generator, std: float):
    """N(0, std) weight encoded as ``qtype``, generated and encoded in row chunks on ``device``."""
    from ..models.weights import QTensor

    qtype = qtype.upper()
    step = max(1, (1 << 26) // max(in_f, 1))
    if qtype == "FP8B":
        codes = torch.empty(out_f, in_f, dtype=torch.uint8, device=device)
        scales = torch.empty(out_f, in_f // 128, dtype=torch.float32, device=device)
        for r in range(0, out_f, step):
            w = torch.empty(min(step, out_f - r), in_f, device=device).normal_(0.0, std, generator=gen)
            codes[r : r + step], scales[r : r + step] = quantize_fp8_block(w)
        return QTensor("FP8B", codes, (out_f, in_f), scales, 128)
    t = ggml_type(qtype)
    data = torch.empty(out_f, in_f // t.block_size * t.type_size, dtype=torch.uint8, device=device)
    for r in range(0, out_f, step):
        w = torch.empty(min(step, out_f - r), in_f, device=device).normal_(0.0, std, generator=gen)
        data[r : r + step] = quantize(qtype, w)
    return QTensor(t.name, data, (out_f, in_f))
