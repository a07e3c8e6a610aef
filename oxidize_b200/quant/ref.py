"""NumPy reference (de)quantizers for the GGUF block formats: the oracle for every kernel.

Block layouts are the ggml ones listed in ``oxidize-core/src/compute/quantization.rs:5-53,241-281``
(Q4_K 144 B / 256 values, Q6_K 210 B, Q8_0 34 B / 32, Q8_K 292 B, NVFP4 36 B / 64).  The decoders
restate the scalar math of ``quant_k_blocks.rs:596`` (Q4_K), ``:682`` (Q6_K) and
``quant_nvfp4.rs:14-41`` (NVFP4) in vectorised form; the encoders are our own (a weighted
least-squares refinement rather than llama.cpp's ``make_qkx1`` search) because only the *decoder*
is part of the file-format contract.

All functions take/return flat arrays: ``dequantize(type, raw_uint8, n)`` → float32[n];
``quantize(type, float32[n])`` → uint8 block bytes.
"""
from __future__ import annotations

from typing import Callable, Dict

import numpy as np

from ..formats.gguf import GGUFError, ggml_type

QK_K = 256

# E2M1 code -> value, doubled (0, .5, 1, 1.5, 2, 3, 4, 6 times two), as the reference keeps
# it (compute/quantization.rs:128-130); the ue4m3 scale decode carries the matching 0.5.
E2M1_DOUBLED = np.array([0, 1, 2, 3, 4, 6, 8, 12, -0.0, -1, -2, -3, -4, -6, -8, -12], dtype=np.float32)
IQ4NL_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def _f16(raw: np.ndarray) -> np.ndarray:
    return raw.view("<f2").astype(np.float32)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit pattern (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (0x7FFF + ((u >> 16) & 1))
    out = (rounded >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


# --------------------------------------------------------------------------- legacy 32-blocks


def dequantize_q8_0(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 34)
    d = _f16(b[:, :2].copy()).reshape(-1, 1)
    q = b[:, 2:].view(np.int8).astype(np.float32)
    return (d * q).reshape(-1)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(xb).max(axis=1, keepdims=True)
    d = amax / 127.0
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0)
    q = np.rint(xb * inv).clip(-127, 127).astype(np.int8)
    out = np.empty((xb.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype("<f2").view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def dequantize_q4_0(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 18)
    d = _f16(b[:, :2].copy()).reshape(-1, 1)
    qs = b[:, 2:]
    lo = (qs & 0xF).astype(np.float32) - 8
    hi = (qs >> 4).astype(np.float32) - 8
    return (d * np.concatenate([lo, hi], axis=1)).reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 32)
    idx = np.abs(xb).argmax(axis=1)
    mx = xb[np.arange(xb.shape[0]), idx].reshape(-1, 1)
    d = mx / -8.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0)
    q = np.clip(np.floor(xb * inv + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((xb.shape[0], 18), dtype=np.uint8)
    out[:, :2] = d.astype("<f2").view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def dequantize_q4_1(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 20)
    d = _f16(b[:, 0:2].copy()).reshape(-1, 1)
    m = _f16(b[:, 2:4].copy()).reshape(-1, 1)
    qs = b[:, 4:]
    q = np.concatenate([qs & 0xF, qs >> 4], axis=1).astype(np.float32)
    return (d * q + m).reshape(-1)


def _q5_high_bits(qh_bytes: np.ndarray) -> np.ndarray:
    qh = qh_bytes.copy().view("<u4").reshape(-1, 1)
    return ((qh >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8)


def dequantize_q5_0(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 22)
    d = _f16(b[:, 0:2].copy()).reshape(-1, 1)
    hb = _q5_high_bits(b[:, 2:6])
    qs = b[:, 6:]
    q = np.concatenate([qs & 0xF, qs >> 4], axis=1) | (hb << 4)
    return (d * (q.astype(np.float32) - 16)).reshape(-1)


def dequantize_q5_1(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 24)
    d = _f16(b[:, 0:2].copy()).reshape(-1, 1)
    m = _f16(b[:, 2:4].copy()).reshape(-1, 1)
    hb = _q5_high_bits(b[:, 4:8])
    qs = b[:, 8:]
    q = np.concatenate([qs & 0xF, qs >> 4], axis=1) | (hb << 4)
    return (d * q.astype(np.float32) + m).reshape(-1)


def quantize_q5_0(x: np.ndarray) -> np.ndarray:
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 32)
    idx = np.abs(xb).argmax(axis=1)
    mx = xb[np.arange(xb.shape[0]), idx].reshape(-1, 1)
    d = mx / -16.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0)
    q = np.clip(np.floor(xb * inv + 16.5), 0, 31).astype(np.uint32)
    out = np.empty((xb.shape[0], 22), dtype=np.uint8)
    out[:, :2] = d.astype("<f2").view(np.uint8).reshape(-1, 2)
    qh = (((q >> 4) & 1) << np.arange(32, dtype=np.uint32)).sum(axis=1).astype("<u4")
    out[:, 2:6] = qh.view(np.uint8).reshape(-1, 4)
    lo = (q & 0xF).astype(np.uint8)
    out[:, 6:] = lo[:, :16] | (lo[:, 16:] << 4)
    return out.reshape(-1)


# --------------------------------------------------------------------------- k-quants


def unpack_scales_k4(sc12: np.ndarray):
    """12 packed bytes -> (8 six-bit scales, 8 six-bit mins); ``get_scale_min_k4``
    (reference: kernels/gemv_f32.cu:240-250)."""
    s = sc12.reshape(-1, 12).astype(np.uint8)
    sc = np.empty((s.shape[0], 8), dtype=np.uint8)
    mn = np.empty((s.shape[0], 8), dtype=np.uint8)
    sc[:, :4] = s[:, 0:4] & 63
    mn[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, mn


def pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.zeros((sc.shape[0], 12), dtype=np.uint8)
    out[:, 0:4] = (sc[:, :4] & 63) | ((sc[:, 4:] >> 4) << 6)
    out[:, 4:8] = (mn[:, :4] & 63) | ((mn[:, 4:] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:] & 0xF) | ((mn[:, 4:] & 0xF) << 4)
    return out


def dequantize_q4_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 144)
    d = _f16(b[:, 0:2].copy()).reshape(-1, 1)
    dmin = _f16(b[:, 2:4].copy()).reshape(-1, 1)
    sc, mn = unpack_scales_k4(b[:, 4:16])
    qs = b[:, 16:].reshape(-1, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)
    scale = (d * sc.astype(np.float32)).reshape(-1, 8, 1)
    minv = (dmin * mn.astype(np.float32)).reshape(-1, 8, 1)
    return (scale * q - minv).reshape(-1)


def _fit_scale_min(xb: np.ndarray, nmax: int, iters: int = 4):
    """Per-row affine fit x ≈ scale*q - min with q in [0,nmax], min >= 0."""
    lo = np.minimum(xb.min(axis=-1, keepdims=True), 0.0)
    hi = xb.max(axis=-1, keepdims=True)
    scale = (hi - lo) / nmax
    mn = -lo
    for _ in range(iters):
        inv = np.where(scale > 0, 1.0 / np.where(scale > 0, scale, 1), 0)
        q = np.clip(np.rint((xb + mn) * inv), 0, nmax)
        n = xb.shape[-1]
        sq = q.sum(-1, keepdims=True)
        sqq = (q * q).sum(-1, keepdims=True)
        sx = xb.sum(-1, keepdims=True)
        sxq = (xb * q).sum(-1, keepdims=True)
        det = n * sqq - sq * sq
        ok = det > 1e-12
        s_new = np.where(ok, (n * sxq - sq * sx) / np.where(ok, det, 1), scale)
        m_new = np.where(ok, (sq * sxq - sqq * sx) / np.where(ok, det, 1), mn)
        good = ok & (s_new > 0)
        scale = np.where(good, s_new, scale)
        mn = np.where(good, np.maximum(m_new, 0), mn)
    return scale, mn


def quantize_q4_k(x: np.ndarray) -> np.ndarray:
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 8, 32)
    scale, mn = _fit_scale_min(xb, 15)
    scale = scale[..., 0]
    mn = mn[..., 0]
    d = scale.max(axis=1, keepdims=True) / 63.0
    dmin = mn.max(axis=1, keepdims=True) / 63.0
    d = d.astype("<f2").astype(np.float32)
    dmin = dmin.astype("<f2").astype(np.float32)
    inv_d = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0)
    inv_dm = np.where(dmin > 0, 1.0 / np.where(dmin > 0, dmin, 1), 0)
    sc = np.clip(np.rint(scale * inv_d), 0, 63)
    mq = np.clip(np.rint(mn * inv_dm), 0, 63)
    eff = (d * sc)[..., None]
    effm = (dmin * mq)[..., None]
    inv = np.where(eff > 0, 1.0 / np.where(eff > 0, eff, 1), 0)
    q = np.clip(np.rint((xb + effm) * inv), 0, 15).astype(np.uint8)
    out = np.empty((xb.shape[0], 144), dtype=np.uint8)
    out[:, 0:2] = d.astype("<f2").view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.astype("<f2").view(np.uint8).reshape(-1, 2)
    out[:, 4:16] = pack_scales_k4(sc, mq)
    qq = q.reshape(-1, 4, 2, 32)
    out[:, 16:] = (qq[:, :, 0, :] | (qq[:, :, 1, :] << 4)).reshape(-1, 128)
    return out.reshape(-1)


def dequantize_q5_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 176)
    d = _f16(b[:, 0:2].copy()).reshape(-1, 1)
    dmin = _f16(b[:, 2:4].copy()).reshape(-1, 1)
    sc, mn = unpack_scales_k4(b[:, 4:16])
    qh = b[:, 16:48]  # 32 bytes, bit (2*chunk + half) of byte l
    qs = b[:, 48:].reshape(-1, 4, 32)
    lo4 = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32)
    bits = ((qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1).astype(np.uint8)
    q = (lo4 + (bits << 4)).astype(np.float32)
    scale = (d * sc.astype(np.float32)).reshape(-1, 8, 1)
    minv = (dmin * mn.astype(np.float32)).reshape(-1, 8, 1)
    return (scale * q - minv).reshape(-1)


def dequantize_q6_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 210)
    ql = b[:, 0:128].reshape(-1, 2, 64)
    qh = b[:, 128:192].reshape(-1, 2, 32)
    sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(-1, 2, 8)
    d = _f16(b[:, 208:210].copy()).reshape(-1, 1, 1)
    l0 = ql[:, :, :32]
    l1 = ql[:, :, 32:]
    q1 = (l0 & 0xF) | (((qh >> 0) & 3) << 4)
    q2 = (l1 & 0xF) | (((qh >> 2) & 3) << 4)
    q3 = (l0 >> 4) | (((qh >> 4) & 3) << 4)
    q4 = (l1 >> 4) | (((qh >> 6) & 3) << 4)
    q = np.stack([q1, q2, q3, q4], axis=2).astype(np.float32) - 32  # [nb, 2, 4, 32]
    # scale index within a half: is = l//16 + 2*k for quarter k
    scv = sc.reshape(-1, 2, 4, 2)  # [nb, half, quarter, l//16]
    scale = np.repeat(scv, 16, axis=3)  # [nb,2,4,32]
    return (d[..., None] * scale * q).reshape(-1)


def quantize_q6_k(x: np.ndarray) -> np.ndarray:
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 16, 16)
    amax = np.abs(xb).max(axis=2)
    sub = amax / 31.0  # ideal per-16 scale (q in [-32,31], use symmetric 31)
    d = sub.max(axis=1, keepdims=True) / 127.0
    d = d.astype("<f2").astype(np.float32)
    inv_d = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0)
    sc = np.clip(np.rint(sub * inv_d), -128, 127)
    sc = np.where((sc == 0) & (amax > 0), 1, sc)
    eff = (d * sc)[..., None]
    inv = np.where(eff != 0, 1.0 / np.where(eff != 0, eff, 1), 0)
    q = (np.clip(np.rint(xb * inv), -32, 31) + 32).astype(np.uint8).reshape(-1, 2, 4, 32)
    out = np.empty((xb.shape[0], 210), dtype=np.uint8)
    lo = q & 0xF
    hi = q >> 4
    ql = np.empty((xb.shape[0], 2, 64), dtype=np.uint8)
    ql[:, :, :32] = lo[:, :, 0] | (lo[:, :, 2] << 4)
    ql[:, :, 32:] = lo[:, :, 1] | (lo[:, :, 3] << 4)
    qh = hi[:, :, 0] | (hi[:, :, 1] << 2) | (hi[:, :, 2] << 4) | (hi[:, :, 3] << 6)
    out[:, 0:128] = ql.reshape(-1, 128)
    out[:, 128:192] = qh.reshape(-1, 64)
    # scales stored so that scale index = half*8 + quarter*2 + l//16; xb sub-block j covers
    # values [16j,16j+16) = half j//8, quarter (j%8)//2, l//16 = j%2 -> same linear order.
    out[:, 192:208] = sc.astype(np.int8).view(np.uint8)
    out[:, 208:210] = d.astype("<f2").view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def dequantize_q2_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 84)
    scales = b[:, 0:16]
    qs = b[:, 16:80].reshape(-1, 2, 32)
    d = _f16(b[:, 80:82].copy()).reshape(-1, 1)
    dmin = _f16(b[:, 82:84].copy()).reshape(-1, 1)
    shifts = np.arange(4, dtype=np.uint8) * 2
    q = ((qs[:, :, None, :] >> shifts[None, None, :, None]) & 3).astype(np.float32)  # [nb,2,4,32]
    q = q.reshape(-1, 16, 16)
    dl = (d * (scales & 0xF).astype(np.float32))[..., None]
    ml = (dmin * (scales >> 4).astype(np.float32))[..., None]
    return (dl * q - ml).reshape(-1)


def dequantize_q3_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 110)
    hm = b[:, 0:32]
    qs = b[:, 32:96].reshape(-1, 2, 32)
    sraw = b[:, 96:108].copy().view("<u4").reshape(-1, 3)
    d = _f16(b[:, 108:110].copy()).reshape(-1, 1)
    k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
    a0, a1, tmp = sraw[:, 0], sraw[:, 1], sraw[:, 2]
    aux = np.stack(
        [
            (a0 & k2) | (((tmp >> 0) & k1) << 4),
            (a1 & k2) | (((tmp >> 2) & k1) << 4),
            ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4),
            ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4),
        ],
        axis=1,
    ).astype("<u4")
    sc = aux.view(np.int8).reshape(-1, 16).astype(np.float32) - 32
    shifts = np.arange(4, dtype=np.uint8) * 2
    q = ((qs[:, :, None, :] >> shifts[None, None, :, None]) & 3).astype(np.float32)  # [nb,2,4,32]
    mbit = np.arange(8, dtype=np.uint8).reshape(2, 4)
    hbit = ((hm[:, None, None, :] >> mbit[None, :, :, None]) & 1).astype(np.float32)
    q = q - 4 * (1 - hbit)
    q = q.reshape(-1, 16, 16)
    return ((d * sc)[..., None] * q).reshape(-1)


def dequantize_q8_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 292)
    d = b[:, 0:4].copy().view("<f4").reshape(-1, 1)
    q = b[:, 4:260].view(np.int8).astype(np.float32)
    return (d * q).reshape(-1)


def quantize_q8_k(x: np.ndarray) -> np.ndarray:
    """Activation quantizer: f32 d = amax/127, 256 int8, 16 int16 block sums
    (reference: kernels/gemv_f32.cu:404)."""
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 256)
    amax = np.abs(xb).max(axis=1, keepdims=True)
    d = (amax / 127.0).astype(np.float32)
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0)
    q = np.clip(np.rint(xb * inv), -127, 127).astype(np.int8)
    bs = q.reshape(-1, 16, 16).astype(np.int32).sum(axis=2).astype("<i2")
    out = np.empty((xb.shape[0], 292), dtype=np.uint8)
    out[:, 0:4] = d.view(np.uint8).reshape(-1, 4)
    out[:, 4:260] = q.view(np.uint8)
    out[:, 260:292] = bs.view(np.uint8).reshape(-1, 32)
    return out.reshape(-1)


def dequantize_iq4_nl(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 18)
    d = _f16(b[:, :2].copy()).reshape(-1, 1)
    qs = b[:, 2:]
    v = np.concatenate([IQ4NL_VALUES[qs & 0xF], IQ4NL_VALUES[qs >> 4]], axis=1)
    return (d * v).reshape(-1)


def dequantize_iq4_xs(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 136)
    d = _f16(b[:, 0:2].copy()).reshape(-1, 1)
    sh = b[:, 2:4].copy().view("<u2").reshape(-1, 1).astype(np.uint32)
    sl = b[:, 4:8]
    qs = b[:, 8:].reshape(-1, 8, 16)
    ib = np.arange(8)
    low = (sl[:, ib // 2] >> (4 * (ib % 2)).astype(np.uint8)) & 0xF
    high = (sh >> (2 * ib).astype(np.uint32)) & 3
    ls = (low.astype(np.int32) | (high.astype(np.int32) << 4)) - 32
    dl = (d * ls.astype(np.float32))[..., None]
    v = np.concatenate([IQ4NL_VALUES[qs & 0xF], IQ4NL_VALUES[qs >> 4]], axis=2)
    return (dl * v).reshape(-1)


# --------------------------------------------------------------------------- fp8 / fp4


def ue4m3_to_f32(b: np.ndarray, honour_sign: bool = False) -> np.ndarray:
    """NVFP4 sub-block scale byte -> f32, *halved* to pair with the doubled E2M1 table
    (``ue4m3_to_f32`` quant_nvfp4.rs:4-12).  0x00 and 0x7F decode to 0.  The reference's
    Rust decoder ignores bit 7; its CUDA decoder (gemv_f32.cu:1503-1511) honours it as a
    sign — ``honour_sign`` selects that behaviour."""
    b = b.astype(np.uint8)
    mag = b & 0x7F
    exp = (mag >> 3).astype(np.int32)
    man = (mag & 7).astype(np.float32)
    normal = np.ldexp(1.0 + man / 8.0, exp - 7)
    sub = np.ldexp(man, -9)
    v = np.where(exp == 0, sub, normal).astype(np.float32) * 0.5
    v = np.where((mag == 0) | (mag == 0x7F), 0.0, v).astype(np.float32)
    if honour_sign:
        v = np.where(b & 0x80, -v, v)
    return v


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest f32 -> fp8 e4m3fn byte (saturating at ±448, no inf)."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.minimum(np.abs(x), 448.0)
    e = np.floor(np.log2(np.maximum(a, 2.0**-20))).astype(np.int32)
    e = np.clip(e, -6, 8)
    step = np.ldexp(1.0, e - 3)
    q = np.rint(a / step) * step  # rint = ties-to-even on the mantissa grid
    q = np.minimum(q, 448.0)
    e2 = np.floor(np.log2(np.maximum(q, 2.0**-20))).astype(np.int32)
    e2 = np.clip(e2, -6, 8)
    man = np.rint(q / np.ldexp(1.0, e2 - 3)).astype(np.int32)
    is_sub = q < 2.0**-6
    man_sub = np.rint(q / 2.0**-9).astype(np.int32)
    byte = np.where(is_sub, man_sub, ((e2 + 7) << 3) | (man - 8)).astype(np.uint8)
    return (byte | sign).astype(np.uint8)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    b = b.astype(np.uint8)
    mag = b & 0x7F
    exp = (mag >> 3).astype(np.int32)
    man = (mag & 7).astype(np.float32)
    v = np.where(exp == 0, np.ldexp(man, -9), np.ldexp(1.0 + man / 8.0, exp - 7)).astype(np.float32)
    v = np.where(mag == 0x7F, np.nan, v)
    return np.where(b & 0x80, -v, v).astype(np.float32)


def dequantize_nvfp4(raw: np.ndarray, honour_sign: bool = False) -> np.ndarray:
    """64-value block: 4 ue4m3 sub-scales (16 values each) then 4×8 nibble bytes; inside a
    sub-block byte j holds value j (low nibble) and j+8 (high nibble)."""
    b = raw.reshape(-1, 36)
    sc = ue4m3_to_f32(b[:, 0:4], honour_sign).reshape(-1, 4, 1)
    qs = b[:, 4:].reshape(-1, 4, 8)
    v = np.concatenate([E2M1_DOUBLED[qs & 0xF], E2M1_DOUBLED[qs >> 4]], axis=2)  # [nb,4,16]
    return (sc * v).reshape(-1)


_E2M1_POS = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], dtype=np.float32)


def quantize_nvfp4(x: np.ndarray) -> np.ndarray:
    """Encoder for the 36-byte NVFP4 block (the reference ships a decoder only)."""
    xb = np.asarray(x, dtype=np.float32).reshape(-1, 4, 16)
    amax = np.abs(xb).max(axis=2, keepdims=True)
    # true scale s so that amax/s <= 6; stored byte decodes (after the 0.5) to s/2 and pairs
    # with doubled codes, i.e. value = (s/2) * (2*e2m1).
    s = amax / 6.0
    sb = f32_to_e4m3(s.reshape(-1)).reshape(s.shape) & 0x7F
    s_dec = e4m3_to_f32(sb)
    # round the scale up when saturation would clip
    bump = (s_dec * 6.0 < amax) & (sb < 0x7E)
    sb = np.where(bump, sb + 1, sb).astype(np.uint8)
    s_dec = np.nan_to_num(e4m3_to_f32(sb))
    inv = np.where(s_dec > 0, 1.0 / np.where(s_dec > 0, s_dec, 1), 0)
    y = xb * inv
    code = np.abs(np.abs(y)[..., None] - _E2M1_POS).argmin(axis=-1).astype(np.uint8)
    code = code | (np.signbit(y).astype(np.uint8) << 3)
    out = np.empty((xb.shape[0], 36), dtype=np.uint8)
    out[:, 0:4] = sb.reshape(-1, 4)
    out[:, 4:] = (code[:, :, :8] | (code[:, :, 8:] << 4)).reshape(-1, 32)
    return out.reshape(-1)


def quantize_fp8_block(x: np.ndarray, block: int = 128):
    """Block-scaled fp8 e4m3: returns (codes uint8[n], scales f32[n/block]); x ≈ code*scale."""
    xb = np.asarray(x, dtype=np.float32).reshape(-1, block)
    amax = np.abs(xb).max(axis=1, keepdims=True)
    scale = np.where(amax > 0, amax / 448.0, 1.0).astype(np.float32)
    return f32_to_e4m3((xb / scale).reshape(-1)), scale.reshape(-1)


def dequantize_fp8_block(codes: np.ndarray, scales: np.ndarray, block: int = 128) -> np.ndarray:
    return (e4m3_to_f32(codes).reshape(-1, block) * scales.reshape(-1, 1)).reshape(-1)


# --------------------------------------------------------------------------- dispatch

_DEQ: Dict[str, Callable[[np.ndarray], np.ndarray]] = {
    "Q4_0": dequantize_q4_0,
    "Q4_1": dequantize_q4_1,
    "Q5_0": dequantize_q5_0,
    "Q5_1": dequantize_q5_1,
    "Q8_0": dequantize_q8_0,
    "Q2_K": dequantize_q2_k,
    "Q3_K": dequantize_q3_k,
    "Q4_K": dequantize_q4_k,
    "Q5_K": dequantize_q5_k,
    "Q6_K": dequantize_q6_k,
    "Q8_K": dequantize_q8_k,
    "IQ4_NL": dequantize_iq4_nl,
    "IQ4_XS": dequantize_iq4_xs,
    "NVFP4": dequantize_nvfp4,
}
_QUANT: Dict[str, Callable[[np.ndarray], np.ndarray]] = {
    "Q4_0": quantize_q4_0,
    "Q5_0": quantize_q5_0,
    "Q8_0": quantize_q8_0,
    "Q4_K": quantize_q4_k,
    "Q6_K": quantize_q6_k,
    "Q8_K": quantize_q8_k,
    "NVFP4": quantize_nvfp4,
}


# i-quants whose decode needs the large ggml codebook grids (256-2048 entries each).  The grids are data
# of the ggml format, not of this framework: they come from the `gguf` package when it is installed.
_CODEBOOK_TYPES = ("IQ1_S", "IQ1_M", "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S")


def _dequantize_codebook(t, raw: np.ndarray) -> np.ndarray:
    try:
        import gguf
        from gguf import quants as gq
    except Exception as e:  # pragma: no cover - depends on the environment
        raise GGUFError(f"{t.name} needs the ggml codebook grids from the `gguf` package, which is not installed") from e
    if raw.size % t.type_size:
        raise GGUFError(f"{t.name}: {raw.size} bytes is not whole {t.type_size}-byte blocks")
    qtype = getattr(gguf.GGMLQuantizationType, t.name)
    return np.asarray(gq.dequantize(raw.reshape(-1, t.type_size), qtype), dtype=np.float32).reshape(-1)


def dequantize(type_name, raw: np.ndarray, n_elements: int | None = None) -> np.ndarray:
    """Decode ``raw`` block bytes of the given ggml type to float32 (dispatch like
    ``dequantize_scalar`` quant_dispatch.rs:4)."""
    t = ggml_type(type_name)
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    if t.name == "F32":
        out = raw.view("<f4").astype(np.float32)
    elif t.name == "F16":
        out = raw.view("<f2").astype(np.float32)
    elif t.name == "BF16":
        out = bf16_to_f32(raw.view("<u2"))
    elif t.name in _DEQ:
        if raw.size % t.type_size:
            raise GGUFError(f"{t.name}: {raw.size} bytes is not whole {t.type_size}-byte blocks")
        out = _DEQ[t.name](raw)
    elif t.name in _CODEBOOK_TYPES:
        out = _dequantize_codebook(t, raw)
    else:
        raise GGUFError(f"no dequantizer for {t.name}")
    if n_elements is not None and out.size != n_elements:
        raise GGUFError(f"{t.name}: decoded {out.size} values, expected {n_elements}")
    return out


def quantize(type_name, x: np.ndarray) -> np.ndarray:
    t = ggml_type(type_name)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if t.name == "F32":
        return x.view(np.uint8)
    if t.name == "F16":
        return x.astype("<f2").view(np.uint8)
    if t.name == "BF16":
        return f32_to_bf16(x).view(np.uint8)
    if t.name not in _QUANT:
        raise GGUFError(f"no quantizer for {t.name}")
    if x.size % t.block_size:
        raise GGUFError(f"{t.name}: {x.size} values is not whole blocks of {t.block_size}")
    return _QUANT[t.name](x)


def can_quantize(type_name) -> bool:
    return ggml_type(type_name).name in _QUANT or ggml_type(type_name).name in ("F32", "F16", "BF16")
