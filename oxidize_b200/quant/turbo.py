"""Block-wise symmetric INT4 / INT8 weight quantizer with a GEMV on the packed form (the reference's "TurboQuant" weight
codec, ``oxidize-core/src/compute/turboquant.rs:28-204``): 32-value blocks along a row, one float scale per block
(``max|w| / qmax``), codes stored offset by ``qmax`` as unsigned values (two per byte, low nibble first, for INT4).  The
same scheme, per 32 channels, is what the KV cache's q8 / q4 modes use; this module is the weight-side form.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

BLOCK = 32


@dataclass
class TurboQuantData:
    bits: int  # 4 or 8
    rows: int
    cols: int
    scales: np.ndarray  # [rows, blocks_per_row] float32
    codes: np.ndarray  # [rows, blocks_per_row, BLOCK // 2] (INT4) or [rows, blocks_per_row, BLOCK] (INT8) uint8

    @property
    def nbytes(self) -> int:
        return self.scales.nbytes + self.codes.nbytes


def quantize(w: np.ndarray, bits: int = 4) -> TurboQuantData:
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    nb = -(-cols // BLOCK)
    padded = np.zeros((rows, nb * BLOCK), dtype=np.float32)
    padded[:, :cols] = w
    blocks = padded.reshape(rows, nb, BLOCK)
    qmax = (1 << (bits - 1)) - 1
    amax = np.abs(blocks).max(axis=2)
    scales = np.where(amax > 0, amax / qmax, 1.0).astype(np.float32)
    q = np.clip(np.rint(blocks / scales[:, :, None]), -qmax, qmax).astype(np.int16) + qmax  # 0 .. 2 qmax
    if bits == 8:
        codes = q.astype(np.uint8)
    else:
        codes = (q[:, :, 0::2] | (q[:, :, 1::2] << 4)).astype(np.uint8)
    return TurboQuantData(bits, rows, cols, scales, codes)


def dequantize(d: TurboQuantData) -> np.ndarray:
    qmax = (1 << (d.bits - 1)) - 1
    if d.bits == 8:
        q = d.codes.astype(np.int16)
    else:
        q = np.empty((d.rows, d.codes.shape[1], BLOCK), dtype=np.int16)
        q[:, :, 0::2] = d.codes & 0x0F
        q[:, :, 1::2] = d.codes >> 4
    out = (q - qmax).astype(np.float32) * d.scales[:, :, None]
    return out.reshape(d.rows, -1)[:, : d.cols]


def gemv(d: TurboQuantData, x: np.ndarray) -> np.ndarray:
    """y = W x on the packed form: per block an integer-valued dot product, then one multiply by the block's scale."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.shape != (d.cols,):
        raise ValueError(f"vector of {x.shape} against {d.cols} columns")
    nb = d.codes.shape[1]
    xp = np.zeros(nb * BLOCK, dtype=np.float32)
    xp[: d.cols] = x
    xb = xp.reshape(nb, BLOCK)
    qmax = (1 << (d.bits - 1)) - 1
    if d.bits == 8:
        q = d.codes.astype(np.float32) - qmax
    else:
        q = np.empty((d.rows, nb, BLOCK), dtype=np.float32)
        q[:, :, 0::2] = (d.codes & 0x0F).astype(np.float32) - qmax
        q[:, :, 1::2] = (d.codes >> 4).astype(np.float32) - qmax
    return (np.einsum("rbk,bk->rb", q, xb) * d.scales).sum(axis=1)
