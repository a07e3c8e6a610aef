"""SafeTensors reader/writer (mmap, zero-copy) — the second checkpoint format the reference loads
(``oxidize-core/src/format/safetensors.rs``).  File layout: ``u64 header_len``, a JSON header
mapping tensor name → ``{dtype, shape, data_offsets}``, then the raw little-endian data."""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np

_DTYPES = {"F32": "<f4", "F16": "<f2", "BF16": "<u2", "F64": "<f8", "I8": "i1", "U8": "u1", "I16": "<i2",
           "I32": "<i4", "I64": "<i8", "BOOL": "u1", "F8_E4M3": "u1"}
MAX_HEADER = 100 << 20


class SafeTensorsError(ValueError):
    pass


class SafeTensorsFile:
    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            size = os.fstat(f.fileno()).st_size
            if size < 8:
                raise SafeTensorsError("file too small")
            self._mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > MAX_HEADER or 8 + hlen > size:
            raise SafeTensorsError("invalid header length")
        try:
            header = json.loads(bytes(self._mm[8 : 8 + hlen]))
        except ValueError as e:
            raise SafeTensorsError(f"bad JSON header: {e}") from e
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self.data_start = 8 + hlen
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            dt, shape = e["dtype"], tuple(int(s) for s in e["shape"])
            b, end = e["data_offsets"]
            if dt not in _DTYPES:
                raise SafeTensorsError(f"{name}: unsupported dtype {dt}")
            n = int(np.prod(shape)) if shape else 1
            if end - b != n * np.dtype(_DTYPES[dt]).itemsize or self.data_start + end > size:
                raise SafeTensorsError(f"{name}: extent does not match shape")
            self.entries[name] = (dt, shape, b, end)

    def keys(self) -> List[str]:
        return list(self.entries)

    def dtype(self, name: str) -> str:
        return self.entries[name][0]

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def tensor(self, name: str) -> np.ndarray:
        """Typed view (BF16 comes back as uint16 bit patterns)."""
        dt, shape, b, e = self.entries[name]
        arr = np.frombuffer(self._mm, dtype=_DTYPES[dt], count=(e - b) // np.dtype(_DTYPES[dt]).itemsize,
                            offset=self.data_start + b)
        return arr.reshape(shape)

    def tensor_f32(self, name: str) -> np.ndarray:
        a = self.tensor(name)
        if self.dtype(name) == "BF16":
            return (a.astype(np.uint32) << 16).view(np.float32)
        return a.astype(np.float32)


def load_sharded(paths: Iterable[str]) -> Dict[str, Tuple[SafeTensorsFile, str]]:
    """name → (file, name) over several shards (``model-0000x-of-0000y.safetensors``)."""
    out: Dict[str, Tuple[SafeTensorsFile, str]] = {}
    for p in paths:
        f = SafeTensorsFile(p)
        for k in f.keys():
            out[k] = (f, k)
    return out


def save_file(tensors: Dict[str, np.ndarray], path: str, metadata: Dict[str, str] = None,
              dtypes: Dict[str, str] = None) -> None:
    """Write arrays; ``dtypes`` can mark uint16 arrays as BF16."""
    inv = {np.dtype(v).str: k for k, v in _DTYPES.items() if k not in ("BOOL", "F8_E4M3", "BF16")}
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, arr in tensors.items():
        a = np.ascontiguousarray(arr)
        dt = (dtypes or {}).get(name) or inv.get(a.dtype.newbyteorder("<").str) or inv.get(a.dtype.str)
        if dt is None:
            raise SafeTensorsError(f"{name}: cannot store dtype {a.dtype}")
        raw = a.tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
