"""GGUF v2/v3 reader (mmap, zero-copy tensor views) and writer.

The checkpoint format is kept byte-compatible with what the reference parses in
``oxidize-core/src/format/gguf.rs:612-717`` (header, 13 metadata value types, tensor
infos, ``general.alignment`` defaulting to 32, extent validation) and with the
split-shard naming ``-NNNNN-of-MMMMM.gguf`` handled at ``gguf.rs:551-610``.

Design notes (ours, not the reference's): the reader returns ``numpy`` views on one
``mmap`` so that a tensor-parallel rank can slice packed quant blocks by row and copy
only its shard to the device; nothing is materialised on the host.
"""
from __future__ import annotations

import mmap
import os
import re
import struct
from dataclasses import dataclass, field
from typing import Any, BinaryIO, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

GGUF_MAGIC = b"GGUF"
GGUF_DEFAULT_ALIGNMENT = 32
GGUF_SUPPORTED_VERSIONS = (2, 3)
MAX_ARRAY_DEPTH = 32
MAX_STRING_BYTES = 1 << 30
MAX_TENSOR_DIMS = 8


class GGUFError(ValueError):
    """Raised for any malformed or unsupported GGUF input."""


class GGUFValueType:
    UINT8 = 0
    INT8 = 1
    UINT16 = 2
    INT16 = 3
    UINT32 = 4
    INT32 = 5
    FLOAT32 = 6
    BOOL = 7
    STRING = 8
    ARRAY = 9
    UINT64 = 10
    INT64 = 11
    FLOAT64 = 12


_SCALAR_FMT = {
    GGUFValueType.UINT8: "<B",
    GGUFValueType.INT8: "<b",
    GGUFValueType.UINT16: "<H",
    GGUFValueType.INT16: "<h",
    GGUFValueType.UINT32: "<I",
    GGUFValueType.INT32: "<i",
    GGUFValueType.FLOAT32: "<f",
    GGUFValueType.UINT64: "<Q",
    GGUFValueType.INT64: "<q",
    GGUFValueType.FLOAT64: "<d",
}
_SCALAR_NP = {
    GGUFValueType.UINT8: np.uint8,
    GGUFValueType.INT8: np.int8,
    GGUFValueType.UINT16: np.dtype("<u2"),
    GGUFValueType.INT16: np.dtype("<i2"),
    GGUFValueType.UINT32: np.dtype("<u4"),
    GGUFValueType.INT32: np.dtype("<i4"),
    GGUFValueType.FLOAT32: np.dtype("<f4"),
    GGUFValueType.UINT64: np.dtype("<u8"),
    GGUFValueType.INT64: np.dtype("<i8"),
    GGUFValueType.FLOAT64: np.dtype("<f8"),
    GGUFValueType.BOOL: np.uint8,
}


@dataclass(frozen=True)
class GGMLTypeInfo:
    """Block geometry of one ggml tensor type: ``block_size`` values in ``type_size`` bytes."""

    name: str
    ggml_id: int
    block_size: int
    type_size: int


# ggml type ids match ``from_ggml_type`` in the reference (gguf.rs:372-414); 40 = NVFP4
# (64 values in 36 bytes), 240-243 = the reference's private "AL" family.
_GGML_TYPES: Tuple[GGMLTypeInfo, ...] = (
    GGMLTypeInfo("F32", 0, 1, 4),
    GGMLTypeInfo("F16", 1, 1, 2),
    GGMLTypeInfo("Q4_0", 2, 32, 18),
    GGMLTypeInfo("Q4_1", 3, 32, 20),
    GGMLTypeInfo("Q5_0", 6, 32, 22),
    GGMLTypeInfo("Q5_1", 7, 32, 24),
    GGMLTypeInfo("Q8_0", 8, 32, 34),
    GGMLTypeInfo("Q8_1", 9, 32, 36),
    GGMLTypeInfo("Q2_K", 10, 256, 84),
    GGMLTypeInfo("Q3_K", 11, 256, 110),
    GGMLTypeInfo("Q4_K", 12, 256, 144),
    GGMLTypeInfo("Q5_K", 13, 256, 176),
    GGMLTypeInfo("Q6_K", 14, 256, 210),
    GGMLTypeInfo("Q8_K", 15, 256, 292),
    GGMLTypeInfo("IQ2_XXS", 16, 256, 66),
    GGMLTypeInfo("IQ2_XS", 17, 256, 74),
    GGMLTypeInfo("IQ3_XXS", 18, 256, 98),
    GGMLTypeInfo("IQ1_S", 19, 256, 50),
    GGMLTypeInfo("IQ4_NL", 20, 32, 18),
    GGMLTypeInfo("IQ3_S", 21, 256, 110),
    GGMLTypeInfo("IQ2_S", 22, 256, 82),
    GGMLTypeInfo("IQ4_XS", 23, 256, 136),
    GGMLTypeInfo("I8", 24, 1, 1),
    GGMLTypeInfo("I16", 25, 1, 2),
    GGMLTypeInfo("I32", 26, 1, 4),
    GGMLTypeInfo("I64", 27, 1, 8),
    GGMLTypeInfo("F64", 28, 1, 8),
    GGMLTypeInfo("IQ1_M", 29, 256, 56),
    GGMLTypeInfo("BF16", 30, 1, 2),
    GGMLTypeInfo("NVFP4", 40, 64, 36),
)
GGML_TYPE_BY_ID: Dict[int, GGMLTypeInfo] = {t.ggml_id: t for t in _GGML_TYPES}
GGML_TYPE_BY_NAME: Dict[str, GGMLTypeInfo] = {t.name: t for t in _GGML_TYPES}


def ggml_type(name_or_id) -> GGMLTypeInfo:
    if isinstance(name_or_id, GGMLTypeInfo):
        return name_or_id
    if isinstance(name_or_id, str):
        try:
            return GGML_TYPE_BY_NAME[name_or_id.upper()]
        except KeyError as e:
            raise GGUFError(f"unknown ggml type name {name_or_id!r}") from e
    try:
        return GGML_TYPE_BY_ID[int(name_or_id)]
    except KeyError as e:
        raise GGUFError(f"unsupported ggml type id {name_or_id}") from e


def quantized_nbytes(type_info: GGMLTypeInfo, n_elements: int) -> int:
    """Bytes of ``n_elements`` values; rejects a count that is not whole blocks
    (same rule as ``quantized_size`` in ``compute/quantization.rs:283-297``)."""
    if n_elements % type_info.block_size:
        raise GGUFError(
            f"{type_info.name}: {n_elements} elements is not a multiple of the block size {type_info.block_size}"
        )
    return n_elements // type_info.block_size * type_info.type_size


def _align_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass
class GGUFTensorInfo:
    name: str
    # dims as stored in the file: dims[0] is the fastest-varying (row length, "ne0")
    dims: Tuple[int, ...]
    type: GGMLTypeInfo
    offset: int  # relative to the data section

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        return quantized_nbytes(self.type, self.n_elements)

    @property
    def shape(self) -> Tuple[int, ...]:
        """Row-major logical shape (slowest first), e.g. ``(out_features, in_features)``."""
        return tuple(reversed(self.dims))

    @property
    def row_nbytes(self) -> int:
        return quantized_nbytes(self.type, self.dims[0])


class _Cursor:
    __slots__ = ("buf", "pos", "end")

    def __init__(self, buf, pos: int = 0):
        self.buf = buf
        self.pos = pos
        self.end = len(buf)

    def take(self, n: int):
        if n < 0 or self.pos + n > self.end:
            raise GGUFError(f"truncated GGUF: need {n} bytes at offset {self.pos}, file has {self.end}")
        out = self.buf[self.pos : self.pos + n]
        self.pos += n
        return out

    def unpack(self, fmt: str):
        size = struct.calcsize(fmt)
        return struct.unpack(fmt, self.take(size))[0]

    def string(self) -> str:
        n = self.unpack("<Q")
        if n > MAX_STRING_BYTES:
            raise GGUFError(f"string length {n} exceeds limit")
        raw = bytes(self.take(n))
        return raw.decode("utf-8", errors="replace")


def _read_value(cur: _Cursor, vtype: int, depth: int = 0) -> Any:
    if vtype in _SCALAR_FMT:
        return cur.unpack(_SCALAR_FMT[vtype])
    if vtype == GGUFValueType.BOOL:
        b = cur.unpack("<B")
        if b not in (0, 1):
            raise GGUFError(f"invalid bool byte {b}")
        return bool(b)
    if vtype == GGUFValueType.STRING:
        return cur.string()
    if vtype == GGUFValueType.ARRAY:
        if depth >= MAX_ARRAY_DEPTH:
            raise GGUFError("metadata array nesting too deep")
        etype = cur.unpack("<I")
        count = cur.unpack("<Q")
        if etype in _SCALAR_NP:
            dt = np.dtype(_SCALAR_NP[etype])
            raw = cur.take(count * dt.itemsize)
            arr = np.frombuffer(raw, dtype=dt, count=count)
            if etype == GGUFValueType.BOOL:
                return [bool(x) for x in arr]
            return arr.tolist()
        if etype not in (GGUFValueType.STRING, GGUFValueType.ARRAY):
            raise GGUFError(f"unknown metadata array element type {etype}")
        if count > cur.end:
            raise GGUFError("array count exceeds file size")
        return [_read_value(cur, etype, depth + 1) for _ in range(count)]
    raise GGUFError(f"unknown metadata value type {vtype}")


@dataclass
class GGUFFile:
    """A parsed GGUF file. ``tensor(name)`` gives a zero-copy ``uint8``/typed view."""

    path: Optional[str]
    version: int
    metadata: Dict[str, Any]
    metadata_types: Dict[str, int]
    tensors: Dict[str, GGUFTensorInfo]
    alignment: int
    data_offset: int
    _buf: Any = field(repr=False, default=None)
    _mmap: Any = field(repr=False, default=None)
    _shards: List["GGUFFile"] = field(repr=False, default_factory=list)

    def get(self, key: str, default: Any = None) -> Any:
        return self.metadata.get(key, default)

    @property
    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", "llama"))

    def arch_get(self, suffix: str, default: Any = None) -> Any:
        return self.metadata.get(f"{self.architecture}.{suffix}", default)

    def has_tensor(self, name: str) -> bool:
        return name in self.tensors

    def tensor_bytes(self, name: str) -> np.ndarray:
        """Raw bytes of a tensor as a 1-D ``uint8`` view on the mapping."""
        info = self.tensors[name]
        owner = getattr(info, "_owner", None) or self
        start = owner.data_offset + info.offset
        return np.frombuffer(owner._buf, dtype=np.uint8, count=info.nbytes, offset=start)

    def tensor_rows(self, name: str) -> np.ndarray:
        """Raw bytes reshaped ``[n_rows, row_nbytes]`` (n_rows = product of outer dims)."""
        info = self.tensors[name]
        raw = self.tensor_bytes(name)
        return raw.reshape(-1, info.row_nbytes)

    def tensor(self, name: str) -> np.ndarray:
        """Typed view for unquantized types; ``uint8`` rows for block-quantized ones."""
        info = self.tensors[name]
        raw = self.tensor_bytes(name)
        t = info.type.name
        if t == "F32":
            return raw.view("<f4").reshape(info.shape)
        if t == "F16":
            return raw.view("<f2").reshape(info.shape)
        if t == "BF16":
            return raw.view("<u2").reshape(info.shape)
        if t == "F64":
            return raw.view("<f8").reshape(info.shape)
        if t in ("I8", "I16", "I32", "I64"):
            return raw.view({"I8": "i1", "I16": "<i2", "I32": "<i4", "I64": "<i8"}[t]).reshape(info.shape)
        return raw.reshape(info.shape[:-1] + (info.row_nbytes,))

    def advise(self, willneed: bool = False, hugepages: bool = False) -> List[str]:
        """Hints to the kernel about the file mapping (the reference's ``--mmap-prefetch`` / ``--mmap-hugepages``,
        ``format/gguf.rs:192``): read the pages ahead of their first use, back the mapping with huge pages where the
        system allows.  Returns the hints that were accepted; a refused hint is not an error."""
        import mmap as _mmap

        done = []
        for owner in [self] + list(self._shards):
            mm = owner._mmap
            if mm is None:
                continue
            for flag, name, const in ((willneed, "willneed", "MADV_WILLNEED"), (hugepages, "hugepages", "MADV_HUGEPAGE")):
                if flag and hasattr(_mmap, const):
                    try:
                        mm.madvise(getattr(_mmap, const))
                        if name not in done:
                            done.append(name)
                    except OSError:
                        pass
        return done

    def close(self) -> None:
        for s in self._shards:
            s.close()
        self._buf = None
        if self._mmap is not None:
            try:
                self._mmap.close()
            except BufferError:
                pass  # live numpy views keep the mapping alive; the OS unmaps at exit
            self._mmap = None


def parse_gguf(buf, path: Optional[str] = None) -> GGUFFile:
    """Parse a GGUF image held in any buffer object (bytes, mmap, memoryview)."""
    cur = _Cursor(buf)
    if bytes(cur.take(4)) != GGUF_MAGIC:
        raise GGUFError("invalid GGUF magic")
    version = cur.unpack("<I")
    if version not in GGUF_SUPPORTED_VERSIONS:
        raise GGUFError(f"unsupported GGUF version {version}")
    tensor_count = cur.unpack("<Q")
    kv_count = cur.unpack("<Q")
    if tensor_count > cur.end or kv_count > cur.end:
        raise GGUFError("header counts exceed file size")

    metadata: Dict[str, Any] = {}
    metadata_types: Dict[str, int] = {}
    for _ in range(kv_count):
        key = cur.string()
        vtype = cur.unpack("<I")
        metadata[key] = _read_value(cur, vtype)
        metadata_types[key] = vtype

    alignment = metadata.get("general.alignment", GGUF_DEFAULT_ALIGNMENT)
    if not isinstance(alignment, int) or alignment <= 0 or alignment & (alignment - 1):
        raise GGUFError(f"general.alignment must be a positive power of two, got {alignment!r}")

    tensors: Dict[str, GGUFTensorInfo] = {}
    for _ in range(tensor_count):
        name = cur.string()
        n_dims = cur.unpack("<I")
        if n_dims > MAX_TENSOR_DIMS:
            raise GGUFError(f"tensor {name!r}: {n_dims} dims exceeds limit")
        dims = tuple(cur.unpack("<Q") for _ in range(n_dims)) or (1,)
        tid = cur.unpack("<I")
        offset = cur.unpack("<Q")
        info = GGUFTensorInfo(name, dims, ggml_type(tid), offset)
        if name in tensors:
            raise GGUFError(f"duplicate tensor name {name!r}")
        tensors[name] = info

    data_offset = _align_up(cur.pos, alignment)
    total = cur.end
    for info in tensors.values():
        if info.offset % alignment:
            raise GGUFError(f"tensor {info.name!r}: offset {info.offset} is not {alignment}-byte aligned")
        end = data_offset + info.offset + info.nbytes
        if end > total:
            raise GGUFError(f"tensor {info.name!r} extends past end of file ({end} > {total})")
    return GGUFFile(path, version, metadata, metadata_types, tensors, alignment, data_offset, _buf=buf)


_SPLIT_RE = re.compile(r"^(?P<stem>.*)-(?P<idx>\d{5})-of-(?P<n>\d{5})\.gguf$")


def collect_split_shards(path: str) -> List[str]:
    """Given any shard ``X-0000i-of-0000n.gguf`` return all n shard paths in order;
    a non-split path returns ``[path]``."""
    m = _SPLIT_RE.match(os.path.basename(path))
    if not m:
        return [path]
    n = int(m.group("n"))
    d = os.path.dirname(path)
    out = [os.path.join(d, f"{m.group('stem')}-{i:05d}-of-{n:05d}.gguf") for i in range(1, n + 1)]
    missing = [p for p in out if not os.path.exists(p)]
    if missing:
        raise GGUFError(f"missing split shards: {missing}")
    return out


def _load_one(path: str, prefault: bool) -> GGUFFile:
    f = open(path, "rb")
    try:
        size = os.fstat(f.fileno()).st_size
        if size < 24:
            raise GGUFError("file too small to be GGUF")
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    finally:
        f.close()
    if hasattr(mm, "madvise"):
        try:
            mm.madvise(mmap.MADV_WILLNEED if prefault else mmap.MADV_RANDOM)
        except (OSError, ValueError):
            pass
    g = parse_gguf(mm, path)
    g._mmap = mm
    return g


def load_gguf(path: str, prefault: bool = False) -> GGUFFile:
    """mmap-load a GGUF file; split shards are merged (metadata from shard 1)."""
    paths = collect_split_shards(path)
    first = _load_one(paths[0], prefault)
    if len(paths) == 1:
        return first
    for p in paths[1:]:
        shard = _load_one(p, prefault)
        for name, info in shard.tensors.items():
            if name in first.tensors:
                raise GGUFError(f"tensor {name!r} appears in more than one shard")
            object.__setattr__(info, "_owner", shard)
            first.tensors[name] = info
        first._shards.append(shard)
    return first


# --------------------------------------------------------------------------- writer


def _infer_value_type(v: Any) -> int:
    if isinstance(v, bool):
        return GGUFValueType.BOOL
    if isinstance(v, int):
        if v < 0:
            return GGUFValueType.INT32 if v >= -(1 << 31) else GGUFValueType.INT64
        return GGUFValueType.UINT32 if v < (1 << 32) else GGUFValueType.UINT64
    if isinstance(v, float):
        return GGUFValueType.FLOAT32
    if isinstance(v, str):
        return GGUFValueType.STRING
    if isinstance(v, (list, tuple, np.ndarray)):
        return GGUFValueType.ARRAY
    raise GGUFError(f"cannot infer GGUF value type for {type(v)}")


def _pack_string(s: str) -> bytes:
    raw = s.encode("utf-8")
    return struct.pack("<Q", len(raw)) + raw


def _pack_value(v: Any, vtype: int, elem_type: Optional[int] = None) -> bytes:
    if vtype in _SCALAR_FMT:
        return struct.pack(_SCALAR_FMT[vtype], v)
    if vtype == GGUFValueType.BOOL:
        return struct.pack("<B", 1 if v else 0)
    if vtype == GGUFValueType.STRING:
        return _pack_string(v)
    if vtype == GGUFValueType.ARRAY:
        seq = list(v)
        if elem_type is None:
            if not seq:
                elem_type = GGUFValueType.INT32
            else:
                types = {_infer_value_type(x) for x in seq}
                if types <= {GGUFValueType.UINT32, GGUFValueType.INT32}:
                    elem_type = GGUFValueType.INT32 if GGUFValueType.INT32 in types else GGUFValueType.UINT32
                elif len(types) == 1:
                    elem_type = types.pop()
                elif types <= {GGUFValueType.UINT32, GGUFValueType.INT32, GGUFValueType.FLOAT32}:
                    elem_type = GGUFValueType.FLOAT32
                else:
                    raise GGUFError("heterogeneous metadata array")
        head = struct.pack("<IQ", elem_type, len(seq))
        if elem_type in _SCALAR_NP and elem_type != GGUFValueType.BOOL:
            return head + np.asarray(seq, dtype=_SCALAR_NP[elem_type]).tobytes()
        return head + b"".join(_pack_value(x, elem_type) for x in seq)
    raise GGUFError(f"unknown value type {vtype}")


class GGUFWriter:
    """Streams a GGUF v3 file: metadata, tensor infos, aligned data section.

    ``add_tensor`` takes raw block bytes (``uint8``) for quantized types or a typed array
    for F32/F16/BF16; ``shape`` is row-major ``(out, in)`` and is stored reversed, the way
    llama.cpp and the reference's converter (``format/safetensors_to_gguf.rs``) write it.
    """

    def __init__(self, path: str, arch: str = "llama", alignment: int = GGUF_DEFAULT_ALIGNMENT, version: int = 3):
        if alignment <= 0 or alignment & (alignment - 1):
            raise GGUFError("alignment must be a power of two")
        self.path = path
        self.alignment = alignment
        self.version = version
        self._kv: List[Tuple[str, int, Optional[int], Any]] = []
        self._tensors: List[Tuple[str, Tuple[int, ...], GGMLTypeInfo, Any]] = []
        self.add("general.architecture", arch)
        if alignment != GGUF_DEFAULT_ALIGNMENT:
            self.add("general.alignment", alignment, GGUFValueType.UINT32)

    def add(self, key: str, value: Any, vtype: Optional[int] = None, elem_type: Optional[int] = None) -> None:
        if vtype is None:
            vtype = _infer_value_type(value)
        self._kv = [kv for kv in self._kv if kv[0] != key]
        self._kv.append((key, vtype, elem_type, value))

    def add_tensor(self, name: str, data, shape: Optional[Sequence[int]] = None, type_name: Optional[str] = None) -> None:
        """``data`` may be an ndarray or a zero-arg callable returning one (lazy, so a
        141 GB model can be streamed tensor by tensor)."""
        if type_name is None:
            arr = data
            type_name = {np.dtype("float32"): "F32", np.dtype("float16"): "F16"}.get(arr.dtype)
            if type_name is None:
                raise GGUFError("type_name required for non-f32/f16 arrays")
        tinfo = ggml_type(type_name)
        if shape is None:
            shape = data.shape
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        quantized_nbytes(tinfo, n)
        if shape[-1] % tinfo.block_size:
            raise GGUFError(f"{name}: row length {shape[-1]} not a multiple of {tinfo.name} block {tinfo.block_size}")
        self._tensors.append((name, shape, tinfo, data))

    def write(self) -> int:
        head = bytearray()
        head += GGUF_MAGIC
        head += struct.pack("<IQQ", self.version, len(self._tensors), len(self._kv))
        for key, vtype, etype, value in self._kv:
            head += _pack_string(key)
            head += struct.pack("<I", vtype)
            head += _pack_value(value, vtype, etype)
        offset = 0
        offsets = []
        for name, shape, tinfo, _ in self._tensors:
            n = 1
            for s in shape:
                n *= s
            nbytes = quantized_nbytes(tinfo, n)
            head += _pack_string(name)
            dims = tuple(reversed(shape))
            head += struct.pack("<I", len(dims))
            for d in dims:
                head += struct.pack("<Q", d)
            head += struct.pack("<IQ", tinfo.ggml_id, offset)
            offsets.append((offset, nbytes))
            offset = _align_up(offset + nbytes, self.alignment)
        data_start = _align_up(len(head), self.alignment)
        with open(self.path, "wb") as f:
            f.write(head)
            f.write(b"\0" * (data_start - len(head)))
            pos = 0
            for (name, shape, tinfo, data), (off, nbytes) in zip(self._tensors, offsets):
                if pos < off:
                    f.write(b"\0" * (off - pos))
                    pos = off
                arr = data() if callable(data) else data
                raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
                if raw.size != nbytes:
                    raise GGUFError(f"{name}: got {raw.size} bytes, expected {nbytes} for {tinfo.name}{shape}")
                f.write(raw.tobytes() if raw.size < (1 << 20) else memoryview(raw))
                pos += nbytes
            end = _align_up(pos, self.alignment)
            f.write(b"\0" * (end - pos))
            return data_start + end


# HF decoder tensor name -> GGUF name (mirrors the table at gguf.rs:791-848).
_HF_LAYER_MAP = {
    "input_layernorm.weight": "attn_norm.weight",
    "self_attn.q_proj.weight": "attn_q.weight",
    "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight",
    "self_attn.o_proj.weight": "attn_output.weight",
    "self_attn.qkv_proj.weight": "attn_qkv.weight",  # Phi-3: fused projections, kept fused in the file
    "mlp.gate_up_proj.weight": "ffn_up.weight",      # Phi-3: gate rows then up rows
    "self_attn.q_proj.bias": "attn_q.bias",
    "self_attn.k_proj.bias": "attn_k.bias",
    "self_attn.v_proj.bias": "attn_v.bias",
    # latent attention (DeepSeek-V2/V3)
    "self_attn.q_a_proj.weight": "attn_q_a.weight",
    "self_attn.q_a_layernorm.weight": "attn_q_a_norm.weight",
    "self_attn.q_b_proj.weight": "attn_q_b.weight",
    "self_attn.kv_a_proj_with_mqa.weight": "attn_kv_a_mqa.weight",
    "self_attn.kv_a_layernorm.weight": "attn_kv_a_norm.weight",
    "self_attn.kv_b_proj.weight": "attn_kv_b.weight",
    "self_attn.q_norm.weight": "attn_q_norm.weight",
    "self_attn.k_norm.weight": "attn_k_norm.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight",
    "mlp.up_proj.weight": "ffn_up.weight",
    "mlp.down_proj.weight": "ffn_down.weight",
    "mlp.gate.weight": "ffn_gate_inp.weight",
    "block_sparse_moe.gate.weight": "ffn_gate_inp.weight",
    "mlp.shared_expert.gate_proj.weight": "ffn_gate_shexp.weight",
    "mlp.shared_expert.up_proj.weight": "ffn_up_shexp.weight",
    "mlp.shared_expert.down_proj.weight": "ffn_down_shexp.weight",
    "mlp.shared_experts.gate_proj.weight": "ffn_gate_shexp.weight",
    "mlp.shared_experts.up_proj.weight": "ffn_up_shexp.weight",
    "mlp.shared_experts.down_proj.weight": "ffn_down_shexp.weight",
    "mlp.shared_expert_gate.weight": "ffn_gate_inp_shexp.weight",
    "mlp.gate.e_score_correction_bias": "exp_probs_b.bias",
    "block_sparse_moe.e_score_correction_bias": "exp_probs_b.bias",
}
# Gemma-2 / Gemma-3 name their four per-layer norms differently: post_attention_layernorm is the norm on the attention
# branch's OUTPUT there (elsewhere it is the norm in front of the FFN)
_HF_LAYER_MAP_GEMMA = {
    "post_attention_layernorm.weight": "post_attention_norm.weight",
    "pre_feedforward_layernorm.weight": "ffn_norm.weight",
    "post_feedforward_layernorm.weight": "post_ffw_norm.weight",
}
# GLM-4: norms on both branch outputs as well, gate and up projection in one tensor (gate rows first)
_HF_LAYER_MAP_GLM4 = {
    "post_self_attn_layernorm.weight": "post_attention_norm.weight",
    "post_mlp_layernorm.weight": "post_ffw_norm.weight",
    "mlp.gate_up_proj.weight": "ffn_up.weight",
}
# Hunyuan: norms on the rotated q / k heads, router under gate.wg, an always-on shared MLP
_HF_LAYER_MAP_HUNYUAN = {
    "self_attn.query_layernorm.weight": "attn_q_norm.weight",
    "self_attn.key_layernorm.weight": "attn_k_norm.weight",
    "mlp.gate.wg.weight": "ffn_gate_inp.weight",
    "mlp.shared_mlp.gate_proj.weight": "ffn_gate_shexp.weight",
    "mlp.shared_mlp.up_proj.weight": "ffn_up_shexp.weight",
    "mlp.shared_mlp.down_proj.weight": "ffn_down_shexp.weight",
}
# Qwen3.5 gated-delta-rule layers, under the names llama.cpp's converter gives them
_HF_LAYER_MAP_QWEN35 = {
    "linear_attn.in_proj_qkv.weight": "attn_qkv.weight",
    "linear_attn.in_proj_z.weight": "attn_gate.weight",
    "linear_attn.in_proj_a.weight": "ssm_alpha.weight",
    "linear_attn.in_proj_b.weight": "ssm_beta.weight",
    "linear_attn.conv1d.weight": "ssm_conv1d.weight",
    "linear_attn.dt_bias": "ssm_dt.bias",
    "linear_attn.A_log": "ssm_a",
    "linear_attn.norm.weight": "ssm_norm.weight",
    "linear_attn.out_proj.weight": "ssm_out.weight",
    "post_attention_layernorm.weight": "post_attention_norm.weight",  # the norm in front of the feed-forward block
}
# LFM2: operator norm, short-convolution tensors, w1 / w3 / w2 feed-forward names, RMSNorm on q / k heads
_HF_LAYER_MAP_LFM2 = {
    "operator_norm.weight": "attn_norm.weight",
    "ffn_norm.weight": "ffn_norm.weight",
    "self_attn.out_proj.weight": "attn_output.weight",
    "self_attn.q_layernorm.weight": "attn_q_norm.weight",
    "self_attn.k_layernorm.weight": "attn_k_norm.weight",
    "feed_forward.w1.weight": "ffn_gate.weight",
    "feed_forward.w3.weight": "ffn_up.weight",
    "feed_forward.w2.weight": "ffn_down.weight",
    "conv.in_proj.weight": "shortconv.in_proj.weight",
    "conv.conv.weight": "shortconv.conv.weight",
    "conv.out_proj.weight": "shortconv.out_proj.weight",
    # LFM2-MoE: router, and the per-expert bias that only steers which experts are picked
    "feed_forward.gate.weight": "ffn_gate_inp.weight",
    "feed_forward.expert_bias": "exp_probs_b.bias",
}
# Mamba (``backbone.layers.N.*``): the norm in front of the mixer and the mixer's tensors
_HF_MAMBA_TOP = {"backbone.embeddings.weight": "token_embd.weight", "backbone.norm_f.weight": "output_norm.weight",
                 "lm_head.weight": "output.weight"}
_HF_MAMBA_LAYER = {
    "norm.weight": "attn_norm.weight",
    "mixer.in_proj.weight": "ssm_in.weight",
    "mixer.conv1d.weight": "ssm_conv1d.weight",
    "mixer.conv1d.bias": "ssm_conv1d.bias",
    "mixer.x_proj.weight": "ssm_x.weight",
    "mixer.dt_proj.weight": "ssm_dt.weight",
    "mixer.dt_proj.bias": "ssm_dt.bias",
    "mixer.A_log": "ssm_a",
    "mixer.D": "ssm_d",
    "mixer.out_proj.weight": "ssm_out.weight",
}
_HF_MAMBA_RE = re.compile(r"^backbone\.layers\.(\d+)\.(.+)$")
_HF_TOP_MAP = {
    "model.embed_tokens.weight": "token_embd.weight",
    "model.norm.weight": "output_norm.weight",
    "lm_head.weight": "output.weight",
}
_HF_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.+)$")
_HF_EXPERT_RE = re.compile(r"^(?:mlp|block_sparse_moe|feed_forward)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj|w1|w2|w3)\.weight$")
_EXPERT_KIND = {"gate_proj": "gate", "w1": "gate", "up_proj": "up", "w3": "up", "down_proj": "down", "w2": "down"}


def map_hf_tensor_name(name: str, arch: Optional[str] = None) -> Optional[Tuple[str, Optional[int]]]:
    """Map a HF decoder tensor name to ``(gguf_name, expert_index)``.

    Per-expert HF tensors map to the stacked ``blk.N.ffn_{gate,up,down}_exps.weight`` and
    return the expert index to stack at; everything else returns ``None`` for the index.
    Unknown names return ``None``.  ``arch`` (the GGUF architecture string) selects the Gemma-2/3 norm names.
    """
    if "language_model." in name:  # text tower of a multimodal checkpoint, under one of several wrappers
        name = name.replace("language_model.", "")
        while name.startswith("model.model."):
            name = name[len("model."):]
    if arch == "mamba":
        if name in _HF_MAMBA_TOP:
            return _HF_MAMBA_TOP[name], None
        mm = _HF_MAMBA_RE.match(name)
        return (f"blk.{mm.group(1)}.{_HF_MAMBA_LAYER[mm.group(2)]}", None) if mm and mm.group(2) in _HF_MAMBA_LAYER else None
    if name in _HF_TOP_MAP:
        return _HF_TOP_MAP[name], None
    if arch in ("lfm2", "lfm2moe") and name == "model.embedding_norm.weight":
        return "token_embd_norm.weight", None  # the norm in front of the head (the name llama.cpp's converter gives it)
    m = _HF_LAYER_RE.match(name)
    if not m:
        return None
    layer, rest = int(m.group(1)), m.group(2)
    if arch in ("gemma2", "gemma3") and rest in _HF_LAYER_MAP_GEMMA:
        return f"blk.{layer}.{_HF_LAYER_MAP_GEMMA[rest]}", None
    if arch in ("lfm2", "lfm2moe") and rest in _HF_LAYER_MAP_LFM2:
        return f"blk.{layer}.{_HF_LAYER_MAP_LFM2[rest]}", None
    if arch and arch.startswith("hunyuan") and rest in _HF_LAYER_MAP_HUNYUAN:
        return f"blk.{layer}.{_HF_LAYER_MAP_HUNYUAN[rest]}", None
    if arch in ("qwen35", "qwen35moe") and rest in _HF_LAYER_MAP_QWEN35:
        return f"blk.{layer}.{_HF_LAYER_MAP_QWEN35[rest]}", None
    if arch == "glm4" and rest in _HF_LAYER_MAP_GLM4:
        return f"blk.{layer}.{_HF_LAYER_MAP_GLM4[rest]}", None
    if rest in _HF_LAYER_MAP:
        return f"blk.{layer}.{_HF_LAYER_MAP[rest]}", None
    e = _HF_EXPERT_RE.match(rest)
    if e:
        return f"blk.{layer}.ffn_{_EXPERT_KIND[e.group(2)]}_exps.weight", int(e.group(1))
    return None
