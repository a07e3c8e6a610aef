"""Shared plumbing of the GGUF-to-GGUF tools: copy metadata with its stored value types, walk the tensors, decode a
weight to float32 and encode it again, and decide which tensors are "weights" at all."""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional, Tuple

import numpy as np

from ..formats.gguf import GGUFFile, GGUFWriter, ggml_type
from ..quant import ref as qref
from ..utils.synth import pick_type

# tensors that stay as they are in every tool unless asked otherwise: 1-D tensors, norms, biases, routers, rotary tables
NEVER_TOUCH = ("norm", ".bias", "ffn_gate_inp", "rope_freqs", "rope_factors")


def is_weight_matrix(g: GGUFFile, name: str) -> bool:
    info = g.tensors[name]
    return len(info.shape) >= 2 and not any(k in name for k in NEVER_TOUCH)


def tensor_kind(name: str) -> str:
    """The projection kind a tensor name stands for (``attn_q``, ``ffn_down``, ``token_embd``, ``output`` ...): what the
    mixed-precision policies key on."""
    parts = name.split(".")
    base = parts[-2] if len(parts) >= 3 else parts[0]
    return base.replace("_exps", "").replace("_shexp", "")


def layer_of(name: str) -> int:
    parts = name.split(".")
    return int(parts[1]) if parts[0] == "blk" and len(parts) > 1 and parts[1].isdigit() else 0


def copy_metadata(g: GGUFFile, w: GGUFWriter, skip: Iterable[str] = ()) -> None:
    skip = set(skip) | {"general.architecture", "general.alignment"}
    for key, value in g.metadata.items():
        if key in skip:
            continue
        w.add(key, value, g.metadata_types.get(key))


def decode_f32(g: GGUFFile, name: str) -> np.ndarray:
    info = g.tensors[name]
    x = qref.dequantize(info.type.name, np.ascontiguousarray(g.tensor_bytes(name)), info.n_elements)
    return np.asarray(x, dtype=np.float32).reshape(info.shape)


def encode(x: np.ndarray, type_name: str) -> np.ndarray:
    type_name = type_name.upper()
    if type_name == "F32":
        return np.ascontiguousarray(x, dtype=np.float32)
    return qref.quantize(type_name, np.ascontiguousarray(x, dtype=np.float32).reshape(-1))


def target_type(policy: str, g: GGUFFile, name: str, n_layers: int) -> str:
    info = g.tensors[name]
    return pick_type(policy, tensor_kind(name), layer_of(name), n_layers, info.shape[-1])


def rewrite(g: GGUFFile, out_path: str, transform: Callable[[str], Optional[Tuple[Callable[[], np.ndarray], str]]],
            metadata_edits: Optional[Dict[str, Tuple[object, Optional[int]]]] = None, drop: Iterable[str] = (),
            extra: Iterable[Tuple[str, Callable[[], np.ndarray], Tuple[int, ...], str]] = ()) -> GGUFWriter:
    """Stream ``g`` into ``out_path``.  ``transform(name)`` returns ``(lazy bytes, type name)`` for a tensor that changes
    and None for one that is copied verbatim; tensors named in ``drop`` are left out; ``extra`` tensors
    ``(name, lazy bytes, shape, type name)`` are appended.  Returns the writer after writing."""
    w = GGUFWriter(out_path, arch=g.architecture, alignment=g.alignment)
    copy_metadata(g, w)
    for key, (value, vtype) in (metadata_edits or {}).items():
        w.add(key, value, vtype)
    dropped = set(drop)
    for name, info in g.tensors.items():
        if name in dropped:
            continue
        t = transform(name)
        if t is None:
            w.add_tensor(name, (lambda name=name: np.ascontiguousarray(g.tensor_bytes(name))), info.shape, info.type.name)
        else:
            gen, type_name = t
            w.add_tensor(name, gen, info.shape, type_name)
    for name, gen, shape, type_name in extra:
        w.add_tensor(name, gen, shape, type_name)
    w.write()
    return w


def n_layers_of(g: GGUFFile) -> int:
    return int(g.arch_get("block_count", 0) or 0) or (1 + max([layer_of(n) for n in g.tensors] or [0]))


__all__ = ["is_weight_matrix", "tensor_kind", "layer_of", "copy_metadata", "decode_f32", "encode", "target_type", "rewrite",
           "n_layers_of", "ggml_type"]
