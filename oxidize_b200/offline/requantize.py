"""GGUF → GGUF requantization (the reference's ``oxidize-quantize``, ``oxidize-quantize/src/main.rs:100-126``): every
weight matrix is decoded and re-encoded in the target type (a plain type such as ``Q8_0`` or a mix such as ``Q4_K_M``),
norms / biases / routers / 1-D tensors are copied, metadata is preserved.  Options of the reference kept: appending an
already-encoded tensor (``name:path:dim0,dim1:type``) and extending the context length with YaRN scaling written into
the metadata.  Tensors stream one at a time, so the tool's memory is one tensor, not one model.

    python -m oxidize_b200.offline.requantize --input in.gguf --output out.gguf --target Q4_K_M
"""
from __future__ import annotations

import argparse
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..formats.gguf import GGUFValueType, load_gguf
from .gguf_edit import decode_f32, encode, ggml_type, is_weight_matrix, n_layers_of, rewrite, target_type

TARGETS = ("F32", "F16", "BF16", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL",
           "IQ4_XS", "NVFP4", "Q4_K_M", "Q4_K_S", "Q5_K_M", "Q5_K_S", "Q3_K_M", "Q3_K_S", "Q3_K_L")
# the _S / _M / _L names of llama.cpp are tensor-type mixes; Q4_K_M has its own rule, the others use their base type
_MIX_BASE = {"Q4_K_S": "Q4_K", "Q5_K_M": "Q5_K", "Q5_K_S": "Q5_K", "Q3_K_M": "Q3_K", "Q3_K_S": "Q3_K", "Q3_K_L": "Q3_K"}


def parse_append(spec: str):
    try:
        name, path, dims, type_name = spec.rsplit(":", 3)
        shape = tuple(int(d) for d in dims.split(","))
        ggml_type(type_name.upper())
    except Exception as e:  # noqa: BLE001
        raise ValueError(f"--append-tensor wants name:path:dim0,dim1:type, got {spec!r} ({e})") from None
    return name, path, shape, type_name.upper()


def requantize_gguf(input_path: str, output_path: str, target: str, context_length: Optional[int] = None,
                    yarn_orig_ctx: Optional[int] = None, append_tensors: Sequence[str] = ()) -> Dict[str, int]:
    """Returns ``{type name: tensors written in it}``."""
    target = target.upper()
    if target not in TARGETS:
        raise ValueError(f"unsupported target type {target}; one of {', '.join(TARGETS)}")
    policy = _MIX_BASE.get(target, target)
    g = load_gguf(input_path)
    L = n_layers_of(g)
    arch = g.architecture
    edits = {"general.quantization_version": (2, GGUFValueType.UINT32)}
    if context_length is not None:
        if context_length <= 0:
            raise ValueError("--context-length must be greater than zero")
        orig = yarn_orig_ctx or int(g.arch_get("context_length", 0) or 0)
        if orig <= 0:
            raise ValueError("--yarn-orig-ctx must be greater than zero")
        edits[f"{arch}.context_length"] = (int(context_length), GGUFValueType.UINT32)
        if context_length > orig:
            edits[f"{arch}.rope.scaling.type"] = ("yarn", None)
            edits[f"{arch}.rope.scaling.factor"] = (float(context_length) / float(orig), GGUFValueType.FLOAT32)
            edits[f"{arch}.rope.scaling.original_context_length"] = (int(orig), GGUFValueType.UINT32)
    counts: Dict[str, int] = {}

    def transform(name: str):
        info = g.tensors[name]
        if not is_weight_matrix(g, name):
            counts[info.type.name] = counts.get(info.type.name, 0) + 1
            return None
        t = target_type(policy, g, name, L)
        counts[t] = counts.get(t, 0) + 1
        if t == info.type.name:
            return None
        return (lambda name=name, t=t: encode(decode_f32(g, name), t)), t

    extra = []
    for name, path, shape, type_name in (parse_append(s) for s in append_tensors):
        extra.append((name, (lambda path=path: np.fromfile(path, dtype=np.uint8)), shape, type_name))
        counts[type_name] = counts.get(type_name, 0) + 1
    rewrite(g, output_path, transform, edits, extra=extra)
    return counts


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oxidize quantize", description="Requantize a GGUF checkpoint")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--target", required=True, help=", ".join(TARGETS))
    ap.add_argument("--append-tensor", action="append", default=[], help="name:path:dim0,dim1:type (already encoded bytes)")
    ap.add_argument("--context-length", type=int, default=None, help="extend the context with YaRN scaling in the metadata")
    ap.add_argument("--yarn-orig-ctx", type=int, default=None, help="training context (default: the input's context_length)")
    a = ap.parse_args(argv)
    try:
        counts = requantize_gguf(a.input, a.output, a.target, a.context_length, a.yarn_orig_ctx, a.append_tensor)
    except (ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    print(f"wrote {a.output}: " + ", ".join(f"{n} x {t}" for t, n in sorted(counts.items())))
    return 0


if __name__ == "__main__":
    sys.exit(main())
