"""LoRA adapters: read one (a PEFT SafeTensors directory or a llama.cpp-style GGUF adapter) and merge it into a GGUF
checkpoint, W' = W + scale * (alpha / r) * B A, re-encoding every touched tensor in its own type (the reference's
``model/lora.rs`` plan and the ``export`` step of ``oxidize-finetuning``).  The merged file is an ordinary checkpoint, so
serving it costs nothing extra.

    python -m oxidize_b200.offline.lora --base base.gguf --adapter adapter_dir --output merged.gguf
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from ..formats.gguf import load_gguf, map_hf_tensor_name
from ..formats.safetensors_io import SafeTensorsFile
from .gguf_edit import decode_f32, encode, rewrite


@dataclass
class LoraPair:
    a: np.ndarray  # [r, in]
    b: np.ndarray  # [out, r]
    scale: float  # alpha / r


_PEFT_RE = re.compile(r"^(?:base_model\.model\.)?(.*)\.lora_([AB])(?:\.default)?\.weight$")


def load_adapter(path: str, arch: Optional[str] = None) -> Dict[str, LoraPair]:
    """GGUF tensor name (``blk.N.attn_q.weight`` ...) → the low-rank pair that applies to it."""
    if os.path.isdir(path) or path.endswith(".safetensors"):
        d = path if os.path.isdir(path) else os.path.dirname(path)
        cfg = {}
        cp = os.path.join(d, "adapter_config.json")
        if os.path.exists(cp):
            with open(cp) as f:
                cfg = json.load(f)
        files = sorted(glob.glob(os.path.join(path, "*.safetensors"))) if os.path.isdir(path) else [path]
        halves: Dict[str, Dict[str, np.ndarray]] = {}
        for p in files:
            st = SafeTensorsFile(p)
            for k in st.keys():
                m = _PEFT_RE.match(k)
                if not m:
                    continue
                mapped = map_hf_tensor_name(m.group(1) + ".weight", arch)
                if mapped is None or mapped[1] is not None:
                    raise ValueError(f"adapter tensor {k} does not map to a tensor of the checkpoint")
                halves.setdefault(mapped[0], {})[m.group(2)] = st.tensor_f32(k)
        out = {}
        for name, h in halves.items():
            if set(h) != {"A", "B"}:
                raise ValueError(f"{name}: adapter has only one of lora_A / lora_B")
            r = h["A"].shape[0]
            alpha = float((cfg.get("alpha_pattern") or {}).get(name, cfg.get("lora_alpha", r)))
            out[name] = LoraPair(h["A"], h["B"], alpha / r)
        return out
    g = load_gguf(path)
    alpha = float(g.get("adapter.lora.alpha", 0.0) or 0.0)
    out = {}
    for n in g.tensors:
        if n.endswith(".lora_a"):
            base = n[: -len(".lora_a")]
            a, b = decode_f32(g, n), decode_f32(g, base + ".lora_b")
            out[base] = LoraPair(a, b, (alpha or a.shape[0]) / a.shape[0])
    return out


def merge_lora_gguf(base_path: str, adapter_path: str, output_path: str, scale: float = 1.0) -> List[str]:
    """Returns the names of the tensors that were changed."""
    g = load_gguf(base_path)
    pairs = load_adapter(adapter_path, g.architecture)
    unknown = [n for n in pairs if n not in g.tensors]
    if unknown:
        raise ValueError(f"adapter targets tensors the checkpoint does not have: {unknown[:4]}")
    for n, p in pairs.items():
        shape = g.tensors[n].shape
        if (p.b.shape[0], p.a.shape[1]) != tuple(shape[-2:]) or p.a.shape[0] != p.b.shape[1]:
            raise ValueError(f"{n}: adapter shapes {p.b.shape} x {p.a.shape} do not fit the weight {shape}")

    def transform(name: str):
        p = pairs.get(name)
        if p is None:
            return None
        t = g.tensors[name].type.name

        def gen():
            w = decode_f32(g, name)
            return encode(w + (scale * p.scale) * (p.b.astype(np.float32) @ p.a.astype(np.float32)), t)

        return gen, t

    rewrite(g, output_path, transform)
    return sorted(pairs)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oxidize lora-merge", description="Merge a LoRA adapter into a GGUF checkpoint")
    ap.add_argument("--base", required=True)
    ap.add_argument("--adapter", required=True, help="PEFT directory / .safetensors file, or a GGUF adapter")
    ap.add_argument("--output", required=True)
    ap.add_argument("--scale", type=float, default=1.0, help="extra multiplier on the adapter's own alpha / r")
    a = ap.parse_args(argv)
    try:
        changed = merge_lora_gguf(a.base, a.adapter, a.output, a.scale)
    except (ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    print(f"wrote {a.output}: {len(changed)} tensors updated")
    return 0


if __name__ == "__main__":
    sys.exit(main())
