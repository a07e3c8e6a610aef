"""Merge two SafeTensors checkpoints of the same architecture by linear or spherical (SLERP) interpolation (the
reference's ``oxidize-merge``, ``oxidize-merge/src/main.rs:8-80``, ``blend.rs``, ``recipe.rs``, ``writer.rs``).

The blend weight ``t`` (0 = model A, 1 = model B) can be set per tensor category (attention, MLP / experts, everything
else) or globally; integer tensors and tensors present on one side only follow the ``missing`` policy.  Inputs are a
``.safetensors`` file or a Hugging Face directory (sharded or not); the output is one file, or a directory with shards of
at most ``max_shard_gib`` and a ``model.safetensors.index.json`` (``config.json`` and tokenizer files are copied from A).

    python -m oxidize_b200.offline.merge --a dirA --b dirB --output merged/ --method slerp --t 0.5
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import shutil
import sys
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..formats.safetensors_io import SafeTensorsFile, save_file

PRESETS = {  # (attention_t, mlp_t, other_t)
    "balanced": (0.5, 0.5, 0.5),
    "keep-a-attention": (0.1, 0.5, 0.3),
    "keep-b-attention": (0.9, 0.5, 0.7),
}
_FLOAT = ("F32", "F16", "BF16", "F64")


def open_checkpoint(path: str) -> Dict[str, Tuple[SafeTensorsFile, str]]:
    files = sorted(glob.glob(os.path.join(path, "*.safetensors"))) if os.path.isdir(path) else [path]
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {path}")
    out: Dict[str, Tuple[SafeTensorsFile, str]] = {}
    for p in files:
        f = SafeTensorsFile(p)
        for k in f.keys():
            out[k] = (f, k)
    return out


def category(name: str) -> str:
    if any(k in name for k in ("self_attn", "attention", ".attn.", "attn_")):
        return "attention"
    if any(k in name for k in ("mlp", "experts", "feed_forward", "ffn")):
        return "mlp"
    return "other"


def slerp(a: np.ndarray, b: np.ndarray, t: float, eps: float = 1e-6) -> np.ndarray:
    """Spherical interpolation of two tensors seen as vectors; falls back to linear interpolation when they are (anti-)
    parallel or one of them is zero.  The norm is interpolated linearly, the direction along the great circle."""
    af, bf = a.reshape(-1).astype(np.float64), b.reshape(-1).astype(np.float64)
    na, nb = np.linalg.norm(af), np.linalg.norm(bf)
    if na < eps or nb < eps:
        return ((1 - t) * a + t * b).astype(np.float32)
    cos = float(np.clip(np.dot(af / na, bf / nb), -1.0, 1.0))
    if abs(cos) > 1.0 - 1e-6:
        return ((1 - t) * a + t * b).astype(np.float32)
    omega = np.arccos(cos)
    so = np.sin(omega)
    direction = (np.sin((1 - t) * omega) / so) * (af / na) + (np.sin(t * omega) / so) * (bf / nb)
    return (direction * ((1 - t) * na + t * nb)).reshape(a.shape).astype(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + 0x7FFF + ((u >> 16) & 1)  # round to nearest, ties to even
    return np.where(np.isnan(x), 0x7FC0, rounded >> 16).astype(np.uint16)


def _store(x: np.ndarray, dtype: str):
    if dtype == "BF16":
        return f32_to_bf16_bits(x), "BF16"
    return x.astype({"F32": np.float32, "F16": np.float16, "F64": np.float64}[dtype]), None


def merge_checkpoints(a_path: str, b_path: str, output: Optional[str], method: str = "slerp", t: Optional[float] = None,
                      attention_t: float = 0.3, mlp_t: float = 0.5, other_t: float = 0.4, preset: Optional[str] = None,
                      missing: str = "error", max_shard_gib: float = 5.0, dry_run: bool = False) -> Dict[str, object]:
    if method not in ("linear", "slerp"):
        raise ValueError("method must be linear or slerp")
    if missing not in ("error", "keep-a", "keep-b", "skip"):
        raise ValueError("missing must be error, keep-a, keep-b or skip")
    if preset is not None:
        if preset not in PRESETS:
            raise ValueError(f"preset must be one of {sorted(PRESETS)}")
        attention_t, mlp_t, other_t = PRESETS[preset]
    weights = {"attention": attention_t, "mlp": mlp_t, "other": other_t}
    if t is not None:
        weights = {k: t for k in weights}
    for v in weights.values():
        if not 0.0 <= v <= 1.0:
            raise ValueError("blend weights must be in [0, 1]")
    A, B = open_checkpoint(a_path), open_checkpoint(b_path)
    names = list(A) + [n for n in B if n not in A]
    plan: List[Tuple[str, str]] = []  # (name, action)
    for n in names:
        if n in A and n in B:
            fa, fb = A[n][0], B[n][0]
            if fa.shape(n) != fb.shape(n):
                raise ValueError(f"{n}: shapes differ, {fa.shape(n)} vs {fb.shape(n)}")
            plan.append((n, "blend" if fa.dtype(n) in _FLOAT and fb.dtype(n) in _FLOAT else "a"))
        elif missing == "error":
            raise ValueError(f"{n} exists in only one checkpoint (see --missing)")
        elif missing == "skip":
            continue
        elif n in A and missing == "keep-a":
            plan.append((n, "a"))
        elif n in B and missing == "keep-b":
            plan.append((n, "b"))
    report = {"tensors": len(plan), "blended": sum(1 for _, act in plan if act == "blend"), "weights": weights}
    if dry_run:
        return report

    def produce(name: str, action: str):
        if action != "blend":
            f = (A if action == "a" else B)[name][0]
            arr = f.tensor(name)
            return np.ascontiguousarray(arr), ("BF16" if f.dtype(name) == "BF16" else None)
        fa, fb = A[name][0], B[name][0]
        tt = weights[category(name)]
        xa, xb = fa.tensor_f32(name), fb.tensor_f32(name)
        y = slerp(xa, xb, tt) if method == "slerp" else ((1 - tt) * xa + tt * xb).astype(np.float32)
        return _store(y, fa.dtype(name))

    single = not (os.path.isdir(output) or not output.endswith(".safetensors"))
    meta = {"format": "pt", "merge_method": method}
    if single:
        tensors, dtypes = {}, {}
        for n, act in plan:
            arr, mark = produce(n, act)
            tensors[n] = arr
            if mark:
                dtypes[n] = mark
        save_file(tensors, output, meta, dtypes)
        report["files"] = [output]
        return report
    os.makedirs(output, exist_ok=True)
    limit = int(max_shard_gib * (1 << 30))
    shards: List[List[Tuple[str, str]]] = [[]]
    size = 0
    for n, act in plan:
        f = (B if act == "b" else A)[n][0]
        nbytes = int(np.prod(f.shape(n)) if f.shape(n) else 1) * f.tensor(n).dtype.itemsize
        if shards[-1] and size + nbytes > limit:
            shards.append([])
            size = 0
        shards[-1].append((n, act))
        size += nbytes
    index = {"metadata": {"merge_method": method}, "weight_map": {}}
    files = []
    for i, group in enumerate(shards):
        fname = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        tensors, dtypes = {}, {}
        for n, act in group:
            arr, mark = produce(n, act)
            tensors[n] = arr
            if mark:
                dtypes[n] = mark
            index["weight_map"][n] = fname
        save_file(tensors, os.path.join(output, fname), meta, dtypes)
        files.append(os.path.join(output, fname))
    if len(shards) > 1:
        with open(os.path.join(output, "model.safetensors.index.json"), "w") as f:
            json.dump(index, f, indent=1)
    if os.path.isdir(a_path):  # the side files that make the directory loadable
        for extra in ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "tokenizer.model",
                      "special_tokens_map.json", "vocab.json", "merges.txt"):
            src = os.path.join(a_path, extra)
            if os.path.exists(src):
                shutil.copy(src, os.path.join(output, extra))
    report["files"] = files
    return report


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oxidize merge", description="Merge two SafeTensors checkpoints (linear or SLERP)")
    ap.add_argument("--a", required=True)
    ap.add_argument("--b", required=True)
    ap.add_argument("--output", help=".safetensors file, or a directory for sharded output")
    ap.add_argument("--method", default="slerp", choices=["linear", "slerp"])
    ap.add_argument("--preset", choices=sorted(PRESETS))
    ap.add_argument("--t", type=float, help="global blend weight toward model B (overrides the per-category weights)")
    ap.add_argument("--attention-t", type=float, default=0.3)
    ap.add_argument("--mlp-t", type=float, default=0.5)
    ap.add_argument("--other-t", type=float, default=0.4)
    ap.add_argument("--missing", default="error", choices=["error", "keep-a", "keep-b", "skip"])
    ap.add_argument("--max-shard-gib", type=float, default=5.0)
    ap.add_argument("--dry-run", action="store_true", help="validate tensor compatibility without writing output")
    a = ap.parse_args(argv)
    try:
        if not a.output and not a.dry_run:
            raise ValueError("--output is required unless --dry-run")
        rep = merge_checkpoints(a.a, a.b, a.output, a.method, a.t, a.attention_t, a.mlp_t, a.other_t, a.preset, a.missing,
                                a.max_shard_gib, a.dry_run)
    except (ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    print(f"{'checked' if a.dry_run else 'merged'} {rep['tensors']} tensors ({rep['blended']} blended) with {rep['weights']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
