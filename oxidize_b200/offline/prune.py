"""GGUF pruning (the reference's ``oxidize-prune``, ``oxidize-prune/src/main.rs:35-100``, ``wanda.rs``, ``mask.rs``):

* ``name-filter``: copy the file keeping / dropping tensors by substring of their names;
* ``magnitude``: in every output row of every weight matrix, zero the ``sparsity`` fraction of smallest ``|w|``;
* ``wanda``: the same with the score ``|w| * ||x||_2`` (Sun et al. 2023), where ``||x||_2`` is the L2 norm of the
  matching input feature over a calibration run (``collect_activation_norms`` or a saved ``.npz``).

Patterns: ``unstructured`` (per row), ``n2of4`` / ``n4of8`` (keep n of every m consecutive inputs; what sparse tensor
cores consume).  Survivors are re-encoded in the tensor's own type, or in ``joint_quantize``'s.  Token embeddings, the
output head, norms and rotary tables are never pruned unless ``keep_name`` says otherwise.

    python -m oxidize_b200.offline.prune --input in.gguf --output out.gguf --method magnitude --sparsity 0.5
"""
from __future__ import annotations

import argparse
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..formats.gguf import load_gguf
from .gguf_edit import decode_f32, encode, is_weight_matrix, n_layers_of, rewrite, target_type

DEFAULT_PROTECTED = ("token_embd", "output", "rope", "norm")
PATTERNS = {"unstructured": None, "n2of4": (2, 4), "n4of8": (4, 8)}


def prune_mask(score: np.ndarray, sparsity: float, pattern: str = "unstructured") -> np.ndarray:
    """Boolean keep-mask of ``score`` [rows, cols]: per row the top (1 - sparsity) fraction, or n of every m columns."""
    if pattern not in PATTERNS:
        raise ValueError(f"pattern must be one of {sorted(PATTERNS)}")
    rows, cols = score.shape
    nm = PATTERNS[pattern]
    if nm is None:
        drop = int(np.floor(cols * sparsity))
        keep = np.ones_like(score, dtype=bool)
        if drop > 0:
            idx = np.argpartition(score, drop - 1, axis=1)[:, :drop]
            np.put_along_axis(keep, idx, False, axis=1)
        return keep
    n, m = nm
    if cols % m:
        raise ValueError(f"{pattern} needs the row length ({cols}) to be a multiple of {m}")
    grp = score.reshape(rows, cols // m, m)
    idx = np.argpartition(grp, m - n - 1, axis=2)[:, :, : m - n]
    keep = np.ones_like(grp, dtype=bool)
    np.put_along_axis(keep, idx, False, axis=2)
    return keep.reshape(rows, cols)


def prune_gguf(input_path: str, output_path: Optional[str], method: str = "name-filter", keep: Sequence[str] = (),
               drop: Sequence[str] = (), sparsity: float = 0.5, pattern: str = "unstructured",
               joint_quantize: Optional[str] = None, keep_name: Sequence[str] = (),
               calibration: Optional[Dict[str, np.ndarray]] = None, dry_run: bool = False) -> Dict[str, object]:
    """Returns a report: tensors kept / removed (name-filter) or pruned with the achieved sparsity per tensor."""
    if method not in ("name-filter", "magnitude", "wanda"):
        raise ValueError("method must be name-filter, magnitude or wanda")
    if not 0.0 <= sparsity < 1.0:
        raise ValueError("sparsity must be in [0, 1)")
    g = load_gguf(input_path)
    if method == "name-filter":
        kept = [n for n in g.tensors if (not keep or any(k in n for k in keep)) and not any(d in n for d in drop)]
        removed = [n for n in g.tensors if n not in set(kept)]
        if not dry_run:
            rewrite(g, output_path, lambda name: None, drop=removed)
        return {"kept": kept, "removed": removed}
    if method == "wanda" and not calibration:
        raise ValueError("wanda needs activation norms (--calibration)")
    protected = tuple(keep_name) or DEFAULT_PROTECTED
    L = n_layers_of(g)
    report: Dict[str, float] = {}

    def pruned(name: str) -> np.ndarray:
        w = decode_f32(g, name)
        flat = w.reshape(-1, w.shape[-1])
        score = np.abs(flat)
        if method == "wanda":
            norms = calibration.get(name)
            if norms is not None:  # tensors the calibration run never saw fall back to magnitude
                score = score * np.asarray(norms, dtype=np.float32)[None, :]
        mask = prune_mask(score, sparsity, pattern)
        report[name] = 1.0 - float(mask.mean())
        return (flat * mask).reshape(w.shape)

    def transform(name: str):
        if not is_weight_matrix(g, name) or any(p in name for p in protected):
            return None
        t = target_type(joint_quantize, g, name, L) if joint_quantize else g.tensors[name].type.name
        if dry_run:
            report[name] = sparsity
            return None
        return (lambda name=name, t=t: encode(pruned(name), t)), t

    if dry_run:
        for n in g.tensors:
            transform(n)
    else:
        rewrite(g, output_path, transform)
    return {"pruned": report}


def collect_activation_norms(llm, prompts: Sequence[Sequence[int]]) -> Dict[str, np.ndarray]:
    """Run ``prompts`` (token id lists) through a CPU engine and return, per GGUF weight name, the L2 norm of every input
    feature over all calibration tokens: the statistic Wanda multiplies ``|w|`` by.  Routed experts see only their own
    tokens in the model; here they all get the norms of the block's input, which is what their router saw."""
    import torch

    from .. import ops

    model = llm.model
    names: Dict[int, List[str]] = {}
    for i, lw in enumerate(model.w.layers):
        p = f"blk.{model.w.first_layer + i}"
        if lw.wqkv is not None:
            names[id(lw.wqkv)] = [f"{p}.attn_q.weight", f"{p}.attn_k.weight", f"{p}.attn_v.weight", f"{p}.attn_qkv.weight"]
        names[id(lw.wo)] = [f"{p}.attn_output.weight"]
        if lw.w_gate_up is not None:
            names[id(lw.w_gate_up)] = [f"{p}.ffn_gate.weight", f"{p}.ffn_up.weight"]
            names[id(lw.w_down)] = [f"{p}.ffn_down.weight"]
        if lw.router is not None:
            names[id(lw.router)] = [f"{p}.ffn_gate_exps.weight", f"{p}.ffn_up_exps.weight", f"{p}.ffn_gate_shexp.weight",
                                    f"{p}.ffn_up_shexp.weight"]
    sums: Dict[str, torch.Tensor] = {}
    real = ops.linear

    def spy(x, w, *a, **kw):
        for n in names.get(id(w), ()):
            s = x.detach().float().pow(2).sum(dim=0)
            sums[n] = sums[n] + s if n in sums else s
        return real(x, w, *a, **kw)

    from ..engine.sampler import SamplingParams
    from ..models import transformer as tr

    ops.linear, tr.ops.linear = spy, spy
    try:
        llm.generate([list(p) for p in prompts], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    finally:
        ops.linear = tr.ops.linear = real
    return {n: s.sqrt().cpu().numpy() for n, s in sums.items()}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oxidize prune", description="Copy a GGUF, pruning weights by Wanda, magnitude, or tensor name")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output")
    ap.add_argument("--method", default="name-filter", choices=["name-filter", "wanda", "magnitude"])
    ap.add_argument("--keep", action="append", default=[], help="keep only tensors whose names contain this (name-filter)")
    ap.add_argument("--drop", action="append", default=[], help="drop tensors whose names contain this (name-filter)")
    ap.add_argument("--calibration", help=".npz of per-tensor input-feature L2 norms (wanda); see --calibrate")
    ap.add_argument("--calibrate", help="text file, one calibration prompt per line: compute the norms with the CPU engine "
                                        "and save them to --calibration")
    ap.add_argument("--sparsity", type=float, default=0.5)
    ap.add_argument("--pattern", default="unstructured", choices=sorted(PATTERNS))
    ap.add_argument("--joint-quantize", help="re-quantize the survivors to this type (default: the tensor's own)")
    ap.add_argument("--keep-name", action="append", default=[], help="names (substring) never pruned; default token_embd, "
                                                                      "output, rope, norm")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    try:
        if a.calibrate:
            from ..engine.llm import LLM, EngineConfig

            llm = LLM.from_gguf(a.input, EngineConfig(max_model_len=2048, max_num_seqs=4), device="cpu")
            with open(a.calibrate) as f:
                prompts = [llm.tokenizer.encode(line.strip()) for line in f if line.strip()]
            norms = collect_activation_norms(llm, prompts)
            if not a.calibration:
                raise ValueError("--calibrate needs --calibration to say where the norms go")
            np.savez(a.calibration, **norms)
            print(f"wrote {a.calibration}: {len(norms)} tensors")
            if not a.output and not a.dry_run:
                return 0
        calib = dict(np.load(a.calibration)) if (a.calibration and a.method == "wanda") else None
        if not a.output and not a.dry_run:
            raise ValueError("--output is required unless --dry-run")
        rep = prune_gguf(a.input, a.output, a.method, a.keep, a.drop, a.sparsity, a.pattern, a.joint_quantize, a.keep_name,
                         calib, a.dry_run)
    except (ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if "kept" in rep:
        print(f"kept {len(rep['kept'])} tensors, removed {len(rep['removed'])}")
        for n in rep["removed"]:
            print(f"  - {n}")
    else:
        pr = rep["pruned"]
        mean = sum(pr.values()) / max(1, len(pr))
        print(f"{'would prune' if a.dry_run else 'pruned'} {len(pr)} tensors, mean sparsity {mean:.3f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
