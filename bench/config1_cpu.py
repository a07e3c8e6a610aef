#!/usr/bin/env python
"""Benchmark configuration 1: tiny Llama on the CPU, this engine against the reference's C engine.

    python bench/config1_cpu.py [--reference-bin baseline/_ref/oxidize-c/oxidize-c]

Model: vocab 32000, d_model 512, 8 layers, 8 query / 2 KV heads (head_dim 64), SwiGLU FFN 1408, RMSNorm eps 1e-5,
RoPE theta 10000; random N(0, 0.02) weights quantized to GGUF Q4_K (rows that are not whole 256-value super-blocks
fall back to Q8_0, norms f32).  Workload: batch 1, 128 pseudo-random prompt tokens, 128 greedy decode tokens, f16 KV
cache, seed 0.  Both engines read the same file; the prompt is text that the file's byte-level vocabulary turns
into exactly 128 tokens.  Prints one JSON line: the two generated texts must be equal ("token_exact").  The CPU path of this engine is its
fp32 correctness oracle (plain PyTorch statements of every operator), not a tuned CPU engine, so the reference's C
kernels are expected to be faster here; the comparison that matters on this configuration is the tokens.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-bin", default=os.path.join(ROOT, "baseline", "_ref", "oxidize-c", "oxidize-c"))
    ap.add_argument("--prompt-tokens", type=int, default=128)
    ap.add_argument("--decode-tokens", type=int, default=128)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--quant", default="Q4_K", help="encoding of the synthetic checkpoint (Q4_K is the named configuration; "
                    "F32 takes the reference's int8 activation quantisation out of the comparison)")
    a = ap.parse_args()
    import reference_arm as ra

    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.engine.sampler import SamplingParams
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    path = os.path.join(tempfile.gettempdir(), f"oxb_config1_tiny_{a.quant.lower()}.gguf")
    if not os.path.exists(path):
        synth_gguf(path, preset("tiny-llama"), a.quant, seed=0)
    text = ra.make_prompt(a.prompt_tokens, seed=0)
    out = {"config": "tiny Llama %s, CPU, batch 1, %d prompt + %d greedy tokens, f16 KV" % (a.quant, a.prompt_tokens, a.decode_tokens)}
    # ---- this engine
    llm = LLM.from_gguf(path, EngineConfig(kv_cache_dtype="f16", max_model_len=512, max_num_seqs=1, num_kv_blocks=64,
                                           prefill_chunk_size=128, max_num_batched_tokens=128, enable_prefix_cache=False),
                        device="cpu")
    ids = llm.tokenizer.encode(text)
    assert len(ids) == a.prompt_tokens, len(ids)
    sp = SamplingParams(temperature=0.0, max_tokens=a.decode_tokens, ignore_eos=True)
    best = None
    for _ in range(a.iters):
        t0 = time.perf_counter()
        first = None
        rid = llm.add_request(ids, sp)
        toks = []
        while llm.has_unfinished:
            for ro in llm.step():
                if first is None and ro.token_ids:
                    first = time.perf_counter()
                if ro.finished:
                    toks = list(ro.token_ids)
        t1 = time.perf_counter()
        r = {"prefill_tok_s": a.prompt_tokens / (first - t0), "decode_tok_s": (len(toks) - 1) / (t1 - first)}
        if best is None or r["decode_tok_s"] > best["decode_tok_s"]:
            best = r
    out["oxidize_b200"] = {k: round(v, 2) for k, v in best.items()}
    out["oxidize_b200"]["tokens"] = toks[:16]
    # ---- the reference's C engine on the same file
    if os.path.exists(a.reference_bin):
        rbest = None
        rtoks = None
        for _ in range(a.iters):
            p = subprocess.run([a.reference_bin, "--model", path, "--prompt", text, "--n-predict", str(a.decode_tokens),
                                "--temperature", "0", "--repeat-penalty", "1", "--kv", "f32", "--ctx", "512"],
                               capture_output=True, text=True, timeout=600)
            m = re.search(r"([0-9.]+) tok/s \((\d+) tokens", p.stderr)
            pf = re.search(r"prefill: \d+ tokens in [0-9.]+s = ([0-9.]+) tok/s", p.stderr)
            if not m:
                out["reference"] = {"error": p.stderr.strip().splitlines()[-1][:200] if p.stderr.strip() else "no output"}
                break
            r = {"decode_tok_s": float(m.group(1)), "prefill_tok_s": float(pf.group(1)) if pf else None}
            rtoks = [int(x) for x in re.findall(r"<(\d+)>", p.stdout)]
            rtext = p.stdout.strip()
            if rbest is None or r["decode_tok_s"] > rbest["decode_tok_s"]:
                rbest = r
        if rbest is not None:
            out["reference"] = rbest
            out["reference"]["tokens"] = rtoks[:16]
            # the reference prints the text of the generated tokens; this file's vocabulary names every token beyond the
            # 256 byte pieces "<id>", so the text identifies the ids
            out["token_exact"] = rtext == llm.tokenizer.decode_without_special_tokens(toks).strip() and len(rtoks) > 0
            # Random N(0, 0.02) weights give nearly flat logits, and the reference multiplies Q4_K weights with int8
            # activations where this engine's CPU path uses fp32: the first near-tie between two tokens ends the match.
            n = 0
            while n < min(len(rtoks), len(toks)) and rtoks[n] == toks[n]:
                n += 1
            out["matching_prefix_tokens"] = n
            out["decode_speedup_vs_reference"] = round(best["decode_tok_s"] / rbest["decode_tok_s"], 3)
    else:
        out["reference"] = {"unavailable": f"{a.reference_bin} not built"}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
