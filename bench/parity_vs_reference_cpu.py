"""Greedy-token parity of this engine's CPU path against the reference's C engine on synthetic F32 checkpoints.

For a handful of small model shapes (dense GQA, partial RoPE, QK-norm, YaRN-scaled RoPE, mixtures of experts) the script writes a random-init GGUF with F32 weights, generates greedily from the same prompts with both
engines and reports whether the generated text agrees.  F32 weights keep the reference on its plain f32 matvec (with
block-quantized weights it multiplies int8-quantized activations, which this engine's fp32 oracle path does not), so
the comparison tests the MODEL SEMANTICS: tensor naming and layout, RoPE pairing, norms, routing, window, KV handling.

    python bench/parity_vs_reference_cpu.py            # needs baseline/_ref/oxidize-c/oxidize-c (python __graft_entry__.py)

Prints one JSON object per case and a summary line.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))


# (seed, prompt length in tokens) of the prompts every case is run on
PROMPTS = [(3, 48), (4, 23), (5, 97), (6, 64), (7, 130), (8, 9)]


def cases():
    from oxidize_b200.models.config import RopeScaling

    base = dict(vocab_size=1000, hidden_size=256, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=32, ffn_size=512,
                context_length=512)
    return {
        "llama-gqa": ("tiny-llama", base),
        "llama-mha-partial-rope": ("tiny-llama", dict(base, n_kv_heads=8, rope_dim=16)),
        "qwen3-qk-norm": ("tiny-llama", dict(base, arch="qwen3", qk_norm=True)),
        # (the reference reads `attention.sliding_window` only for its Gemma-style architectures, so a windowed Llama /
        # Mistral file is not a case the two engines can be compared on)
        # Mixtral checkpoints are written by llama.cpp's converter as architecture "llama" with expert_count set
        "mixtral-moe": ("mixtral-8x7b", dict(base, arch="llama", n_experts=4, n_experts_used=2, expert_ffn_size=256)),
        "qwen3moe": ("qwen3-30b-a3b", dict(base, n_experts=8, n_experts_used=2, expert_ffn_size=128, qk_norm=True)),
        "qwen2-qkv-bias": ("tiny-llama", dict(base, arch="qwen2", attn_bias=True)),
        "mistral": ("tiny-llama", dict(base, arch="mistral", n_kv_heads=4)),
        "llama-yarn-rope": ("tiny-llama", dict(base, rope_scaling=RopeScaling(type="yarn", factor=4.0,
                                                                            original_context_length=32))),
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-bin", default=os.path.join(ROOT, "baseline", "_ref", "oxidize-c", "oxidize-c"))
    ap.add_argument("--prompts", type=int, default=len(PROMPTS))
    ap.add_argument("--decode-tokens", type=int, default=24)
    ap.add_argument("--only", default="", help="comma-separated case names")
    a = ap.parse_args()
    import reference_arm as ra

    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.engine.sampler import SamplingParams
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    if not os.path.exists(a.reference_bin):
        print(json.dumps({"unavailable": f"{a.reference_bin} not built"}))
        return 0
    want = set(filter(None, a.only.split(",")))
    results = {}
    for name, (pname, kw) in cases().items():
        if want and name not in want:
            continue
        cfg = preset(pname, **kw)
        path = os.path.join(tempfile.gettempdir(), f"oxb_parity_{name}.gguf")
        synth_gguf(path, cfg, "F32", seed=7, norm_jitter=0.3)
        llm = LLM.from_gguf(path, EngineConfig(kv_cache_dtype="f32", max_model_len=256, max_num_seqs=1, num_kv_blocks=32,
                                               prefill_chunk_size=64, max_num_batched_tokens=64, enable_prefix_cache=False),
                            device="cpu")
        sp = SamplingParams(temperature=0.0, max_tokens=a.decode_tokens, ignore_eos=True)
        exact, distinct, generated, worst_prefix, err = True, set(), 0, None, None
        # several prompts of different lengths: random-init models soon settle on one token, so the variety of the
        # comparison comes from the first tokens after each prompt
        for seed, n_prompt in PROMPTS[:a.prompts]:
            text = ra.make_prompt(n_prompt, seed=seed)
            ids = llm.tokenizer.encode(text)
            mine = llm.generate([ids], sp)[0].token_ids
            p = subprocess.run([a.reference_bin, "--model", path, "--prompt", text, "--n-predict", str(a.decode_tokens),
                                "--temperature", "0", "--repeat-penalty", "1", "--kv", "f32", "--ctx", "256"],
                               capture_output=True, timeout=600)
            # bytes, decoded here: text mode would turn a generated "\r" byte token into "\n"
            ref_text = p.stdout.decode("utf-8", errors="replace").strip()
            ref_err = p.stderr.decode("utf-8", errors="replace").strip()
            # compare through the text (the vocabulary names every token beyond the byte pieces "<id>")
            mine_text = llm.tokenizer.decode_without_special_tokens(mine).strip()
            n = 0
            while n < min(len(ref_text), len(mine_text)) and ref_text[n] == mine_text[n]:
                n += 1
            if not ref_text:
                err = ref_err.splitlines()[-1][:200] if ref_err else "no output"
            same = bool(ref_text) and ref_text == mine_text
            exact = exact and same
            if not same:
                worst_prefix = n if worst_prefix is None else min(worst_prefix, n)
            distinct |= set(mine)
            generated += len(mine)
        r = {"case": name, "arch": cfg.arch, "exact": exact, "prompts": min(a.prompts, len(PROMPTS)),
             "distinct_tokens": len(distinct), "generated": generated, "shortest_matching_text_prefix": worst_prefix,
             "reference_error": err}
        results[name] = r
        print(json.dumps(r), flush=True)
    print(json.dumps({"exact": sorted(k for k, v in results.items() if v["exact"]),
                      "differ": sorted(k for k, v in results.items() if not v["exact"])}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
