"""Reference arm of the benchmark: the UNMODIFIED reference engine, built from a plain copy of its
``oxidize-c`` directory under ``baseline/_ref/`` (``make cuda CUDA_ARCHS=100``), driven through its
stock command line on a synthetic GGUF of the benchmark's shape.

Nothing of this repository's engine runs in this process.  The only thing taken from the package is
the file writer: a child process (``python -m oxidize_b200.utils.synth``) writes the random-init GGUF
(the checkpoint format is shared with the reference, and it needs tokenizer metadata inside the
file), after which the reference binary is the only program that touches the GPU.

The reference's CUDA backend is single-GPU and serves one sequence at a time
(``oxidize-c/src/cli/main.c``: ``oc_cuda_init`` → ``oc_cuda_fast_prefill`` / ``oc_cuda_fast_decode``),
so whatever ``--gpus`` says it uses one GPU, and its output tok/s for a workload of B concurrent
requests is its batch-1 decode rate: requests queue behind each other.  The numbers reported are the
ones the binary prints itself (``prefill: N tokens in Ts`` and ``X tok/s (N tokens in Ts)``), plus the
wall clock of the whole child process.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref", "oxidize-c")
REF_BIN = os.path.join(REF_DIR, "oxidize-c")
REF_SRC = os.environ.get("OXB_REFERENCE_SRC", "/root/reference/oxidize-c")


def build_reference(log=None) -> str:
    """Build the reference C engine with its CUDA backend for sm_100 from an unmodified copy of its
    sources.  Returns "" on success, else the tail of the build output."""
    if os.path.exists(REF_BIN):
        return ""
    if not os.path.isdir(REF_DIR):
        if not os.path.isdir(REF_SRC):
            return f"reference sources not found at {REF_SRC} and no copy under baseline/_ref"
        os.makedirs(os.path.dirname(REF_DIR), exist_ok=True)
        shutil.copytree(REF_SRC, REF_DIR)
    p = subprocess.run(["make", "-j", str(min(32, os.cpu_count() or 4)), "cuda", "CUDA_ARCHS=100"], cwd=REF_DIR,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log:
        with open(log, "w") as f:
            f.write(p.stdout)
    if p.returncode != 0 or not os.path.exists(REF_BIN):
        return "make cuda failed: " + " | ".join(p.stdout.strip().splitlines()[-3:])
    return ""


def _cache_dir(need_bytes: int) -> str:
    """A directory with room for the model file: $OXB_REF_CACHE, else /dev/shm, else /tmp."""
    cands = [os.environ.get("OXB_REF_CACHE"), "/dev/shm", "/tmp"]
    best, best_free = None, -1
    for c in cands:
        if not c or not os.path.isdir(c):
            continue
        free = shutil.disk_usage(c).free
        if free > need_bytes * 1.05 + (8 << 30):
            return os.path.join(c, "oxb_ref_models")
        if free > best_free:
            best, best_free = c, free
    raise OSError(28, f"no space for a {need_bytes / 1e9:.0f} GB model file (largest free: {best_free / 1e9:.0f} GB on {best})")


_SIZES = {  # rough file sizes, to pick a place for the file before writing it
    ("llama3-70b", "BF16"): 144e9, ("llama3-8b", "Q4_K_M"): 5.2e9, ("llama3-8b", "BF16"): 16.1e9,
    ("tiny-llama", "Q4_K_M"): 4e7,
}


def ensure_model(model: str, quant: str, context: int) -> str:
    need = int(_SIZES.get((model, quant.upper()), 20e9))
    d = _cache_dir(need)
    os.makedirs(d, exist_ok=True)
    # The reference's CUDA embedding lookup handles f32 and block-quantized tables only (a bf16 / f16 table
    # fails with "prefill forward failed at token 0 (backend error)"): such models get an f32 table.
    embed = "F32" if quant.upper() in ("BF16", "F16") else None
    path = os.path.join(d, f"{model}-{quant.upper()}{'-embF32' if embed else ''}-ctx{context}.gguf")
    done = path + ".done"
    if os.path.exists(path) and os.path.exists(done):
        return path
    env = dict(os.environ)
    env.pop("RANK", None)
    t0 = time.time()
    p = subprocess.run([sys.executable, "-m", "oxidize_b200.utils.synth", "--preset", model, "--quant", quant, "--out", path,
                        "--context", str(context)] + (["--embed-type", embed] if embed else []), cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True)
    if p.returncode != 0:
        try:
            os.remove(path)
        except OSError:
            pass
        raise RuntimeError("model file synthesis failed: " + " | ".join(p.stdout.strip().splitlines()[-2:]))
    with open(done, "w") as f:
        f.write(f"{time.time() - t0:.1f}\n")
    return path


def make_prompt(n_tokens: int, seed: int = 0) -> str:
    """Text that the file's byte-level vocabulary (no merges) encodes as exactly ``n_tokens`` tokens:
    lower-case words separated by single spaces, one token per character."""
    import random

    r = random.Random(seed)
    out = []
    while len(out) < n_tokens:
        for _ in range(r.randint(2, 9)):
            out.append(r.choice("abcdefghijklmnopqrstuvwxyz"))
        out.append(" ")
    return "".join(out[:n_tokens]).rstrip(" ").ljust(n_tokens, "x")


def run_reference(path: str, prompt_tokens: int, out_tokens: int, ctx: int, device_index: int = 0, timeout: float = 1500.0,
                  backend: str = "cuda"):
    """One request through the stock CLI.  Returns a dict with the binary's own figures."""
    env = dict(os.environ)
    if backend == "cuda":
        env["CUDA_VISIBLE_DEVICES"] = str(device_index)
    cmd = [REF_BIN, "--model", path, "--prompt", make_prompt(prompt_tokens), "--n-predict", str(out_tokens), "--backend",
           backend, "--temperature", "0", "--repeat-penalty", "1", "--ctx", str(ctx)]
    t0 = time.time()
    p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=timeout)
    wall = time.time() - t0
    err = p.stderr
    res = {"returncode": p.returncode, "wall_s": round(wall, 2)}
    m = re.search(r"prompt: (\d+) tokens", err)
    if m:
        res["prompt_tokens"] = int(m.group(1))
    m = re.search(r"prefill: (\d+) tokens in ([0-9.]+)s = ([0-9.]+) tok/s", err)
    if m:
        res["prefill_s"] = float(m.group(2))
        res["prefill_tok_s"] = float(m.group(3))
    m = re.search(r"([0-9.]+) tok/s \((\d+) tokens in ([0-9.]+)s\)", err)
    if m:
        res["decode_tok_s"] = float(m.group(1))
        res["decode_tokens"] = int(m.group(2))
        res["decode_s"] = float(m.group(3))
    res["fast_path"] = "cuda: fast path" in err
    res["on_gpu"] = "model uploaded to GPU" in err
    if p.returncode != 0 or "decode_tok_s" not in res:
        res["error"] = " | ".join((err.strip().splitlines() or ["no output"])[-3:])[:400]
    res["tokens_text"] = p.stdout.strip()[:200]
    return res


def main(args) -> int:
    """Entry used by ``bench.py --impl reference``; prints one JSON line on rank 0."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0  # the reference uses one GPU: the other ranks have nothing to run

    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why[:600]}))
        return 0

    err = build_reference()
    if err:
        return unavailable(err)
    B = args.batch
    mean_prompt = (args.prompt_min + args.prompt_max) // 2
    # the decode rate of the reference does not depend on how many of the output tokens are timed beyond
    # the context growth; --steps bounds the timed tokens so that the arm ends within minutes
    out_tokens = max(8, min(args.out_tokens, args.steps + args.warmup))
    ctx = 1 << (mean_prompt + args.out_tokens + 16 - 1).bit_length()
    try:
        path = ensure_model(args.model, args.quant, ctx)
    except Exception as e:  # no room for the file, synthesis failed, ...
        return unavailable(f"{type(e).__name__}: {e}")
    try:
        r = run_reference(path, mean_prompt, out_tokens, ctx, int(os.environ.get("LOCAL_RANK", "0")))
    except subprocess.TimeoutExpired:
        return unavailable("reference binary did not finish one request within its time limit")
    finally:
        # a file of this size in /dev/shm is host memory the other arm's ranks may need: do not keep it
        if os.path.getsize(path) > (64 << 30) and not os.environ.get("OXB_REF_KEEP"):
            for f in (path, path + ".done"):
                try:
                    os.remove(f)
                except OSError:
                    pass
    if "error" in r:
        return unavailable("reference run failed: " + r["error"])
    tok_s = r["decode_tok_s"]
    # whole request through the CLI process: model upload excluded, prompt processing included
    e2e = r["decode_tokens"] / (r.get("prefill_s", 0.0) + r["decode_s"])
    out = {
        "metric": "output tok/s (box, max over ranks) 70B-shape TP8 bs64; p50 TTFT; bs1 tok/s",
        "impl": "reference", "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": args.gpus, "n_gpus_used": 1,
        "steps": r["decode_tokens"], "warmup": 0, "ms_per_step": round(1e3 / tok_s, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if args.quant.upper() == "BF16" else args.quant,
        "data": "synthetic (random N(0,0.02) weights in a GGUF file, fixed pseudo-random prompt text)",
        "config": {"model": args.model, "global_batch": B,
                   "weights": args.quant + (" (token embedding table f32: the reference's CUDA lookup has no bf16 row kernel)"
                                            if args.quant.upper() in ("BF16", "F16") else ""), "kv_cache": "f16, contiguous (the reference's CUDA KV)",
                   "seq_len": f"prompt {r.get('prompt_tokens', mean_prompt)} + {r['decode_tokens']} generated",
                   "parallelism": "single GPU, one sequence at a time (the reference has no batched or multi-GPU decode)",
                   "same_config": False,
                   "note": f"the {B} concurrent requests queue behind each other, so the box's output tok/s is the batch-1 "
                           "decode rate; timed by the binary's own wall clock around its decode loop"},
        "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                "note": "decode tokens / (prefill + decode) of one request inside the reference's CLI process"},
        "ttft_p50_s": round((B - 1) / 2 * (r["prefill_s"] + args.out_tokens / tok_s) + r["prefill_s"], 3) if "prefill_s" in r else None,
        "ttft_note": f"median over {B} requests served one after the other: (B-1)/2 whole requests (prefill + "
                     f"{args.out_tokens} tokens) ahead, then the request's own prefill",
        "bs1_tok_s": round(tok_s, 2), "prefill_tok_s": r.get("prefill_tok_s"), "fast_path": r["fast_path"],
        "command": "oxidize-c --model <synthetic.gguf> --prompt <text> --n-predict N --backend cuda --temperature 0 "
                   "--repeat-penalty 1 --ctx C", "wall_s": r["wall_s"],
    }
    print(json.dumps(out))
    return 0
