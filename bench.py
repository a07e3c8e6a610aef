#!/usr/bin/env python
"""Headline benchmark: output tok/s of continuous-batching decode, Llama-3-70B shape, bf16,
64 concurrent requests with paged KV (16-token pages), tensor parallel over N GPUs.

    python bench.py --gpus N --steps K --warmup W          (N>1: launched under torchrun)

One "step" is one engine iteration in the steady state of the workload: every one of the 64
running sequences (contexts = prompt U[256, 2048] + tokens generated so far) produces one
output token.  Two numbers are reported:

* ``value``  — device time of K captured decode steps replayed back to back (CUDA events,
  max over ranks).  Each step streams this rank's whole weight shard (17.6 GB at TP8, 141 GB at
  TP1) plus the KV pages, far more than the 126 MB L2, so no cache flush is needed.
* ``e2e``    — the same K steps through the public ``LLM.step()`` API: host scheduler, pinned
  host → device copy of the step's inputs, forward, sampling, device → host read of the tokens.

Weights are random N(0, 0.02) of the named architecture and prompts are uniform random token
ids (no network for checkpoints or datasets).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="oxidize_b200", choices=["oxidize_b200", "reference"])
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--quant", default="BF16")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=256)
    ap.add_argument("--prompt-max", type=int, default=2048)
    ap.add_argument("--out-tokens", type=int, default=512)
    ap.add_argument("--kv-dtype", default="bf16")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the result invalid)")
    ap.add_argument("--shard-sim", type=int, default=0,
                    help="debug only: run ONE rank's shard shapes of an N-way tensor-parallel job on one GPU, without "
                         "collectives (marks the result invalid); used to profile per-GPU kernels of the TP8 config")
    ap.add_argument("--max-batched-tokens", type=int, default=0,
                    help="token budget of one engine step (prefill chunks + decode rows); 0 = chosen from the per-rank shapes")
    ap.add_argument("--no-prefill", action="store_true",
                    help="fill the KV cache with random pages instead of running the prompts through prefill")
    ap.add_argument("--no-workload", action="store_true",
                    help="skip the whole-workload run (all requests from arrival to their last token)")
    ap.add_argument("--sync-decode", action="store_true", help="do not keep a decode step in flight ahead of the host")
    ap.add_argument("--fold-norms", action="store_true", help="fold RMSNorm into the GEMM epilogues around it (A/B measurement)")
    ap.add_argument("--no-fold-norms", action="store_true", help="keep RMSNorm as stand-alone kernels (the default)")
    ap.add_argument("--expert-quant", default=None, help="encoding of the MoE expert matrices when it differs from --quant")
    ap.add_argument("--draft-model", default=None, help="preset of a draft model: measure speculative decoding as well")
    ap.add_argument("--draft-tokens", type=int, default=4)
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of this rank's GPU while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()
        self.begin = 0.0  # samples older than this (nvidia-smi start-up, warm-up) are dropped

    def mark_begin(self):
        self.begin = time.time()

    def run(self):
        # one nvidia-smi process that prints a line every 100 ms (read-only query), read until told to stop
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                                     str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            return
        self.proc = proc
        try:
            for line in proc.stdout:
                f = [x.strip() for x in line.split(",")]
                if len(f) >= 6:
                    try:
                        self.samples.append((float(f[0]), float(f[1]), f[2], f[3], f[4], f[5], time.time()))
                    except ValueError:
                        pass
                if self.stop_flag.is_set():
                    break
        finally:
            try:
                proc.terminate()
                proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        timed = [s for s in self.samples if s[6] >= self.begin]
        self.samples = timed or self.samples[-1:]
        mhz = sorted(s[0] for s in self.samples)
        reasons = []
        for name, col in (("hw_slowdown", 2), ("hw_thermal_slowdown", 3), ("sw_thermal_slowdown", 4), ("sw_power_cap", 5)):
            if any(s[col].lower().startswith("active") for s in self.samples):
                reasons.append(name)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.samples[0][1], "reasons": reasons,
                "samples": len(self.samples)}


def reference_arm(args):
    """The unmodified reference engine through its own CLI (see baseline/reference_arm.py)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra

    return ra.main(args)


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    # last-resort guard: never sit on a GPU box forever if something blocks
    guard = threading.Timer(1500.0, lambda: os._exit(3))
    guard.daemon = True
    guard.start()
    import torch
    import torch.distributed as dist

    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.engine.sampler import SamplingParams
    from oxidize_b200.models.config import preset
    from oxidize_b200.ops import cuda as C
    from oxidize_b200.parallel.comm import TorchComm, init_distributed
    from oxidize_b200.utils.synth import synth_weights

    layout = init_distributed()
    world, rank = layout.world_size, layout.rank
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun --nproc-per-node {args.gpus}")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = preset(args.model)
    if args.layers:
        cfg.n_layers = args.layers
    if args.shard_sim > 1:
        n = args.shard_sim
        cfg.n_heads //= n
        cfg.n_kv_heads = max(1, cfg.n_kv_heads // n)
        cfg.ffn_size //= n
        cfg.vocab_size //= n
    B = args.batch
    rng = np.random.default_rng(0)
    prompt_lens = rng.integers(args.prompt_min, args.prompt_max + 1, size=B)
    # steady state: every request is somewhere inside its generation
    gen_so_far = rng.integers(0, max(1, args.out_tokens - args.steps - args.warmup - 8), size=B)
    ctx = (prompt_lens + gen_so_far).astype(int)
    total_steps = args.steps * 3 + args.warmup * 3 + 8
    if args.draft_model:
        total_steps += (args.steps + max(2, args.warmup) + 2) * (args.draft_tokens + 1)
    if not args.no_prefill:
        # sequences that finish their prefill early keep decoding while the others are still prefilling
        total_steps += int(ctx.sum()) // 1900 + 8
    max_len = int(max(ctx.max() + total_steps, args.prompt_max + args.out_tokens) + 16)
    page = 16
    nblocks = int(sum((c + total_steps + page) // page + 1 for c in ctx)) + 8
    nblocks_workload = int(sum((p + args.out_tokens + page) // page + 1 for p in prompt_lens)) + 8

    t0 = time.time()
    comm = None
    if world > 1:
        if args.comm == "fused":
            from oxidize_b200.parallel.fused import FusedComm

            comm = FusedComm(dev, max_tokens=max(B, 2048), hidden=cfg.hidden_size)
        else:
            comm = TorchComm()
    weights = synth_weights(cfg, dev, args.quant, seed=0, tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world,
                            expert_quant=args.expert_quant)
    # The whole-workload run needs KV for every request's prompt and all of its output tokens at once; it is run only
    # where that fits beside the weights (it does not beside 141 GB of bf16 weights on a single GPU).
    run_workload = not (args.no_workload or args.no_prefill or args.shard_sim or args.layers)
    if run_workload and nblocks_workload > nblocks:
        kvh = max(1, cfg.n_kv_heads // world)
        bpe = {"bf16": 2, "f16": 2, "f32": 4, "q8": 1.125, "q4": 0.625}.get(args.kv_dtype, 2)
        extra = (nblocks_workload - nblocks) * page * kvh * cfg.head_dim * 2 * bpe * cfg.n_layers
        need_now = nblocks * page * kvh * cfg.head_dim * 2 * bpe * cfg.n_layers
        free_b, _ = torch.cuda.mem_get_info(dev)
        fits = torch.tensor([1 if free_b > need_now + extra + (8 << 30) else 0], device=dev)
        if world > 1:
            dist.all_reduce(fits, op=dist.ReduceOp.MIN)
        if int(fits.item()):
            nblocks = nblocks_workload
        else:
            run_workload = False
    ec = EngineConfig(kv_cache_dtype=args.kv_dtype, kv_page_size=page, num_kv_blocks=nblocks, max_model_len=max_len,
                      max_num_seqs=B, max_num_batched_tokens=(B if args.no_prefill else (max(B, args.max_batched_tokens) if args.max_batched_tokens > 0 else 0)),
                      prefill_chunk_size=512, enable_prefix_cache=False, tp_size=world, ep_size=world,
                      fold_norms=args.fold_norms and not args.no_fold_norms, async_decode=not args.sync_decode)
    llm = LLM(weights, ec, comm)
    torch.cuda.synchronize()
    load_s = time.time() - t0

    # ---- the whole workload: every request from its arrival (all at t = 0) to its last output token
    workload = None
    if run_workload:
        wsp = SamplingParams(temperature=0.0, max_tokens=args.out_tokens, ignore_eos=True)
        wrng = np.random.default_rng(1)
        for i in range(B):
            llm.add_request(wrng.integers(3, cfg.vocab_size, size=int(prompt_lens[i])).tolist(), wsp)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        w_t0 = time.perf_counter()
        w_first, w_done, w_tokens = {}, 0, 0
        while llm.has_unfinished:
            for ro in llm.step():
                if ro.token_ids and ro.request_id not in w_first:
                    w_first[ro.request_id] = time.perf_counter() - w_t0
                if ro.finished:
                    w_done += 1
                    w_tokens += len(ro.token_ids)
        torch.cuda.synchronize()
        w_s = time.perf_counter() - w_t0
        wt = torch.tensor([w_s], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(wt, op=dist.ReduceOp.MAX)
        w_s = float(wt.item())
        workload = {"output_tok_s": round(w_tokens / w_s, 2), "seconds": round(w_s, 3), "requests": w_done,
                    "output_tokens": w_tokens, "prompt_tokens": int(prompt_lens.sum()),
                    "ttft_p50_s": round(float(np.median(list(w_first.values()))), 4) if w_first else None,
                    "ttft_max_s": round(float(max(w_first.values())), 4) if w_first else None,
                    "note": "all requests arrive at t=0; first arrival to last finished token, prefill included, through LLM.step()"}

    sp = SamplingParams(temperature=0.0, max_tokens=total_steps + 8, ignore_eos=True)
    ttft_p50 = None
    prefill_s = None
    if args.no_prefill:
        # place every sequence directly in the running state with a random-filled context
        from oxidize_b200.engine.scheduler import SeqStatus, Sequence

        for kvd in llm.kv.data:
            if kvd.dtype in (torch.bfloat16, torch.float16):
                kvd.normal_(0.0, 1.0)
        for i in range(B):
            toks = rng.integers(3, cfg.vocab_size, size=int(ctx[i])).tolist()
            s = Sequence(toks, sp, arrival=time.perf_counter())
            need = (len(toks) + page) // page
            s.blocks = [llm.pool.allocate() for _ in range(need)]
            s.num_computed = len(toks) - 1
            s.prompt = toks[:-1]
            s.output = [toks[-1]]
            s.status = SeqStatus.RUNNING
            llm.scheduler.running.append(s)
    else:
        for i in range(B):
            llm.add_request(rng.integers(3, cfg.vocab_size, size=int(ctx[i])).tolist(), sp)
        t_pf = time.perf_counter()
        first = {}
        while any(s.remaining_prefill > 0 or not s.output for s in list(llm.scheduler.running) + list(llm.scheduler.waiting)):
            for ro in llm.step():
                if ro.token_ids and ro.request_id not in first:
                    first[ro.request_id] = time.perf_counter() - t_pf
        ttft_p50 = float(np.median(list(first.values()))) if first else None
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t_pf
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- e2e: K steps through the public API (scheduler + H2D + forward + sample + D2H)
    sampler = ClockSampler(local)  # started now so that nvidia-smi is up when the timed regions begin
    sampler.start()
    for _ in range(args.warmup):
        llm.step()
    st0 = dict(llm.stats)
    barrier()
    sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        llm.step()
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), 0.0)
    e2e_wall_ms = (time.perf_counter() - w0) * 1e3
    llm.drain()
    torch.cuda.synchronize()
    st1 = dict(llm.stats)
    h2d = (st1["h2d_bytes"] - st0["h2d_bytes"]) / args.steps
    d2h = (st1["d2h_bytes"] - st0["d2h_bytes"]) / args.steps

    # ---- device-timed: replay the captured decode step K times
    from oxidize_b200.engine.runner import _bucket

    Bk = _bucket(B)
    graph = llm.runner.graphs.get(Bk)
    launches_per_step = getattr(llm.runner, "launches_per_step", {}).get(Bk, 0)
    for _ in range(args.warmup):
        llm.step()
    llm.drain()
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    if graph is not None:
        for _ in range(args.steps):
            graph.replay()
    else:
        for _ in range(args.steps):
            llm.step()
    k1.record()
    barrier()
    dev_ms = k0.elapsed_time(k1)
    sampler.stop_flag.set()
    sampler.join(timeout=3)

    # ---- batch 1: the first sequence alone (same engine, same weights), decode step device-timed
    bs1_ms = 0.0
    if llm.scheduler.running:
        keep = llm.scheduler.running[0]
        parked = [s for s in llm.scheduler.running if s is not keep]
        llm.scheduler.running = [keep]
        for _ in range(max(args.warmup, 3)):
            llm.step()
        llm.drain()
        g1 = llm.runner.graphs.get(_bucket(1))
        barrier()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(args.steps):
            if g1 is not None:
                g1.replay()
            else:
                llm.step()
        b1.record()
        barrier()
        bs1_ms = b0.elapsed_time(b1) / args.steps
        llm.scheduler.running = [keep] + parked

    # ---- speculative decoding (draft model of a named shape, random weights): cost structure of draft + verify
    spec_out = None
    if args.draft_model:
        from oxidize_b200.engine.spec import DraftModelProposer, SpecDecoder

        llm.drain()
        dcfg = preset(args.draft_model, vocab_size=cfg.vocab_size)
        dw = synth_weights(dcfg, dev, "BF16", seed=1)
        k = args.draft_tokens
        llm.spec = SpecDecoder(DraftModelProposer(dw, k, B, max_len), k)
        llm.spec.update_health = lambda a, p: (setattr(llm.spec.stats, "proposed", llm.spec.stats.proposed + p),
                                               setattr(llm.spec.stats, "accepted", llm.spec.stats.accepted + a))
        for _ in range(max(2, args.warmup)):
            llm.step()
        barrier()
        n0 = sum(len(s.output) for s in llm.scheduler.running)
        st = llm.spec.stats
        p0, a0, f0 = st.proposed, st.accepted, st.target_forwards
        s0 = time.perf_counter()
        for _ in range(args.steps):
            llm.step()
        barrier()
        sp_s = time.perf_counter() - s0
        emitted = sum(len(s.output) for s in llm.scheduler.running) - n0
        prop, acc, fw = st.proposed - p0, st.accepted - a0, st.target_forwards - f0
        tpf = emitted / max(fw, 1) / max(len(llm.scheduler.running), 1)
        spec_out = {"draft_model": args.draft_model, "draft_tokens": k, "tok_s": round(emitted / sp_s, 2),
                    "acceptance_rate": round(acc / max(prop, 1), 4), "tokens_per_target_forward": round(tpf, 3),
                    "target_forwards_per_s": round(fw / sp_s, 2),
                    # the same step rate if every draft were accepted (k + 1 tokens per sequence and step): the
                    # ceiling that a trained draft approaches; random-init drafts are accepted by chance only
                    "tok_s_at_full_acceptance": round(fw / sp_s * (k + 1) * len(llm.scheduler.running), 2),
                    "acceptance_normalized_tok_s": round(emitted / sp_s / max(tpf, 1e-9), 2)}
        llm.spec = None

    times = torch.tensor([dev_ms, e2e_ms, e2e_wall_ms, bs1_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, e2e_wall_ms, bs1_ms = [float(x) for x in times.tolist()]
    code, detail, count = C.status()
    tokens = B * args.steps
    value = tokens / (dev_ms / 1e3)
    e2e_val = tokens / (max(e2e_ms, e2e_wall_ms) / 1e3)
    if rank == 0:
        out = {
            "metric": "output tok/s (box, max over ranks) 70B-shape TP8 bs64; p50 TTFT; bs1 tok/s",
            "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random N(0,0.02) weights, uniform random token ids)",
            "impl": "oxidize_b200",
            "config": {"model": args.model, "global_batch": B, "seq_len": f"prompt U[{args.prompt_min},{args.prompt_max}] + up to {args.out_tokens} generated",
                       "mean_context": float(ctx.mean()), "parallelism": f"tp{world}" + (f"+ep{world}" if cfg.is_moe else ""),
                       "weights": args.quant + (f" (experts {args.expert_quant})" if args.expert_quant else ""),
                       "kv_cache": f"paged, {page}-token pages, {args.kv_dtype}", "comm": args.comm if world > 1 else "none",
                       "l2_policy": "inputs larger than L2 (weight shard + KV pages streamed every step)",
                       "layers": cfg.n_layers, "valid": not bool(args.layers or args.shard_sim),
                       "async_decode": not args.sync_decode, "step_token_budget": llm.config.max_num_batched_tokens},
            "e2e": {"value": round(e2e_val, 2), "unit": "tok/s", "ms_per_step": round(max(e2e_ms, e2e_wall_ms) / args.steps, 4),
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches_per_step * args.steps) if graph is not None else int(C.launch_count),
            "clocks": sampler.summary(),
            "workload": workload, "speculative": spec_out, "steady_state_prefill_ttft_p50_s": ttft_p50,
            "steady_state_prefill_s": round(prefill_s, 4) if prefill_s else None,
            "ttft_p50_s": workload["ttft_p50_s"] if workload else ttft_p50, "bs1_tok_s": round(1e3 / bs1_ms, 2) if bs1_ms > 0 else None,
            "bs1_ms_per_step": round(bs1_ms, 4), "load_s": round(load_s, 1),
            "device_status": {"code": code, "detail": detail, "count": count},
        }
        print(json.dumps(out))
    sys.stdout.flush()
    sys.stderr.flush()
    # Orderly shutdown: the step in flight and the captured graphs go first, then the peer mappings (after a barrier),
    # then the process group.  A watchdog ends the process if a peer has already gone and the teardown cannot finish.
    if world > 1:
        bye = threading.Timer(30.0, lambda: os._exit(0))
        bye.daemon = True
        bye.start()
    llm.close()
    if world > 1:
        if hasattr(comm, "close"):
            comm.close()
        else:
            dist.barrier()
        del llm
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
