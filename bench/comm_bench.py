#!/usr/bin/env python
"""Micro-benchmark of the fused collectives on the headline shapes (one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29541 bench/comm_bench.py [--tokens 64]

For the two row-parallel projections of the 70B shape it times, per call and as the max over ranks,
  * the plain GEMM (no collective),
  * GEMM + NCCL all-reduce (the baseline),
  * the fused GEMM + all-reduce kernel in both exchanges (one-shot push with flags, two-shot with in-data flags),
and the stand-alone all-reduce of the [tokens, 8192] bf16 tensor (NCCL vs both exchanges).
Each figure is 20 calls captured in one CUDA graph and replayed, timed with CUDA events.
Roofline for the fused kernel: max(GEMM bytes / HBM bandwidth, NVLink bytes / 770 GB/s).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def timeit(fn, n=20, reps=3):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(n):
            fn()
    best = 1e9
    for _ in range(reps):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n * 1e3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        best = min(best, float(t))
    return best  # µs per call, max over ranks, best of reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from oxidize_b200.models.weights import LinearWeight, QTensor
    from oxidize_b200.ops import cuda as C
    from oxidize_b200.parallel.fused import FusedComm

    comm = FusedComm(dev, max_tokens=256, hidden=8192)
    T = a.tokens
    rows = []
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm = json.load(open(p))["hbm_gbs"] if os.path.exists(p) else 6650.0
    for name, N, Kfull in [("attn_output", 8192, 8192), ("ffn_down", 8192, 28672)]:
        K = Kfull // 8  # the TP8 per-rank shape whatever the rank count, so figures compare across N
        x = torch.randn(T, K, device=dev).to(torch.bfloat16)
        ws = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(max(2, int(300e6 // (N * K * 2))))]
        lw = [LinearWeight([QTensor("BF16", w, (N, K))]) for w in ws]
        out = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
        it = [0]

        def plain():
            it[0] += 1
            C.gemm_bf16(x, ws[it[0] % len(ws)], out)

        def nccl():
            it[0] += 1
            C.gemm_bf16(x, ws[it[0] % len(ws)], out)
            dist.all_reduce(out)

        def fused():
            it[0] += 1
            comm.linear_allreduce(x, lw[it[0] % len(lw)])

        r = {"op": f"gemm+allreduce {name}", "T": T, "N": N, "K": K, "world": world, "gemm_us": timeit(plain),
             "gemm_nccl_us": timeit(nccl)}
        for mode, mw in (("oneshot", 99), ("ll", 2)):
            C.lib().oxb_set_ar_ll_min_world(mw)
            r[f"fused_{mode}_us"] = timeit(fused)
        gemm_s = (N * K + T * K + T * N) * 2 / (hbm * 1e9)
        link_s = 2.0 * (world - 1) / world * T * N * 2 / 770e9
        r["roofline_us"] = max(gemm_s, link_s) * 1e6
        rows.append(r)
        del ws, lw
    x = torch.randn(T, 8192, device=dev).to(torch.bfloat16)
    r = {"op": "allreduce", "T": T, "N": 8192, "world": world, "nccl_us": timeit(lambda: dist.all_reduce(x))}
    for mode, mw in (("oneshot", 99), ("ll", 2)):
        C.lib().oxb_set_ar_ll_min_world(mw)
        r[f"fused_{mode}_us"] = timeit(lambda: comm.all_reduce(x))
    rows.append(r)
    # phase latencies of one eager call (piece 0 on this rank), from in-kernel globaltimer stamps
    import ctypes

    trace = torch.zeros(16, dtype=torch.int64, device=dev)
    C.lib().oxb_set_ar_trace.argtypes = [ctypes.c_void_p]
    C.lib().oxb_set_ar_trace(trace.data_ptr())
    phases = {}
    for mode, mw in (("oneshot", 99), ("ll", 2)):
        C.lib().oxb_set_ar_ll_min_world(mw)
        for _ in range(3):
            dist.barrier()
            torch.cuda.synchronize()
            comm.all_reduce(x)
            torch.cuda.synchronize()
        tr = trace.cpu().tolist()
        n = 6 if mode == "oneshot" else 4
        phases[mode] = {"kernel_entry_to_exchange_ns": tr[0] - tr[9], "steps_ns": [tr[i + 1] - tr[i] for i in range(n - 1)],
                        "exchange_end_to_grid_end_ns": tr[10] - tr[n - 1]}
    C.lib().oxb_set_ar_trace(None)
    rows.append({"op": "allreduce phases", "world": world, **phases})
    st = C.status()
    if rank == 0:
        for r in rows:
            print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in r.items()}), flush=True)
        print("status", st, "fused_calls", comm.fused_calls, "fallback_calls", comm.fallback_calls, flush=True)
        if a.json:
            json.dump(rows, open(a.json, "w"), indent=1)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
