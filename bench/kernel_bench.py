#!/usr/bin/env python
"""Micro-benchmarks of the hot kernels on the shapes of the headline config, with roofline
fractions against the measured peaks in MEASURED_PEAKS.json (fallback 6.65 TB/s, 1.59 PFLOP/s).

    python bench/kernel_bench.py [--what gemm,attn] [--json out.json]

Timing: CUDA events on the launching stream, 5 warm-up launches, then 20 timed launches that
rotate through enough distinct weight / KV copies to exceed the 126 MB L2.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oxidize_b200.ops import cuda as C  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, n_warm=5, n=20):
    """Seconds per launch.  The n launches are captured in one CUDA graph and replayed, so the
    figure is device time, free of the host's per-launch cost (which would hide 3 µs kernels)."""
    for i in range(n_warm):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(n_warm + i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e-3


OPTS = {}  # command-line options shared with the bench functions


def bench_gemm(rows):
    hbm, tf, kind = peaks()
    shapes = [("qkv/tp8", 1280, 8192), ("o/tp8", 8192, 1024), ("gate_up/tp8", 7168, 8192), ("down/tp8", 8192, 3584),
              ("lm_head/tp8", 16032, 8192)]
    only = OPTS.get("shapes")
    for name, N, K in shapes:
        if only and name.split("/")[0] not in only.split(","):
            continue
        copies = max(2, int(400e6 // (N * K * 2)) + 1)
        ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        for T in [int(v) for v in OPTS.get("tokens", "1,16,64,256,2048").split(",")]:
            x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
            out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
            plan = C.gemm_plan(T, N, K)
            t = timeit(lambda i: C.gemm_bf16(x, ws[i % copies], out))
            t_ref = timeit(lambda i: torch.matmul(x, ws[i % copies].t(), out=out))
            by = (N * K + T * K + T * N) * 2
            fl = 2.0 * T * N * K
            roof = max(by / (hbm * 1e9), fl / (tf * 1e12))
            rows.append({"kernel": "gemm_bf16", "shape": name, "T": T, "N": N, "K": K, "us": t * 1e6,
                         "cublas_us": t_ref * 1e6, "GBps": by / t / 1e9, "TFLOPs": fl / t / 1e12,
                         "frac_of_roofline": roof / t, "peaks": kind, "splits": plan["splits"], "tn": plan["tn"]})
            print(rows[-1], flush=True)
        del ws


class _Meta:
    pass


def bench_attn(rows):
    from oxidize_b200.engine.kv_pool import KVCache, KVCacheSpec

    hbm, tf, kind = peaks()
    for (B, ctx, nq, nkv, kvd) in [(64, 1400, 8, 1, "bf16"), (64, 1400, 64, 8, "bf16"), (1, 2048, 8, 1, "bf16"),
                                   (64, 1400, 8, 1, "q8"), (32, 768, 32, 8, "q8")]:
        hd, page = 128, 16
        per = (ctx + page - 1) // page
        layers = max(2, int(300e6 // (B * per * nkv * 2 * page * hd * 2)) + 1)
        kv = KVCache(KVCacheSpec(layers, nkv, hd, page, kvd), B * per + 1, "cuda")
        for d in kv.data:
            if d.dtype == torch.uint8:
                d.random_(0, 255)
            else:
                d.normal_()
        for s in kv.scales:
            if s is not None:
                s.uniform_(0.001, 0.01)
        m = _Meta()
        m.block_tables = (torch.arange(B * per, dtype=torch.int32, device="cuda").view(B, per) + 1).contiguous()
        m.seq_lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        m.query_start = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        m.max_query_len, m.max_seq_len = 1, ctx
        q = torch.randn(B, nq, hd, device="cuda").to(torch.bfloat16)
        if OPTS.get("attn_trace"):
            import ctypes

            trace = torch.zeros(16, dtype=torch.int64, device="cuda")
            C.lib().oxb_set_attn_trace.argtypes = [ctypes.c_void_p]
            C.lib().oxb_set_attn_trace(trace.data_ptr())
            for i in range(3):
                C.paged_attention(q, kv, i % layers, m, hd ** -0.5, 0)
                torch.cuda.synchronize()
            tr = trace.cpu().tolist()
            print("attention phases of CTA 0 (ns): entry->dep wait, ->setup, ->first page, ->pages done, ->drain, ->cta merge, "
                  "->ticket+final", [tr[i + 1] - tr[i] for i in range(7)], flush=True)
            C.lib().oxb_set_attn_trace(None)
        for splits in (None, 1, 2, 4, 8):
            t = timeit(lambda i: C.paged_attention(q, kv, i % layers, m, hd ** -0.5, 0, splits=splits))
            eb = {"bf16": 2, "q8": 1 + 4 / 32}[kvd]
            by = B * ctx * nkv * 2 * hd * eb
            rows.append({"kernel": "paged_attention_decode", "B": B, "ctx": ctx, "nq": nq, "nkv": nkv, "kv": kvd,
                         "splits": splits, "us": t * 1e6, "GBps": by / t / 1e9, "frac_of_hbm": by / t / 1e9 / hbm,
                         "peaks": kind})
            print(rows[-1], flush=True)
        del kv


def small_case(spec: str, launches: int):
    """A handful of eager launches of ONE kernel on a small case (for a profiler capture):
    gemm:TxNxK rotates over weight copies that together exceed the L2; attn:BxCTXxNQxNKV[:kv] walks
    layers of one KV cache the same way.  Device memory stays below 1 GB."""
    kind, _, rest = spec.partition(":")
    if kind == "gemm":
        T, N, K = (int(v) for v in rest.split("x"))
        copies = max(2, int(300e6 // (N * K * 2)) + 1)
        ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
        for i in range(launches):
            C.gemm_bf16(x, ws[i % copies], out)
    elif kind == "attn":
        from oxidize_b200.engine.kv_pool import KVCache, KVCacheSpec

        dims, _, kvd = rest.partition(":")
        B, ctx, nq, nkv = (int(v) for v in dims.split("x"))
        kvd = kvd or "bf16"
        hd, page = 128, 16
        per = (ctx + page - 1) // page
        layers = max(2, int(300e6 // (B * per * nkv * 2 * page * hd * 2)) + 1)
        kv = KVCache(KVCacheSpec(layers, nkv, hd, page, kvd), B * per + 1, "cuda")
        for d in kv.data:
            d.random_(0, 255) if d.dtype == torch.uint8 else d.normal_()
        for sc in kv.scales:
            if sc is not None:
                sc.uniform_(0.001, 0.01)
        m = _Meta()
        m.block_tables = (torch.arange(B * per, dtype=torch.int32, device="cuda").view(B, per) + 1).contiguous()
        m.seq_lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        m.query_start = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        m.max_query_len, m.max_seq_len = 1, ctx
        q = torch.randn(B, nq, hd, device="cuda").to(torch.bfloat16)
        for i in range(launches):
            C.paged_attention(q, kv, i % layers, m, hd ** -0.5, 0)
    elif kind == "mmq":  # mmq:QTYPE:TxNxK  dequant-fused tcgen05 GEMM on packed weights
        from oxidize_b200.models.weights import QTensor
        from oxidize_b200.quant.torch_quant import random_quantized

        qt, _, dims = rest.partition(":")
        T, N, K = (int(v) for v in dims.split("x"))
        copies = 3
        gen = torch.Generator(device="cuda")
        gen.manual_seed(0)
        ws = [random_quantized(N, K, qt, torch.device("cuda"), gen, 0.02) for _ in range(copies)]
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        for i in range(launches):
            C.linear(x, [ws[i % copies]])
    elif kind == "swiglu":  # swiglu:TxFxK  gate_up GEMM with the SwiGLU epilogue
        T, F, K = (int(v) for v in rest.split("x"))
        copies = max(2, int(300e6 // (2 * F * K * 2)) + 1)
        ws = [C.interleave_gate_up((torch.randn(2 * F, K, device="cuda") * 0.02).to(torch.bfloat16)) for _ in range(copies)]
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        for i in range(launches):
            C.linear_swiglu(x, ws[i % copies])
    elif kind == "rmsnorm":  # rmsnorm:TxH  residual add + RMSNorm
        T, H = (int(v) for v in rest.split("x"))
        w = torch.ones(H, device="cuda")
        hs = [torch.randn(T, H, device="cuda").to(torch.bfloat16) for _ in range(4)]
        res = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        for i in range(launches):
            C.add_rmsnorm(hs[i % 4], res, w, 1e-5)
    elif kind == "sample":  # sample:RxV  device sampler (top-k / top-p rows)
        from oxidize_b200.ops import cuda_sampling

        R, V = (int(v) for v in rest.split("x"))
        logits = torch.randn(R, V, device="cuda")
        temp = torch.full((R,), 0.8, device="cuda")
        topk = torch.full((R,), 40, dtype=torch.int32, device="cuda")
        topp = torch.full((R,), 0.9, device="cuda")
        minp = torch.zeros(R, device="cuda")
        rnd = torch.rand(R, device="cuda")
        for i in range(launches):
            cuda_sampling.sample(logits, temp, topk, topp, minp, rnd, "lowest")
    elif kind == "moe":  # moe:TxExKtop  routing kernel
        from oxidize_b200.models.config import ModelConfig
        from oxidize_b200.ops import cuda_moe

        T, E, k = (int(v) for v in rest.split("x"))
        cfg = ModelConfig(n_experts=E, n_experts_used=k)
        logits = torch.randn(T, E, device="cuda")
        scale = torch.empty(E, T, device="cuda")
        for i in range(launches):
            cuda_moe.moe_route(logits, cfg, None, scale, 0, E)
    elif kind == "gemmnorm":  # gemmnorm:TxNxK  folded RMSNorm: producer (accumulate-into + sums of squares), then consumer
        T, N, K = (int(v) for v in rest.split("x"))
        copies = max(2, int(300e6 // (N * K * 2)) + 1)
        ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        wc = [(torch.randn(K, N, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        r = torch.randn(T, N, device="cuda").to(torch.bfloat16)
        acc = torch.zeros(2, T * C.SUMSQ_STRIDE, dtype=torch.int64, device="cuda")
        for i in range(launches):
            C.gemm_bf16(x, ws[i % copies], out=r, add_into=True, sumsq_out=acc[0])
            C.gemm_bf16(r, wc[i % copies], sumsq_in=acc[0], eps=1e-5, clear=acc[1])
            acc[0].zero_()
    elif kind == "moelayer":  # moelayer:PRESETxLOCALxT  routed-expert block: route, dispatch, grouped GEMMs, combine
        from oxidize_b200.models.config import preset
        from oxidize_b200.models.weights import ExpertWeights, QTensor
        from oxidize_b200.ops import cuda_moe

        name, nloc, T = rest.split("x")
        nloc, T = int(nloc), int(T)
        cfg = preset(name)
        H, F = cfg.hidden_size, cfg.expert_ffn_size
        gu = [QTensor("BF16", (torch.randn(2 * F, H, device="cuda") * 0.02).to(torch.bfloat16), (2 * F, H)) for _ in range(nloc)]
        dn = [QTensor("BF16", (torch.randn(H, F, device="cuda") * 0.02).to(torch.bfloat16), (H, F)) for _ in range(nloc)]
        ex = ExpertWeights(gu, dn, 0)
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        logits = torch.randn(T, cfg.n_experts, device="cuda")
        for i in range(launches):
            cuda_moe.moe_layer(x, logits, cfg, None, ex, None, None, True)
    elif kind == "specverify":  # specverify:SxKxV  speculative verification, sampled rows
        S, K, V = (int(v) for v in rest.split("x"))
        i32, f32 = dict(dtype=torch.int32, device="cuda"), dict(dtype=torch.float32, device="cuda")
        tl = torch.randn(S * (K + 1), V, **f32)
        dl = tl.view(S, K + 1, V)[:, :K].reshape(S * K, V) + 0.3 * torch.randn(S * K, V, **f32)
        dtok = dl.argmax(-1).view(S, K).to(torch.int32)
        for i in range(launches):
            C.spec_verify(tl, dl, dtok, torch.arange(S, **i32) * (K + 1), torch.full((S,), K, **i32), torch.full((S,), 0.8, **f32),
                          torch.rand(S, 2 * K + 1, **f32), K)
    else:
        raise SystemExit(f"unknown case {spec}")
    torch.cuda.synchronize()
    print("status", C.status())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,attn")
    ap.add_argument("--json", default="")
    ap.add_argument("--case", default="", help="small case for a profiler: gemm:TxNxK or attn:BxCTXxNQxNKV[:kv]")
    ap.add_argument("--launches", type=int, default=6)
    ap.add_argument("--shapes", default="", help="GEMM shapes to run, by name before the slash (qkv,o,gate_up,down,lm_head)")
    ap.add_argument("--tokens", default="1,16,64,256,2048", help="token counts of the GEMM sweep")
    ap.add_argument("--attn-trace", action="store_true", help="print the in-kernel phase timestamps of attention CTA 0")
    ap.add_argument("--prefill-tn", type=int, default=-1, help="force the token tile of prefill-sized GEMMs (128 / 256 / 0 = auto)")
    a = ap.parse_args()
    OPTS.update(shapes=a.shapes, tokens=a.tokens, attn_trace=a.attn_trace)
    if a.prefill_tn >= 0:
        C.lib().oxb_set_gemm_prefill_tn(a.prefill_tn)
    if a.case:
        small_case(a.case, a.launches)
        return
    rows = []
    if "gemm" in a.what:
        bench_gemm(rows)
    if "attn" in a.what:
        bench_attn(rows)
    print("status", C.status())
    if a.json:
        json.dump(rows, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
