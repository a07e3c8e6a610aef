"""Child process of the multi-rank tests (launched with torch.distributed.run).

    python -m torch.distributed.run --nproc-per-node N tests/mp_worker.py <case> [--device cpu|cuda]

Every case prints ``RANK r OK <case>`` on success and exits non-zero on failure.
"""
import argparse
import os
import sys
import tempfile

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxidize_b200.engine.llm import LLM, EngineConfig  # noqa: E402
from oxidize_b200.engine.sampler import SamplingParams  # noqa: E402
from oxidize_b200.formats.gguf import load_gguf  # noqa: E402
from oxidize_b200.models.config import config_from_gguf, preset  # noqa: E402
from oxidize_b200.models.weights import load_weights  # noqa: E402
from oxidize_b200.parallel.comm import TorchComm, init_distributed  # noqa: E402
from oxidize_b200.utils.synth import synth_gguf  # noqa: E402


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def make_comm(kind, dev):
    if kind == "fused":
        from oxidize_b200.parallel.fused import FusedComm

        return FusedComm(dev, max_tokens=1024, hidden=8192, fused_max_tokens=1024)
    return TorchComm()


def case_gemm_ar(dev, comm_kind):
    from oxidize_b200.models.weights import LinearWeight, QTensor
    from oxidize_b200.ops import cuda as C

    comm = make_comm("fused", dev)
    W, rank = comm.size, comm.rank
    shapes = [(64, 8192, 1024), (64, 8192, 3584), (1, 1024, 512), (200, 2048, 256), (16, 4096, 1792)]
    # both exchanges at every rank count: one-shot (push to all) and two-shot (owner reduces, broadcasts)
    cases = [(m, s) for m in (99, 2) for s in shapes]
    cases += [(2, (600, 2048, 256)), (2, (1024, 8192, 512))]  # prefill-sized: several waves of 256-token tiles
    for min_world, (T, N, K) in cases:
        C.lib().oxb_set_ar_ll_min_world(min_world)
        for rep in range(3):
            g = torch.Generator(device=dev)
            g.manual_seed(1000 * rank + 17 * rep + T)
            x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
            w = (torch.randn(N, K, device=dev, generator=g) * 0.03).to(torch.bfloat16)
            res = torch.randn(T, N, device=dev, generator=g).to(torch.bfloat16) if rep == 2 else None
            y = comm.linear_allreduce(x, LinearWeight([QTensor("BF16", w, (N, K))]), res)
            part = x.float() @ w.float().t()
            dist.all_reduce(part)
            if res is not None:
                part = part + res.float()
            torch.cuda.synchronize()
            assert rel_err(y, part) < 1e-2, (T, N, K, rep, rel_err(y, part))
            allb = [torch.empty_like(y) for _ in range(W)]
            dist.all_gather(allb, y.contiguous())
            if res is None:
                assert all(torch.equal(allb[0], t) for t in allb), "ranks disagree bitwise"
    assert comm.fused_calls > 0
    # stand-alone all-reduce, both exchanges
    for min_world in (99, 2):
        C.lib().oxb_set_ar_ll_min_world(min_world)
        for T, N in [(64, 8192), (3, 1024), (256, 4096)]:
            x = torch.randn(T, N, device=dev).to(torch.bfloat16)
            want = x.float().clone()
            dist.all_reduce(want)
            got = comm.all_reduce(x.clone())
            assert rel_err(got, want) < 1e-2
    C.lib().oxb_set_ar_ll_min_world(2)
    code, detail, count = C.status()
    assert code == 0, (code, detail, count)


def _tiny_file(rank):
    path = os.path.join(tempfile.gettempdir(), f"oxb_tp_tiny_{os.environ.get('MASTER_PORT', '0')}.gguf")
    if rank == 0:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        cfg = preset("tiny-llama", n_layers=2, vocab_size=512, n_heads=8, n_kv_heads=max(2, min(world, 8)))
        synth_gguf(path, cfg, "BF16", seed=0, norm_jitter=0.1)
    dist.barrier()
    return path


def case_tp_model(dev, comm_kind):
    layout = init_distributed()
    path = _tiny_file(layout.rank)
    g = load_gguf(path)
    cfg = config_from_gguf(g)
    act = torch.bfloat16 if dev.type == "cuda" else torch.float32
    ec = dict(max_model_len=128, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=32, max_num_batched_tokens=64,
              cuda_graphs=False)
    comm = make_comm(comm_kind, dev) if dev.type == "cuda" else TorchComm()
    w_tp = load_weights(g, cfg, dev, act, layout.rank, layout.world_size)
    w_1 = load_weights(g, cfg, dev, act, 0, 1)
    tp = LLM(w_tp, EngineConfig(tp_size=layout.world_size, **ec), comm)
    one = LLM(w_1, EngineConfig(**ec))
    tp.runner.keep_logits = one.runner.keep_logits = True
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    for p in ([5, 9, 200, 31, 7], list(range(3, 40))):
        tp.add_request(p, sp)
        one.add_request(p, sp)
    while tp.has_unfinished:
        tp.step()
        one.step()
        a, b = tp.last_step[1].logits, one.last_step[1].logits
        tol = 3e-2 if dev.type == "cuda" else 1e-4
        assert a.shape == b.shape and rel_err(a, b) < tol, rel_err(a, b)
    # greedy generation: identical tokens on every rank (distributed argmax over vocabulary shards)
    tp.runner.keep_logits = False
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = tp.generate([[4, 8, 15, 16, 23, 42]], sp)
    toks = torch.tensor(outs[0].token_ids, dtype=torch.int64, device=dev)
    gathered = [torch.empty_like(toks) for _ in range(layout.world_size)]
    dist.all_gather(gathered, toks)
    assert all(torch.equal(gathered[0], t) for t in gathered)
    if dev.type == "cuda":
        from oxidize_b200.ops import cuda as C

        assert C.status()[0] == 0
        if comm_kind == "fused":
            assert comm.fused_calls > 0


def case_tp_families(dev, comm_kind):
    """Tensor-parallel shards of a Gemma-3 model (branch-output norms, two rotary bases) and of a latent-attention
    DeepSeek model (heads of the per-head up-projection split over the ranks, latent cache replicated) give the
    single-rank logits."""
    layout = init_distributed()
    small = dict(n_layers=3, vocab_size=512, hidden_size=64, context_length=4096)
    cfgs = {
        "gemma3": preset("gemma3-27b", **small, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=128, sliding_window=16,
                         embedding_scale=8.0, attn_scale=0.2, sliding_window_pattern=2),
        "mla": preset("deepseek-v3", **small, n_heads=4, n_kv_heads=4, head_dim=24, rope_dim=8, qk_nope_dim=16, v_head_dim=24,
                      kv_lora_rank=32, q_lora_rank=48, ffn_size=96, n_experts=8, n_experts_used=2, expert_ffn_size=48,
                      expert_group_count=4, expert_group_used_count=2, leading_dense_blocks=1, shared_expert_ffn_size=48),
    }
    ec = dict(max_model_len=128, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=32, max_num_batched_tokens=64,
              cuda_graphs=False, kv_cache_dtype="f32")
    for name, cfg0 in cfgs.items():
        path = os.path.join(tempfile.gettempdir(), f"oxb_tp_{name}_{os.environ.get('MASTER_PORT', '0')}.gguf")
        if layout.rank == 0:
            synth_gguf(path, cfg0, "F32", seed=3, norm_jitter=0.2)
        dist.barrier()
        g = load_gguf(path)
        cfg = config_from_gguf(g)
        w_tp = load_weights(g, cfg, dev, torch.float32, layout.rank, layout.world_size, ep_rank=0, ep_size=1)
        w_1 = load_weights(g, cfg, dev, torch.float32, 0, 1)
        tp = LLM(w_tp, EngineConfig(tp_size=layout.world_size, **ec), TorchComm())
        one = LLM(w_1, EngineConfig(**ec))
        tp.runner.keep_logits = one.runner.keep_logits = True
        sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
        for p in ([5, 9, 200, 31, 7], list(range(3, 50))):
            tp.add_request(p, sp)
            one.add_request(p, sp)
        while tp.has_unfinished:
            tp.step()
            one.step()
            a, b = tp.last_step[1].logits, one.last_step[1].logits
            assert a.shape == b.shape and rel_err(a, b) < 1e-4, (name, rel_err(a, b))
        dist.barrier()


def case_ep1_model(dev, comm_kind):
    """Tensor parallelism with every expert replicated on every rank (ep_size = 1) == single rank."""
    return case_ep_model(dev, comm_kind, replicate_experts=True)


def case_ep_model(dev, comm_kind, replicate_experts=False):
    """Expert parallelism (experts split over the ranks, attention tensor-parallel) == single rank."""
    layout = init_distributed()
    path = os.path.join(tempfile.gettempdir(), f"oxb_ep_tiny_{os.environ.get('MASTER_PORT', '0')}.gguf")
    if layout.rank == 0:
        big = dev.type == "cuda"  # the GPU attention kernels take head_dim 64 / 128
        cfg = preset("mixtral-8x7b", hidden_size=256 if big else 128, n_layers=2, n_heads=4, n_kv_heads=2,
                     head_dim=64 if big else 32, ffn_size=512 if big else 256, expert_ffn_size=128 if big else 64,
                     vocab_size=256, n_experts=4, n_experts_used=2, n_shared_experts=1 if replicate_experts else 0,
                     shared_expert_ffn_size=(128 if big else 64) if replicate_experts else 0)
        synth_gguf(path, cfg, "BF16", seed=2, norm_jitter=0.1)
    dist.barrier()
    g = load_gguf(path)
    cfg = config_from_gguf(g)
    act = torch.bfloat16 if dev.type == "cuda" else torch.float32
    ec = dict(max_model_len=128, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=32, max_num_batched_tokens=64,
              cuda_graphs=False)
    comm = make_comm(comm_kind, dev) if dev.type == "cuda" else TorchComm()
    W = layout.world_size
    if replicate_experts:
        w_ep = load_weights(g, cfg, dev, act, layout.rank, W, 0, 1)
        assert len(w_ep.layers[0].experts.gate_up) == cfg.n_experts and w_ep.layers[0].shared_gate_up is not None
    else:
        w_ep = load_weights(g, cfg, dev, act, layout.rank, W, layout.rank, W)
        assert len(w_ep.layers[0].experts.gate_up) == cfg.n_experts // W
    w_1 = load_weights(g, cfg, dev, act, 0, 1)
    ep = LLM(w_ep, EngineConfig(tp_size=W, ep_size=1 if replicate_experts else W, **ec), comm)
    one = LLM(w_1, EngineConfig(**ec))
    ep.runner.keep_logits = one.runner.keep_logits = True
    # one sampled token: the logits of the prompt are compared; with more, a near-tie in bf16 may pick
    # different tokens in the two runs and the later logits are no longer comparable
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    for p in ([5, 9, 200, 31, 7], list(range(3, 40))):
        ep.add_request(p, sp)
        one.add_request(p, sp)
    while ep.has_unfinished:
        ep.step()
        one.step()
        a, b = ep.last_step[1].logits, one.last_step[1].logits
        tol = 3e-2 if dev.type == "cuda" else 1e-4
        assert a.shape == b.shape and rel_err(a, b) < tol, rel_err(a, b)


def case_pp_model(dev, comm_kind):
    """Two pipeline stages (each holds half of the layers) produce the single-process tokens."""
    from oxidize_b200.engine.kv_pool import KVCache, KVCacheSpec
    from oxidize_b200.models.transformer import BatchMeta, Transformer
    from oxidize_b200.parallel.pp import PipelineStage, StageIO, split_layers

    layout = init_distributed()
    path = _tiny_file(layout.rank)
    g = load_gguf(path)
    cfg = config_from_gguf(g)
    act = torch.bfloat16 if dev.type == "cuda" else torch.float32
    W, rank = layout.world_size, layout.rank
    lo, hi = split_layers(cfg.n_layers, W)[rank]
    w_stage = load_weights(g, cfg, dev, act, 0, 1, layer_range=(lo, hi))
    assert len(w_stage.layers) == hi - lo
    stage = PipelineStage(Transformer(w_stage), StageIO(rank, W))
    kv = KVCache(KVCacheSpec(hi - lo, cfg.n_kv_heads, cfg.head_dim, 16, "f32" if dev.type == "cpu" else "bf16"), 8, dev)
    prompt = [4, 8, 15, 16, 23, 42, 7]
    n_new = 5

    def meta_for(tokens, start):
        n = len(tokens)
        i32 = dict(dtype=torch.int32, device=dev)
        pos = torch.arange(start, start + n, **i32)
        return BatchMeta(token_ids=torch.tensor(tokens, **i32), positions=pos, slot_mapping=pos.clone(),
                         query_start=torch.tensor([0, n], **i32), seq_lens=torch.tensor([start + n], **i32),
                         block_tables=torch.arange(8, **i32)[None, :], logits_indices=torch.tensor([n - 1], **i32),
                         max_query_len=n, max_seq_len=start + n, num_seqs=1)

    toks = list(prompt)
    feed, start = list(prompt), 0
    out = []
    for _ in range(n_new):
        t = stage.forward_microbatch(meta_for(feed, start), kv)
        if stage.io.is_last:
            nxt = int(t[0])
        else:
            nxt = int(stage.io.recv_tokens_from_last(1, dev)[0]) if stage.io.is_first else 0
        stage.drain()
        b = torch.tensor([nxt], dtype=torch.int64, device=dev)
        dist.broadcast(b, src=W - 1)
        nxt = int(b[0])
        out.append(nxt)
        start += len(feed)
        feed = [nxt]
    # single-process reference
    ref = LLM(load_weights(g, cfg, dev, act, 0, 1), EngineConfig(max_model_len=64, max_num_seqs=2, num_kv_blocks=16,
                                                                  cuda_graphs=False))
    want = ref.generate([prompt], SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))[0].token_ids
    assert out == want, (out, want)


def case_pp_engine(dev, comm_kind):
    """The engine with pp_size = world (or tp 2 x pp 2 on four ranks): stage-local layers, micro-batched steps,
    activations over isend / recv, tokens broadcast from the last stage; same tokens as one process."""
    from oxidize_b200.parallel.pp import make_pipeline_groups

    layout = init_distributed()
    W, rank = layout.world_size, layout.rank
    tp = 2 if W == 4 else 1
    pp = W // tp
    path = _tiny_file(rank)
    io, tp_group = make_pipeline_groups(W, rank, tp, pp)
    assert io is not None and io.world == pp
    comm = None
    if tp > 1:
        if dev.type == "cuda" and comm_kind == "fused":
            from oxidize_b200.parallel.fused import FusedComm

            comm = FusedComm(dev, max_tokens=1024, hidden=8192, group=tp_group)
        else:
            comm = TorchComm(tp_group)
    ec = dict(max_model_len=128, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=16, max_num_batched_tokens=48)
    llm = LLM.from_gguf(path, EngineConfig(tp_size=tp, pp_size=pp, **ec), device=dev, comm=comm, tp_rank=rank % tp, pipe=io)
    n_layers = config_from_gguf(load_gguf(path)).n_layers
    assert len(llm.weights.layers) < n_layers, "a stage must hold only its own layers"
    prompts = [[4, 8, 15, 16, 23, 42, 7], list(range(3, 40)), [9, 9], [60, 61, 62, 63]]
    sp = SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)
    got = [o.token_ids for o in llm.generate(prompts, sp)]
    # a sampled request too: the last stage draws, every stage must learn the same tokens
    sps = SamplingParams(temperature=0.8, top_k=20, max_tokens=6, ignore_eos=True, seed=5)
    got_s = [o.token_ids for o in llm.generate(prompts[:2], sps)]
    if tp == 1:
        one = LLM.from_gguf(path, EngineConfig(**ec), device=dev)
    else:
        # Splitting the layers over stages does not change the arithmetic, splitting the heads over ranks does (bf16
        # partial sums): the exact reference for tp x pp is the same tensor-parallel group running all layers.
        one = LLM.from_gguf(path, EngineConfig(tp_size=tp, **ec), device=dev, comm=comm, tp_rank=rank % tp)
    want = [o.token_ids for o in one.generate(prompts, sp)]
    assert got == want, (got, want)
    box = [None] * W
    dist.all_gather_object(box, got_s)
    assert all(b == box[0] for b in box), "stages disagree on the sampled tokens"
    assert all(len(t) == 6 for t in got_s)


def case_tp_graph(dev, comm_kind):
    """Decode under CUDA graphs with the fused collectives gives the same tokens as eager."""
    layout = init_distributed()
    path = _tiny_file(layout.rank)
    g = load_gguf(path)
    cfg = config_from_gguf(g)
    comm = make_comm(comm_kind, dev)
    w_tp = load_weights(g, cfg, dev, torch.bfloat16, layout.rank, layout.world_size)
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    prompts = [[4, 8, 15, 16, 23, 42], list(range(50, 75)), [7, 7, 7]]
    res = []
    for graphs in (False, True):
        llm = LLM(w_tp, EngineConfig(tp_size=layout.world_size, max_model_len=128, max_num_seqs=4, num_kv_blocks=64,
                                     prefill_chunk_size=32, max_num_batched_tokens=64, cuda_graphs=graphs), comm)
        res.append([o.token_ids for o in llm.generate(prompts, sp)])
    assert res[0] == res[1], (res[0], res[1])
    from oxidize_b200.ops import cuda as C

    assert C.status()[0] == 0


def case_rank_exit(dev, comm_kind):
    """A rank that leaves between steps is noticed on the host (store heartbeat) before the
    survivors launch their next collective."""
    from oxidize_b200.parallel.health import Heartbeat

    layout = init_distributed()
    hb = Heartbeat.from_env(layout.rank, layout.world_size, interval_s=0.05, stale_after_s=0.5)
    hb.start()
    x = torch.ones(4, device=dev)
    dist.all_reduce(x)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    if layout.rank == layout.world_size - 1:
        hb.stop(announce_exit=True)
        return
    import time

    deadline = time.time() + 10
    while time.time() < deadline and not hb.dead_ranks():
        time.sleep(0.05)
    assert hb.dead_ranks() == [layout.world_size - 1], hb.dead_ranks()
    hb.stop()


CASES = {"gemm_ar": case_gemm_ar, "tp_model": case_tp_model, "tp_families": case_tp_families, "tp_graph": case_tp_graph, "rank_exit": case_rank_exit, "ep_model": case_ep_model, "ep1_model": case_ep1_model, "pp_model": case_pp_model, "pp_engine": case_pp_engine}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--comm", default="fused")
    a = ap.parse_args()
    layout = init_distributed("gloo" if a.device == "cpu" else None, timeout_s=120)
    if a.device == "cuda":
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
    else:
        dev = torch.device("cpu")
    CASES[a.case](dev, a.comm)
    print(f"RANK {layout.rank} OK {a.case}", flush=True)
    if a.case != "rank_exit":
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
