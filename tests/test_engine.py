"""Block pool, scheduler, sampler and engine-level equivalence properties (CPU only).

The equivalence properties mirror the reference's model tests (model/inference.rs:2759-3268):
batched == standalone, chunked prefill == one-shot prefill, mid-flight admission == standalone,
rewind-then-reforward is lossless."""
import numpy as np
import pytest
import torch

from oxidize_b200.engine.kv_pool import BlockPool, KVCache, KVCacheSpec, OutOfBlocks, block_hash
from oxidize_b200.engine.llm import LLM, EngineConfig
from oxidize_b200.engine.sampler import (SamplingError, SamplingParams, sample, speculative_accept)
from oxidize_b200.engine.scheduler import Scheduler, SchedulerConfig, Sequence
from oxidize_b200.models.config import preset
from oxidize_b200.utils.synth import synth_gguf, synth_weights


# --------------------------------------------------------------------------- block pool
def test_block_hash_is_fnv_style():
    h = 0xCBF29CE484222325
    for t in (1, 2, 3):
        h = (h * 0x100000001B3) % (1 << 64)
        h ^= t
    assert block_hash([1, 2, 3]) == h
    assert block_hash([3], block_hash([1, 2])) == h


def test_pool_alloc_free_refcount():
    p = BlockPool(4, 16)
    a, b = p.allocate(), p.allocate()
    assert (a, b) == (0, 1) and p.num_free == 2
    p.incref(a)
    assert p.is_shared(a)
    p.release(a)
    assert not p.is_shared(a) and p.num_free == 2
    p.release(a)
    assert p.num_free == 3
    with pytest.raises(RuntimeError):
        p.release(a)
    p.allocate(), p.allocate(), p.allocate()
    with pytest.raises(OutOfBlocks):
        p.allocate()


def test_prefix_cache_hit_and_lru_eviction():
    p = BlockPool(3, 4)
    toks = list(range(10))
    b0, b1 = p.allocate(), p.allocate()
    h0 = block_hash(toks[:4])
    h1 = block_hash(toks[4:8], h0)
    p.publish(b0, h0)
    p.publish(b1, h1)
    p.release(b0)
    p.release(b1)
    assert p.num_free == 3  # cached blocks stay evictable
    blocks, covered = p.match_prefix(toks)
    assert blocks == [b0, b1] and covered == 8 and p.hits == 2
    p.release_all(blocks)
    # exhaust: the free block first, then the least recently used cached block
    got = [p.allocate() for _ in range(3)]
    assert sorted(got) == [0, 1, 2]
    assert p.match_prefix(toks) == ([], 0)


# --------------------------------------------------------------------------- scheduler
def _sched(nblocks=64, **kw):
    pool = BlockPool(nblocks, 16)
    return Scheduler(SchedulerConfig(**kw), pool), pool


def _run(s: Scheduler, steps=1000, tok=7):
    order = []
    for _ in range(steps):
        out = s.schedule()
        if out.is_empty:
            break
        order.append([(ss.seq.seq_id, ss.num_tokens, ss.is_prefill) for ss in out.scheduled])
        s.postprocess(out, {ss.seq.seq_id: [tok] for ss in out.scheduled if ss.sample})
    return order


def test_decode_first_then_prefill_then_admit():
    s, _ = _sched(max_num_batched_tokens=20, prefill_chunk_size=16, max_num_running_seqs=8, enable_prefix_cache=False)
    a = Sequence(list(range(40)), SamplingParams(max_tokens=3))
    s.add(a)
    o1 = s.schedule()
    assert [(x.num_tokens, x.is_prefill, x.sample) for x in o1.scheduled] == [(16, True, False)]
    s.postprocess(o1, {})
    b = Sequence(list(range(5)), SamplingParams(max_tokens=3))
    s.add(b)
    o2 = s.schedule()
    # a continues its prefill (16), b is admitted with the 4 tokens of budget left
    assert [(x.seq is a, x.num_tokens) for x in o2.scheduled] == [(True, 16), (False, 4)]
    s.postprocess(o2, {})
    o3 = s.schedule()
    assert [(x.seq is a, x.num_tokens, x.sample) for x in o3.scheduled] == [(True, 8, True), (False, 1, True)]
    s.postprocess(o3, {a.seq_id: [1], b.seq_id: [1]})
    o4 = s.schedule()
    assert all(not x.is_prefill and x.num_tokens == 1 for x in o4.scheduled) and o4.num_decode_tokens == 2


def test_max_running_and_finish_reasons():
    s, pool = _sched(max_num_batched_tokens=512, prefill_chunk_size=64, max_num_running_seqs=2, enable_prefix_cache=False)
    seqs = [Sequence([1, 2, 3], SamplingParams(max_tokens=2, stop_token_ids=(9,))) for _ in range(3)]
    for q in seqs:
        s.add(q)
    o = s.schedule()
    assert len(o.scheduled) == 2 and len(s.waiting) == 1
    s.postprocess(o, {seqs[0].seq_id: [9], seqs[1].seq_id: [4]})
    assert seqs[0].finish_reason == "stop" and seqs[0].output == [9]  # the stop token is yielded
    _run(s)
    assert [q.finish_reason for q in seqs] == ["stop", "length", "length"]
    assert pool.num_free == pool.num_blocks


def test_eos_and_stop_sequences():
    s, _ = _sched(enable_prefix_cache=False)
    a = Sequence([1], SamplingParams(max_tokens=10, stop_sequences=((5, 6),)))
    b = Sequence([1], SamplingParams(max_tokens=10))
    c = Sequence([1], SamplingParams(max_tokens=10, ignore_eos=True))
    for q in (a, b, c):
        s.add(q)
    feed = {a.seq_id: [5, 6, 7], b.seq_id: [2, 2, 2], c.seq_id: [2, 2, 2]}
    for i in range(3):
        o = s.schedule()
        s.postprocess(o, {ss.seq.seq_id: [feed[ss.seq.seq_id][i]] for ss in o.scheduled}, eos_token_id=2)
    assert a.finish_reason == "stop" and a.output == [5, 6]
    assert b.finish_reason == "stop" and b.output == [2]
    assert not c.is_finished and c.output == [2, 2, 2]


def test_prefix_cache_shares_blocks_and_cow():
    s, pool = _sched(nblocks=32, max_num_batched_tokens=512, prefill_chunk_size=512)
    prompt = list(range(100, 140))  # 40 tokens: 2 full blocks + 8
    a = Sequence(prompt, SamplingParams(max_tokens=2))
    s.add(a)
    _run(s)
    used_after_a = pool.num_used
    assert used_after_a == 0 and len(pool.cache) == 2
    b = Sequence(prompt, SamplingParams(max_tokens=2))
    s.add(b)
    o = s.schedule()
    assert b.num_cached_tokens == 32 and o.scheduled[0].start == 32 and o.scheduled[0].num_tokens == 8
    # identical 32-token prompt: the last cached block may not be fully reused (last token recomputed)
    c = Sequence(prompt[:32], SamplingParams(max_tokens=2))
    s.add(c)
    o2 = s.schedule()
    sc = [x for x in o2.scheduled if x.seq is c][0]
    assert c.num_cached_tokens == 16 and sc.start == 16


def test_preemption_requeues_front_and_completes():
    s, pool = _sched(nblocks=6, max_num_batched_tokens=512, prefill_chunk_size=512, max_num_running_seqs=4,
                     enable_prefix_cache=False)
    a = Sequence(list(range(30)), SamplingParams(max_tokens=40, ignore_eos=True))
    b = Sequence(list(range(30)), SamplingParams(max_tokens=40, ignore_eos=True))
    s.add(a)
    s.add(b)
    _run(s, steps=400)
    assert a.is_finished and b.is_finished and s.num_preemptions >= 1
    assert len(a.output) + len(getattr(a, "_preempted_outputs", [])) == 40
    assert len(b.output) + len(getattr(b, "_preempted_outputs", [])) == 40
    assert pool.num_free == pool.num_blocks


def test_too_long_prompt_rejected():
    s, _ = _sched(nblocks=2)
    with pytest.raises(OutOfBlocks):
        s.add(Sequence(list(range(100)), SamplingParams()))


def test_sjf_policy_orders_by_job_size():
    s, _ = _sched(max_num_running_seqs=1, policy="sjf", enable_prefix_cache=False, max_num_batched_tokens=512,
                  prefill_chunk_size=512)
    big = Sequence(list(range(50)), SamplingParams(max_tokens=5))
    small = Sequence(list(range(5)), SamplingParams(max_tokens=5))
    s.add(big)
    s.add(small)
    assert s.schedule().scheduled[0].seq is small


# --------------------------------------------------------------------------- sampler
def test_sampling_validation_and_greedy():
    logits = np.array([0.1, 3.0, 3.0, -1.0], dtype=np.float32)
    with pytest.raises(SamplingError):
        sample(logits, SamplingParams(top_k=0), 0.5)
    with pytest.raises(SamplingError):
        sample(logits, SamplingParams(top_p=1.5), 0.5)
    with pytest.raises(SamplingError):
        sample(logits, SamplingParams(), 1.0)
    assert sample(logits, SamplingParams(temperature=0.0), 0.3) == 1
    assert sample(logits, SamplingParams(temperature=0.0, tie="highest"), 0.3) == 2
    assert sample(logits, SamplingParams(temperature=1.0, top_k=1), 0.99) == 1
    assert sample(logits, SamplingParams(temperature=0.0), 0.3, suppressed=[1, 2]) == 0


def test_sampling_filters_and_distribution():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float64)).astype(np.float32)
    p = SamplingParams(temperature=1.0, top_p=0.8)
    draws = {sample(logits, p, r) for r in np.linspace(0, 0.999, 200)}
    assert draws == {0, 1}  # 0.5 + 0.3 reaches 0.8
    p = SamplingParams(temperature=1.0, min_p=0.5)
    assert {sample(logits, p, r) for r in np.linspace(0, 0.999, 50)} == {0, 1}
    p = SamplingParams(temperature=1.0, top_k=3)
    assert {sample(logits, p, r) for r in np.linspace(0, 0.999, 200)} == {0, 1, 2}
    # unfiltered: inverse CDF in index order
    p = SamplingParams(temperature=1.0)
    assert sample(logits, p, 0.49) == 0 and sample(logits, p, 0.51) == 1 and sample(logits, p, 0.96) == 3
    # penalties are additive
    p = SamplingParams(temperature=0.0, frequency_penalty=2.0)
    assert sample(np.array([1.0, 0.5], dtype=np.float32), p, 0.1, recent=[0]) == 1


def test_speculative_accept_rules():
    V = 6
    tl = np.full((4, V), -5.0, dtype=np.float32)
    tl[0, 2] = tl[1, 3] = tl[2, 1] = tl[3, 4] = 5.0
    toks, n = speculative_accept([2, 3, 1], None, tl, SamplingParams(temperature=0.0), [])
    assert (toks, n) == ([2, 3, 1, 4], 3)  # all accepted + bonus
    toks, n = speculative_accept([2, 0, 1], None, tl, SamplingParams(temperature=0.0), [])
    assert (toks, n) == ([2, 3], 1)  # first mismatch replaced by the target's token
    # stochastic: q puts all mass on a token the target dislikes -> reject and resample from max(p-q,0)
    q = [np.eye(V)[0]]
    tl2 = np.zeros((2, V), dtype=np.float32)
    tl2[0, 0] = -50.0
    toks, n = speculative_accept([0], q, tl2, SamplingParams(temperature=1.0), [0.5, 0.1, 0.2])
    assert n == 0 and toks[0] != 0


def test_device_sampler_matches_host_oracle():
    from oxidize_b200.engine.device_sampler import sample_torch

    rng = np.random.default_rng(0)
    R, V = 16, 200
    logits = torch.from_numpy(rng.standard_normal((R, V)).astype(np.float32) * 3)
    temps = np.array([0.0, 1.0, 0.7, 1.3] * 4, dtype=np.float32)
    topk = np.array([0, 0, 5, 50] * 4, dtype=np.int32)
    topp = np.array([1.0, 0.9, 1.0, 0.5] * 4, dtype=np.float32)
    minp = np.array([0.0, 0.0, 0.1, 0.0] * 4, dtype=np.float32)
    rnd = rng.random(R).astype(np.float32) * 0.999
    got = sample_torch(logits, torch.from_numpy(temps), torch.from_numpy(topk), torch.from_numpy(topp),
                       torch.from_numpy(minp), torch.from_numpy(rnd)).tolist()
    for r in range(R):
        p = SamplingParams(temperature=float(temps[r]), top_k=int(topk[r]) or None,
                           top_p=float(topp[r]) if topp[r] < 1 else (1.0 if topk[r] or minp[r] else None),
                           min_p=float(minp[r]) or None)
        if temps[r] > 0 and not p.has_filters:
            continue  # the unfiltered oracle path draws in index order, the batched path in sorted order
        assert got[r] == sample(logits[r].numpy(), p, float(rnd[r])), r


# --------------------------------------------------------------------------- engine equivalences
@pytest.fixture(scope="module")
def tiny_path(tmp_path_factory):
    cfg = preset("tiny-llama", n_layers=2, vocab_size=300)
    p = str(tmp_path_factory.mktemp("m") / "tiny.gguf")
    synth_gguf(p, cfg, "Q4_K_M", seed=0, norm_jitter=0.05)
    return p


def _gen(path, prompts, sp, **ec):
    base = dict(max_model_len=256, max_num_seqs=4, num_kv_blocks=96, prefill_chunk_size=16, max_num_batched_tokens=64)
    base.update(ec)
    llm = LLM.from_gguf(path, EngineConfig(**base), device="cpu")
    return [o.token_ids for o in llm.generate(prompts, sp)], llm


def test_batched_equals_standalone_and_chunking_is_invisible(tiny_path):
    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 300, size=n).tolist() for n in (5, 33, 17, 64)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    batched, _ = _gen(tiny_path, prompts, sp)
    for p, want in zip(prompts, batched):
        solo, _ = _gen(tiny_path, [p], sp, max_num_seqs=1, prefill_chunk_size=256, max_num_batched_tokens=256,
                       enable_prefix_cache=False)
        assert solo[0] == want


def test_midflight_admission_equals_standalone(tiny_path):
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    a, b = list(range(10, 40)), list(range(50, 70))
    solo_a, _ = _gen(tiny_path, [a], sp)
    solo_b, _ = _gen(tiny_path, [b], sp)
    llm = LLM.from_gguf(tiny_path, EngineConfig(max_model_len=256, max_num_seqs=4, num_kv_blocks=96,
                                                prefill_chunk_size=16, max_num_batched_tokens=64), device="cpu")
    ra = llm.add_request(a, sp)
    done = {}
    for i in range(200):
        if i == 5:
            rb = llm.add_request(b, sp)
        for ro in llm.step():
            if ro.finished:
                done[ro.request_id] = ro.token_ids
        if i > 5 and not llm.has_unfinished:
            break
    assert done[ra] == solo_a[0] and done[rb] == solo_b[0]


def test_prefix_cache_reuse_gives_same_tokens(tiny_path):
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    p = list(range(20, 70))
    llm = LLM.from_gguf(tiny_path, EngineConfig(max_model_len=256, max_num_seqs=2, num_kv_blocks=64,
                                                prefill_chunk_size=64, max_num_batched_tokens=128), device="cpu")
    first = llm.generate([p], sp)[0]
    second = llm.generate([p], sp)[0]
    assert second.num_cached_tokens == 48 and second.token_ids == first.token_ids


def test_preemption_recompute_is_lossless(tiny_path):
    sp = SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)
    prompts = [list(range(3, 33)), list(range(40, 70))]
    want, _ = _gen(tiny_path, prompts, sp)
    got, llm = _gen(tiny_path, prompts, sp, num_kv_blocks=6, enable_prefix_cache=False)
    assert llm.scheduler.num_preemptions >= 1
    assert got == want


@pytest.mark.parametrize("kvd", ["f16", "q8", "q4"])
def test_quantized_kv_cache_close_to_f32(tiny_path, kvd):
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    p = list(range(5, 45))
    outs = {}
    for d in ("f32", kvd):
        llm = LLM.from_gguf(tiny_path, EngineConfig(max_model_len=128, max_num_seqs=1, num_kv_blocks=16,
                                                    prefill_chunk_size=16, max_num_batched_tokens=64,
                                                    kv_cache_dtype=d), device="cpu")
        llm.runner.keep_logits = True
        llm.add_request(p, sp)
        while llm.has_unfinished:
            llm.step()
        outs[d] = llm.last_step[1].logits
    err = float((outs[kvd] - outs["f32"]).norm() / outs["f32"].norm())
    assert err < {"f16": 1e-3, "q8": 2e-2, "q4": 0.25}[kvd]


def test_moe_families_run_and_batch_consistently():
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    for name, kw in (("mixtral-8x7b", dict(n_experts=4, n_experts_used=2)),
                     ("qwen3-30b-a3b", dict(n_experts=8, n_experts_used=2)),
                     ("mixtral-8x7b", dict(arch="deepseek2", n_experts=8, n_experts_used=2, expert_gating="sigmoid",
                                           expert_group_count=4, expert_group_used_count=2, n_shared_experts=1,
                                           shared_expert_ffn_size=64, expert_weights_scale=2.5,
                                           leading_dense_blocks=1))):
        cfg = preset(name, hidden_size=64, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=128,
                     expert_ffn_size=64, vocab_size=128, **kw)
        w = synth_weights(cfg, "cpu", "F32", seed=1)
        ec = EngineConfig(max_model_len=64, max_num_seqs=3, num_kv_blocks=32, prefill_chunk_size=8,
                          max_num_batched_tokens=32)
        prompts = [[3, 4, 5, 6, 7, 8, 9, 10, 11], [20, 21, 22]]
        both = [o.token_ids for o in LLM(w, ec).generate(prompts, sp)]
        for p, want in zip(prompts, both):
            assert LLM(w, ec).generate([p], sp)[0].token_ids == want


def test_kv_cache_state_roundtrip():
    spec = KVCacheSpec(2, 2, 32, 16, "q8")
    kv = KVCache(spec, 8)
    for d in kv.data:
        d.random_(0, 255)
    for s in kv.scales:
        s.uniform_(0, 1)
    st = kv.state_dict([1, 5])
    kv2 = KVCache(spec, 8)
    kv2.load_state_dict(st, [2, 3])
    assert torch.equal(kv2.data[1][2], kv.data[1][1]) and torch.equal(kv2.scales[0][3], kv.scales[0][5])


# --------------------------------------------------------------------------- C++ host runtime
def test_native_block_pool_matches_python_pool_on_random_traces():
    """The C++ pool must hand out the same block ids as the Python specification for the same calls."""
    import random

    from oxidize_b200.engine import native
    from oxidize_b200.engine.kv_pool import FNV_OFFSET, BlockPool, OutOfBlocks, block_hash

    if native.lib() is None:
        pytest.skip("liboxbrt could not be built")
    assert native.block_hash([1, 2, 3, 70000], FNV_OFFSET) == block_hash([1, 2, 3, 70000], FNV_OFFSET)
    for seed in range(6):
        rng = random.Random(seed)
        py, cc = BlockPool(24, 4), native.NativeBlockPool(24, 4)
        held = []  # blocks we hold a reference on (same list for both pools)
        for step in range(600):
            op = rng.random()
            if op < 0.35:
                try:
                    a = py.allocate()
                except OutOfBlocks:
                    with pytest.raises(OutOfBlocks):
                        cc.allocate()
                    continue
                assert cc.allocate() == a
                held.append(a)
            elif op < 0.6 and held:
                b = held.pop(rng.randrange(len(held)))
                py.release(b)
                cc.release(b)
            elif op < 0.75 and held:
                b, h = rng.choice(held), rng.randrange(1, 40)
                py.publish(b, h)
                cc.publish(b, h)
            elif op < 0.9:
                h = rng.randrange(1, 40)
                a, c = py.lookup(h), cc.lookup(h)
                assert a == c
                if a is not None:
                    held.append(a)
            else:
                toks = [rng.randrange(3) for _ in range(rng.randrange(1, 14))]
                pa, na = py.match_prefix(toks)
                pc, nc = cc.match_prefix(toks)
                assert pa == pc and na == nc
                held += pa
            assert py.num_free == cc.num_free
            assert all(py.ref[b] == cc.ref[b] for b in range(24))
        assert (py.hits, py.misses) == (cc.hits, cc.misses)
    with pytest.raises(RuntimeError):
        cc2 = native.NativeBlockPool(2, 4)
        b = cc2.allocate()
        cc2.release(b)
        cc2.release(b)


def test_native_pool_prefix_sharing_through_the_engine(tmp_path):
    """Same generations with the C++ pool and with the Python pool (OXB_NATIVE_RUNTIME=0 semantics)."""
    from oxidize_b200.engine import native
    from oxidize_b200.engine.kv_pool import BlockPool
    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.engine.sampler import SamplingParams
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    if native.lib() is None:
        pytest.skip("liboxbrt could not be built")
    cfg = preset("tiny-llama", n_layers=1, vocab_size=300, n_heads=4, n_kv_heads=2)
    path = str(tmp_path / "t.gguf")
    synth_gguf(path, cfg, "F32", seed=5)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompts = [list(range(5, 45)), list(range(5, 45)) + [7, 8], [9] * 20]
    outs = []
    for use_native in (True, False):
        llm = LLM.from_gguf(path, EngineConfig(max_model_len=128, max_num_seqs=4, num_kv_blocks=40), device="cpu")
        if not use_native:
            llm.pool = llm.scheduler.pool = BlockPool(llm.pool.num_blocks, llm.pool.page_size, True)
        else:
            assert isinstance(llm.pool, native.NativeBlockPool)
        outs.append([o.token_ids for o in llm.generate(prompts, sp)])
        second = llm.generate(prompts[:1], sp)  # served from the prefix cache
        assert second[0].num_cached_tokens >= 32
    assert outs[0] == outs[1]


# --------------------------------------------------------------------------- host sampler paths, grammar, beam search
def _tiny_llm(tmp_path, **kw):
    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    cfg = preset("tiny-llama", n_layers=1, vocab_size=64, n_heads=4, n_kv_heads=2)
    path = str(tmp_path / "t.gguf")
    synth_gguf(path, cfg, "F32", seed=11)
    return LLM.from_gguf(path, EngineConfig(max_model_len=128, max_num_seqs=8, num_kv_blocks=64, **kw), device="cpu")


def test_mirostat_and_penalties_reach_the_host_sampler(tmp_path):
    import numpy as np

    from oxidize_b200.engine.sampler import SamplingParams, sample

    # unit: Mirostat keeps the observed surprise near tau and updates mu
    rng = np.random.default_rng(0)
    logits = rng.normal(0, 2, 200).astype(np.float32)
    p = SamplingParams(temperature=1.0, mirostat_tau=3.0, mirostat_eta=0.2)
    state = {}
    toks = [sample(logits, p, float(rng.random()), state=state) for _ in range(200)]
    assert "mirostat_mu" in state and 0.5 < state["mirostat_mu"] < 12.0
    assert len(set(toks)) > 3
    # engine: a presence penalty strong enough forbids immediate repeats under greedy-like sampling
    llm = _tiny_llm(tmp_path)
    base = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))[0].token_ids
    pen = llm.generate([[1, 2, 3]], SamplingParams(temperature=1e-6, top_k=1, presence_penalty=50.0, max_tokens=12,
                                                   ignore_eos=True))[0].token_ids
    assert len(pen) == 12 and len(set(pen)) == 12  # every token new: the penalty was applied
    assert len(base) == 12
    mir = llm.generate([[1, 2, 3]], SamplingParams(temperature=1.0, mirostat_tau=2.0, seed=3, max_tokens=8, ignore_eos=True))
    assert len(mir[0].token_ids) == 8


def test_token_grammar_constrains_generation(tmp_path):
    from oxidize_b200.engine.constrained import GrammarError, TokenGrammar
    from oxidize_b200.engine.sampler import SamplingParams

    # root := 10 list 11 ; list := item | item 12 list ; item := 20 | 21 | 22
    g = TokenGrammar({"root": [[10, "list", 11]], "list": [["item"], ["item", 12, "list"]], "item": [[20], [21], [22]]},
                     eos_token_ids=[2])
    assert g.accepts([10, 20, 11]) and g.accepts([10, 21, 12, 22, 11])
    assert not g.accepts([10, 11]) and not g.accepts([10, 20, 12, 11]) and not g.accepts([10, 20])
    st = {}
    assert g.allowed_tokens(st) == {10}
    g.advance(st, 10)
    assert g.allowed_tokens(st) == {20, 21, 22}
    with pytest.raises(GrammarError):
        g.advance(st, 11)
    with pytest.raises(GrammarError):
        TokenGrammar({"root": [["missing"]]})
    llm = _tiny_llm(tmp_path)
    for seed in range(4):
        sp = SamplingParams(temperature=1.0, seed=seed, max_tokens=30, grammar=g, stop_token_ids=(2,))
        out = llm.generate([[5, 6, 7]], sp)[0].token_ids
        body = out[:-1] if out and out[-1] == 2 else out
        state = {}
        for t in body:  # every prefix is a valid parse prefix
            g.advance(state, t)
        if out and out[-1] == 2:
            assert g.accepts(body)


def test_beam_search_finds_the_best_sequence(tmp_path):
    import numpy as np

    from oxidize_b200.engine.constrained import beam_search

    # toy scorer: token 1 then 2 then EOS(0) is the best path, but greedy's first step prefers token 3
    def scorer(seqs):
        out = []
        for s in seqs:
            g = s[1:]  # drop the prompt token
            if not g:
                row = [-9, np.log(0.4), -9, np.log(0.6)]
            elif g == [1]:
                row = [-9, -9, np.log(0.95), np.log(0.05)]
            elif g == [1, 2]:
                row = [np.log(0.99), -9, -9, np.log(0.01)]
            else:
                row = [np.log(0.3), np.log(0.3), np.log(0.2), np.log(0.2)]
            out.append(row)
        return np.asarray(out, dtype=np.float64)

    best = beam_search(scorer, [7], beam_width=3, max_new_tokens=4, eos_token_id=0, length_penalty=0.0)
    assert best[0][0] == [1, 2, 0]
    llm = _tiny_llm(tmp_path)
    beams = llm.beam_search([1, 2, 3, 4], beam_width=3, max_tokens=4)
    assert 1 <= len(beams) <= 3 and all(len(t) <= 4 for t, _ in beams)
    assert beams[0][1] >= beams[-1][1]
    # width 1 is greedy decoding
    from oxidize_b200.engine.sampler import SamplingParams

    greedy = llm.generate([[1, 2, 3, 4]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))[0].token_ids
    one = llm.beam_search([1, 2, 3, 4], beam_width=1, max_tokens=4)
    assert one[0][0][: len(greedy)] == greedy[: len(one[0][0])]


def test_decode_builder_writes_the_same_batch_as_the_general_builder(tmp_path):
    import numpy as np

    from oxidize_b200.engine.sampler import SamplingParams

    llm = _tiny_llm(tmp_path)
    rng = np.random.default_rng(3)
    for n, mt in ((5, 40), (21, 3), (33, 40), (16, 40), (9, 6)):
        llm.add_request(rng.integers(3, 64, size=n).tolist(), SamplingParams(temperature=0.0, max_tokens=mt, ignore_eos=True))
    names = ("token_ids", "positions", "slot_mapping", "query_start", "seq_lens", "logits_indices", "block_tables")
    r = llm.runner
    checked = 0
    sizes = set()
    for _ in range(30):
        out = llm.scheduler.schedule()
        sch = out.scheduled
        if sch and all((not s.is_prefill) and s.num_tokens == 1 for s in sch):
            for pad in (None, 8):
                a = r.build(sch, pad)
                want = {k: r.buf.h(k).copy() for k in names}
                b = r.build_decode(sch, pad)  # also exercises the row-ownership record right after build() voided it
                b2 = r.build_decode(sch, pad)  # ... and with the record in place
                assert a[:5] == b[:5] == b2[:5]
                assert [(x[0].seq.seq_id, x[1], x[2]) for x in a[5]] == [(x[0].seq.seq_id, x[1], x[2]) for x in b[5]]
                T, B, nl = a[0], a[1], a[2]
                M = r.max_blocks
                for k in names:
                    got = r.buf.h(k)
                    if k == "block_tables":
                        for i, s in enumerate(sch):
                            nb = len(s.seq.blocks)
                            assert np.array_equal(got[i * M : i * M + nb], want[k][i * M : i * M + nb])
                    else:
                        n = {"token_ids": T, "positions": T, "slot_mapping": T, "query_start": B + 1, "seq_lens": B,
                             "logits_indices": nl}[k]
                        assert np.array_equal(got[:n], want[k][:n]), k
                checked += 1
            sizes.add(len(sch))
        # let the step run for real so sequences grow, finish and shift rows
        res = r.execute(out)
        llm.scheduler.postprocess(out, res.tokens, None, 0.0)
    assert checked >= 10 and len(sizes) >= 2  # rows moved to other sequences at least once


def _tiny_async_llm(tmp_path, async_decode, **kw):
    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    cfg = preset("tiny-llama", n_layers=2, vocab_size=97, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96)
    path = str(tmp_path / "tiny_async.gguf")
    synth_gguf(path, cfg, "F32", seed=5, norm_jitter=0.2)
    ec = dict(max_model_len=96, max_num_seqs=8, num_kv_blocks=64, prefill_chunk_size=16, max_num_batched_tokens=64,
              kv_page_size=4, enable_prefix_cache=False)
    ec.update(kw)
    return LLM.from_gguf(path, EngineConfig(async_decode=async_decode, **ec), device="cpu")


def test_run_ahead_decode_matches_synchronous_decode(tmp_path):
    """One step in flight ahead of the host: same tokens, finish reasons and step count as the synchronous loop, with
    sequences that end by length, by a stop token in the middle of the run, and a request that arrives late."""
    from oxidize_b200.engine.sampler import SamplingParams

    prompts = [[5, 9, 20, 31, 7], list(range(3, 30)), [1, 2, 3], [40, 41, 42, 43, 44, 45, 46, 47, 48]]
    ref = _tiny_async_llm(tmp_path, False)
    base = ref.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    # a stop token that really occurs in the middle of one of the generations
    stop_tok = base[1].token_ids[9]
    lens = [24, 17, 24, 5]

    def run(async_decode):
        llm = _tiny_async_llm(tmp_path, async_decode)
        sps = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True, stop_token_ids=[stop_tok] if i == 1 else [])
               for i, n in enumerate(lens)]
        ids = [llm.add_request(p, sp) for p, sp in zip(prompts[:3], sps[:3])]
        final, steps, ahead = {}, 0, 0
        late = False
        while llm.has_unfinished or not late:
            if steps == 6 and not late:
                ids.append(llm.add_request(prompts[3], sps[3]))
                late = True
            for ro in llm.step():
                if ro.finished:
                    assert ro.request_id not in final, "a request finished twice"
                    final[ro.request_id] = ro
            ahead += getattr(llm, "_inflight", None) is not None
            steps += 1
            assert steps < 200
        assert llm.pool.num_free == llm.pool.num_blocks, "blocks leaked"
        return [final[i] for i in ids], ahead

    sync, a0 = run(False)
    asyn, a1 = run(True)
    assert a0 == 0 and a1 > 5, "the run-ahead path was not taken"
    for x, y in zip(sync, asyn):
        assert x.token_ids == y.token_ids and x.finish_reason == y.finish_reason
    assert sync[1].finish_reason == "stop" and len(sync[1].token_ids) <= 17


def test_run_ahead_decode_survives_abort_and_drain(tmp_path):
    from oxidize_b200.engine.sampler import SamplingParams

    llm = _tiny_async_llm(tmp_path, True)
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    a = llm.add_request([5, 6, 7, 8], sp)
    b = llm.add_request([9, 10, 11], sp)
    for _ in range(6):
        llm.step()
    assert getattr(llm, "_inflight", None) is not None
    assert llm.abort(a)
    outs = llm.step()  # the surplus row of the aborted request is dropped, the other request goes on
    assert [o.request_id for o in outs] == [b]
    n_before = len(llm._seqs[b].output)
    llm.drain()
    assert getattr(llm, "_inflight", None) is None and len(llm._seqs[b].output) >= n_before
    final = {}
    while llm.has_unfinished:
        for ro in llm.step():
            if ro.finished:
                final[ro.request_id] = ro
    assert len(final[b].token_ids) == 40
    assert llm.pool.num_free == llm.pool.num_blocks


def test_interleaved_local_global_attention_layers(tmp_path):
    """sliding_window_pattern = n: every n-th layer sees the whole context, the others the window."""
    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.engine.sampler import SamplingParams
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    base = dict(n_layers=2, vocab_size=97, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96)
    ec = dict(max_model_len=96, max_num_seqs=2, num_kv_blocks=32, prefill_chunk_size=64, max_num_batched_tokens=64,
              kv_page_size=4, enable_prefix_cache=False)
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    prompt = list(range(3, 43))

    def run(want, **kw):
        cfg = preset("tiny-llama", **base, **kw)
        assert [cfg.layer_sliding_window(i) for i in range(2)] == want
        p = str(tmp_path / f"w_{kw.get('sliding_window', 0)}_{kw.get('sliding_window_pattern', 0)}.gguf")
        synth_gguf(p, cfg, "F32", seed=9, norm_jitter=0.2)
        llm = LLM.from_gguf(p, EngineConfig(**ec), device="cpu")
        llm.runner.keep_logits = True
        llm.add_request(prompt, sp)
        llm.step()
        return llm.last_step[1].logits.float()

    full = run([0, 0])
    uniform = run([8, 8], sliding_window=8)
    all_global = run([0, 0], sliding_window=8, sliding_window_pattern=1)
    mixed = run([8, 0], sliding_window=8, sliding_window_pattern=2)
    assert torch.allclose(all_global, full, atol=1e-5)
    assert not torch.allclose(uniform, full, atol=1e-4)
    assert not torch.allclose(mixed, full, atol=1e-4) and not torch.allclose(mixed, uniform, atol=1e-4)


def test_phi3_fused_tensor_layout_gives_the_same_logits_as_the_split_layout(tmp_path):
    """A Phi-3 checkpoint stores one attn_qkv tensor and one gate-then-up ffn_up tensor per layer; loaded (also
    sharded two ways) it must compute exactly what the same weights in the Llama layout compute."""
    import dataclasses

    from oxidize_b200.formats.gguf import load_gguf
    from oxidize_b200.models.config import config_from_gguf
    from oxidize_b200.models.weights import load_weights

    cfg = preset("tiny-llama", n_layers=2, vocab_size=97, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96)
    plain, fused = str(tmp_path / "plain.gguf"), str(tmp_path / "phi3.gguf")
    synth_gguf(plain, cfg, "F32", seed=4, norm_jitter=0.2)
    synth_gguf(fused, dataclasses.replace(cfg, arch="phi3"), "F32", seed=4, norm_jitter=0.2, fused_layout=True)
    g = load_gguf(fused)
    assert g.has_tensor("blk.0.attn_qkv.weight") and not g.has_tensor("blk.0.attn_q.weight")
    assert not g.has_tensor("blk.0.ffn_gate.weight")
    c2 = config_from_gguf(g)
    assert c2.arch == "phi3" and c2.ffn_size == 96 and c2.n_kv_heads == 2
    ec = EngineConfig(max_model_len=64, max_num_seqs=2, num_kv_blocks=32, prefill_chunk_size=32, max_num_batched_tokens=32)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompts = [[5, 9, 20, 31, 7], list(range(3, 30))]
    a = [o.token_ids for o in LLM.from_gguf(plain, ec, device="cpu").generate(prompts, sp)]
    b = [o.token_ids for o in LLM.from_gguf(fused, ec, device="cpu").generate(prompts, sp)]
    assert a == b
    # the shard of a fused tensor is the same rows the split tensors give
    w_plain = load_weights(load_gguf(plain), cfg, "cpu", torch.float32, 1, 2)
    w_fused = load_weights(g, c2, "cpu", torch.float32, 1, 2)
    for la, lb in zip(w_plain.layers, w_fused.layers):
        for pa, pb in zip(la.wqkv.parts + la.w_gate_up.parts, lb.wqkv.parts + lb.w_gate_up.parts):
            assert torch.equal(pa.data, pb.data)


def test_rope_frequency_factors_of_the_checkpoint_are_applied(tmp_path):
    """rope_freqs.weight (Llama-3.1 and later) divides the rotary frequencies pair by pair."""
    from oxidize_b200.ops import ref as opref

    cfg = preset("tiny-llama", n_layers=2, vocab_size=97, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96)
    factors = np.array([1.0, 1.0, 1.0, 2.0, 4.0, 8.0, 8.0, 8.0], dtype=np.float32)
    p0, p1 = str(tmp_path / "plain.gguf"), str(tmp_path / "scaled.gguf")
    synth_gguf(p0, cfg, "F32", seed=4, norm_jitter=0.2)
    synth_gguf(p1, cfg, "F32", seed=4, norm_jitter=0.2, rope_freqs=factors)
    ec = EngineConfig(max_model_len=64, max_num_seqs=2, num_kv_blocks=32, prefill_chunk_size=64, max_num_batched_tokens=64)
    l0, l1 = LLM.from_gguf(p0, ec, device="cpu"), LLM.from_gguf(p1, ec, device="cpu")
    base = opref.rope_inv_freq(16, cfg.rope_theta)
    assert torch.allclose(l0.model.rope.inv_freq, base)
    assert torch.allclose(l1.model.rope.inv_freq, base / torch.from_numpy(factors))
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    for llm in (l0, l1):
        llm.runner.keep_logits = True
        llm.add_request(list(range(3, 40)), sp)
        llm.step()
    assert not torch.allclose(l0.last_step[1].logits.float(), l1.last_step[1].logits.float(), atol=1e-4)
    with pytest.raises(ValueError):
        opref.rope_inv_freq(16, 10000.0, freq_factors=[1.0, 2.0])


def test_streamed_layers_give_the_same_tokens_with_bounded_residency(tmp_path):
    """Layer-wise execution: only `resident_layers` decoder layers are loaded at a time, the rest stream from the file
    mapping as the forward pass reaches them."""
    from oxidize_b200.models.weights import StreamedLayers

    path = str(tmp_path / "m.gguf")
    synth_gguf(path, preset("tiny-llama", n_layers=5, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16,
                            ffn_size=96), "Q8_0", seed=2, norm_jitter=0.1)
    ec = dict(max_model_len=64, max_num_seqs=2, num_kv_blocks=32, prefill_chunk_size=32, max_num_batched_tokens=32)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompts = [[5, 9, 20, 31, 7], list(range(3, 30))]
    full = LLM.from_gguf(path, EngineConfig(**ec), device="cpu")
    want = [o.token_ids for o in full.generate(prompts, sp)]
    llm = LLM.from_gguf(path, EngineConfig(**ec, resident_layers=2), device="cpu")
    layers = llm.weights.layers
    assert isinstance(layers, StreamedLayers) and len(layers) == 5 and layers.loads == 0
    assert [o.token_ids for o in llm.generate(prompts, sp)] == want
    assert len(layers.resident()) == 2 and layers.evictions > 0 and layers.loads == layers.evictions + 2
    assert llm.weights.nbytes() < full.weights.nbytes()
    # a cache as large as the model is the ordinary resident list
    assert isinstance(LLM.from_gguf(path, EngineConfig(**ec, resident_layers=5), device="cpu").weights.layers, list)
    with pytest.raises(IndexError):
        layers[5]


def test_pages_outside_a_uniform_attention_window_return_to_the_pool(tmp_path):
    """Sliding-window model (every layer windowed): a running sequence keeps only the pages its window still reaches;
    the tokens are those of an engine that keeps everything; interleaved local / global models keep everything."""
    path = str(tmp_path / "swa.gguf")
    synth_gguf(path, preset("tiny-llama", arch="mistral", n_layers=2, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2,
                            head_dim=16, ffn_size=96, sliding_window=24), "F32", seed=5, norm_jitter=0.1)
    ec = dict(max_model_len=256, max_num_seqs=2, num_kv_blocks=40, prefill_chunk_size=32, max_num_batched_tokens=64)
    sp = SamplingParams(temperature=0.0, max_tokens=100, ignore_eos=True)
    prompts = [list(range(3, 73)), [5, 9, 20, 31, 7]]
    keep_all = LLM.from_gguf(path, EngineConfig(**ec), device="cpu")
    assert keep_all.scheduler.config.attention_window == 24
    keep_all.scheduler.config.attention_window = 0
    want = [o.token_ids for o in keep_all.generate(prompts, sp)]
    llm = LLM.from_gguf(path, EngineConfig(**ec), device="cpu")
    for p in prompts:
        llm.add_request(p, sp)
    peak_live, total = 0, llm.pool.num_free
    while llm.has_unfinished:
        llm.step()
        for s in llm.scheduler.running:
            live = len(s.blocks) - s._released
            peak_live = max(peak_live, live)
            assert len(set(s.blocks[: s._released + 1])) <= 1  # released slots repeat the first live page's id
    assert peak_live <= 24 // 16 + 3  # window pages + the page being filled + chunk slack, not 170 / 16 = 11
    assert llm.pool.num_free == total  # everything came back, nothing twice
    llm2 = LLM.from_gguf(path, EngineConfig(**ec), device="cpu")
    assert [o.token_ids for o in llm2.generate(prompts, sp)] == want
    # a pool too small for whole sequences is enough once dead pages return: 2 x 170 tokens need 22 pages, 12 suffice
    small = LLM.from_gguf(path, EngineConfig(**{**ec, "num_kv_blocks": 12}), device="cpu")
    assert [o.token_ids for o in small.generate(prompts, sp)] == want and small.scheduler.num_preemptions == 0
    mixed = str(tmp_path / "mixed.gguf")
    synth_gguf(mixed, preset("tiny-llama", n_layers=2, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16,
                             ffn_size=96, sliding_window=24, sliding_window_pattern=2), "F32", seed=5)
    assert LLM.from_gguf(mixed, EngineConfig(**ec), device="cpu").scheduler.config.attention_window == 0


def test_latent_attention_batched_statement_matches_the_paged_reference():
    """ops.ref.latent_attention (what a GPU runs for DeepSeek latent attention) against the generic paged reference on
    the same cache: decode steps (batched path), chunked prefill rows, f32 and q8 caches."""
    from oxidize_b200.engine.kv_pool import KVCache, KVCacheSpec
    from oxidize_b200.models.transformer import BatchMeta
    from oxidize_b200.ops import ref as opref

    torch.manual_seed(0)
    c, r, H, page = 64, 32, 4, 16
    for kvd, tol in (("f32", 1e-5), ("q8", 1e-5)):
        kv = KVCache(KVCacheSpec(1, 1, c + r, page, kvd), 16, "cpu")
        lens = [37, 5, 64]
        tables = torch.tensor([[0, 1, 2, 0], [3, 0, 0, 0], [4, 5, 6, 7]], dtype=torch.int32)
        for b, L in enumerate(lens):
            rows = torch.randn(L, 1, c + r)
            slots = torch.tensor([int(tables[b, p // page]) * page + p % page for p in range(L)], dtype=torch.int32)
            opref.kv_write(kv, 0, rows, rows, slots)
        i32 = dict(dtype=torch.int32)
        # decode: one row per sequence
        q = torch.randn(3, H, c + r)
        meta = BatchMeta(None, None, None, torch.tensor([0, 1, 2, 3], **i32), torch.tensor(lens, **i32), tables, None, 1, 64, 3)
        want = opref.paged_attention(q, kv, 0, meta, 0.1)[:, :, :c]
        assert torch.allclose(opref.latent_attention(q, kv, 0, meta, 0.1, c), want, atol=tol)
        # mixed step: 7 prefill rows of sequence 0, 1 row of sequence 1, 3 rows of sequence 2
        q = torch.randn(11, H, c + r)
        meta = BatchMeta(None, None, None, torch.tensor([0, 7, 8, 11], **i32), torch.tensor(lens, **i32), tables, None, 7, 64, 3)
        want = opref.paged_attention(q, kv, 0, meta, 0.1)[:, :, :c]
        assert torch.allclose(opref.latent_attention(q, kv, 0, meta, 0.1, c), want, atol=tol)


def test_latent_attention_model_gives_the_same_logits_through_the_batched_statement(tmp_path):
    """The DeepSeek model path a GPU takes (ops.ref.latent_attention inside the layer) against the CPU's paged reference:
    prefill chunks and decode steps, two sequences."""
    path = str(tmp_path / "ds.gguf")
    cfg = preset("deepseek-v3", n_layers=3, vocab_size=512, hidden_size=64, n_heads=4, n_kv_heads=4, head_dim=48, rope_dim=32,
                 qk_nope_dim=16, v_head_dim=24, kv_lora_rank=32, q_lora_rank=48, ffn_size=96, n_experts=8, n_experts_used=2,
                 expert_ffn_size=48, expert_group_count=4, expert_group_used_count=2, leading_dense_blocks=1,
                 shared_expert_ffn_size=48, context_length=4096)
    synth_gguf(path, cfg, "F32", seed=0, norm_jitter=0.1)
    ec = dict(max_model_len=128, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=16, max_num_batched_tokens=32)
    prompts = [[5, 9, 200, 31, 7], list(range(3, 60))]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    outs = []
    for statement in (False, True):
        for kvd in ("f32", "q8"):
            llm = LLM.from_gguf(path, EngineConfig(**ec, kv_cache_dtype=kvd), device="cpu")
            llm.model.latent_statement = statement
            outs.append([o.token_ids for o in llm.generate(prompts, sp)])
    assert outs[0] == outs[2] and outs[1] == outs[3]


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_traffic_on_a_small_pool_with_window_release(tmp_path, seed):
    """Random arrivals, lengths and aborts on a sliding-window model with a pool that forces preemption: every request
    finishes with the tokens a roomy, keep-everything engine gives, and the pool is whole again at the end (no page freed
    twice or lost across release, preemption, prefix sharing and abort)."""
    import random

    rnd = random.Random(seed)
    path = str(tmp_path / "swa.gguf")
    synth_gguf(path, preset("tiny-llama", arch="mistral", n_layers=2, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2,
                            head_dim=16, ffn_size=96, sliding_window=20), "F32", seed=7, norm_jitter=0.1)
    shared = [rnd.randrange(3, 290) for _ in range(40)]  # a common prefix: prefix-cache sharing among requests
    reqs = []
    for i in range(10):
        prompt = (shared[: rnd.choice([0, 16, 32, 40])] + [rnd.randrange(3, 290) for _ in range(rnd.randrange(1, 50))])
        reqs.append((prompt, rnd.randrange(1, 60)))
    ec = dict(max_model_len=160, max_num_seqs=4, prefill_chunk_size=16, max_num_batched_tokens=48)
    roomy = LLM.from_gguf(path, EngineConfig(**ec, num_kv_blocks=128), device="cpu")
    roomy.scheduler.config.attention_window = 0
    want = {}
    for i, (p, n) in enumerate(reqs):
        want[f"r{i}"] = roomy.generate([p], SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True))[0].token_ids
    llm = LLM.from_gguf(path, EngineConfig(**ec, num_kv_blocks=7), device="cpu")
    assert llm.scheduler.config.attention_window == 20
    pending = list(enumerate(reqs))
    got, aborted = {}, set()
    steps = 0
    while pending or llm.has_unfinished:
        for _ in range(rnd.randrange(0, 3)):
            if pending:
                i, (p, n) = pending.pop(0)
                llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True), request_id=f"r{i}")
        if steps == 25 and llm.scheduler.running:
            victim = llm.scheduler.running[0].request_id  # one request is cancelled in mid-flight
            llm.abort(victim)
            aborted.add(victim)
        for o in llm.step():
            if o.finished:
                got[o.request_id] = o.token_ids
        steps += 1
        assert steps < 5000
    for rid, toks in want.items():
        if rid not in aborted:
            assert got[rid] == toks, rid
    assert not llm.scheduler.running and not llm.scheduler.waiting
    # every page is free or held only by the prefix cache (refcount zero): a fresh request can take the whole pool
    assert llm.pool.can_allocate(7)
    assert llm.scheduler.num_preemptions > 0  # the pool was small enough to make the scheduler evict and recompute


def test_experts_per_token_override(tmp_path):
    path = str(tmp_path / "moe.gguf")
    synth_gguf(path, preset("mixtral-8x7b", n_layers=2, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16,
                            ffn_size=96, n_experts=4, n_experts_used=2, expert_ffn_size=32), "F32", seed=0)
    ec = dict(max_model_len=64, max_num_seqs=2, num_kv_blocks=16)
    base = LLM.from_gguf(path, EngineConfig(**ec), device="cpu")
    more = LLM.from_gguf(path, EngineConfig(**ec), device="cpu", experts_per_token=4)
    assert base.cfg.n_experts_used == 2 and more.cfg.n_experts_used == 4
    a, b = base.next_token_logits([[5, 9, 20]]), more.next_token_logits([[5, 9, 20]])
    assert not np.allclose(a, b, atol=1e-5)
    with pytest.raises(ValueError):
        LLM.from_gguf(path, EngineConfig(**ec), device="cpu", experts_per_token=5)


def test_weights_are_transcoded_at_load_time_on_request(tmp_path):
    path = str(tmp_path / "m.gguf")
    synth_gguf(path, preset("tiny-llama", n_layers=2, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16,
                            ffn_size=96), "F32", seed=2, norm_jitter=0.1)
    ec = dict(max_model_len=64, max_num_seqs=2, num_kv_blocks=16)
    f32 = LLM.from_gguf(path, EngineConfig(**ec), device="cpu")
    q8 = LLM.from_gguf(path, EngineConfig(**ec, weight_transcode="Q8_0"), device="cpu")
    q4 = LLM.from_gguf(path, EngineConfig(**ec, weight_transcode="q4_0"), device="cpu")
    lw = q8.weights.layers[0]
    assert {p.qtype for p in lw.wqkv.parts + lw.wo.parts + lw.w_gate_up.parts + lw.w_down.parts} == {"Q8_0"}
    assert q8.weights.embed.qtype == "F32" and q4.weights.layers[1].w_down.parts[0].qtype == "Q4_0"
    assert q4.weights.nbytes() < q8.weights.nbytes() < f32.weights.nbytes()
    a, b, c = (m.next_token_logits([[5, 9, 20, 31]])[0] for m in (f32, q8, q4))
    e8, e4 = np.abs(a - b).max() / np.abs(a).max(), np.abs(a - c).max() / np.abs(a).max()
    assert 0 < e8 < 0.02 and e8 < e4 < 0.3
    with pytest.raises(ValueError):
        LLM.from_gguf(path, EngineConfig(**ec, weight_transcode="Q6_K"), device="cpu")
