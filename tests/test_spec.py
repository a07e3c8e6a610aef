"""Speculative decoding keeps greedy output exact, for a perfect draft, a bad draft and the MTP head."""
import numpy as np
import pytest

from oxidize_b200.engine.llm import LLM, EngineConfig
from oxidize_b200.engine.sampler import SamplingParams
from oxidize_b200.engine.spec import (DraftModelProposer, MtpProposer, SpecDecoder, SpecStats, attach_speculation,
                                      verify_greedy)
from oxidize_b200.models.config import preset
from oxidize_b200.utils.synth import synth_gguf, synth_weights

EC = dict(max_model_len=160, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=32, max_num_batched_tokens=96)
SP = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
PROMPTS = [[5, 9, 200, 31, 7], list(range(3, 40)), [100, 101]]


def test_verify_greedy_rule():
    assert verify_greedy([1, 2, 3], [1, 2, 3, 9]) == [1, 2, 3, 9]
    assert verify_greedy([1, 2, 3], [1, 7, 3, 9]) == [1, 7]
    assert verify_greedy([4], [5, 6]) == [5]


def test_stats():
    s = SpecStats(proposed=40, accepted=30, target_forwards=10, emitted=40)
    assert s.acceptance_rate == 0.75 and s.tokens_per_target_forward == 4.0
    assert s.estimated_speedup(0.1, 4) == pytest.approx(4.0 / 1.4)


@pytest.fixture(scope="module")
def target_path(tmp_path_factory):
    cfg = preset("tiny-llama", n_layers=2, vocab_size=300)
    p = str(tmp_path_factory.mktemp("spec") / "target.gguf")
    synth_gguf(p, cfg, "F16", seed=0, norm_jitter=0.05)
    return p


def _plain(path):
    return [o.token_ids for o in LLM.from_gguf(path, EngineConfig(**EC), device="cpu").generate(PROMPTS, SP)]


def test_perfect_draft_accepts_everything(target_path):
    want = _plain(target_path)
    llm = LLM.from_gguf(target_path, EngineConfig(**EC), device="cpu")
    spec = attach_speculation(llm, target_path, k=3)
    got = [o.token_ids for o in llm.generate(PROMPTS, SP)]
    assert got == want
    assert spec.stats.acceptance_rate > 0.95 and spec.stats.tokens_per_target_forward > 2.0
    assert llm.pool.num_free == llm.pool.num_blocks and spec.proposer.pool.num_free == spec.proposer.pool.num_blocks


def test_bad_draft_is_still_exact(target_path, tmp_path):
    want = _plain(target_path)
    dcfg = preset("tiny-llama", n_layers=1, vocab_size=300, hidden_size=128, n_heads=4, n_kv_heads=2, head_dim=32,
                  ffn_size=256)
    dpath = str(tmp_path / "draft.gguf")
    synth_gguf(dpath, dcfg, "F16", seed=7)
    llm = LLM.from_gguf(target_path, EngineConfig(**EC), device="cpu")
    spec = attach_speculation(llm, dpath, k=4)
    got = [o.token_ids for o in llm.generate(PROMPTS, SP)]
    assert got == want
    assert spec.stats.proposed > 0 and spec.stats.acceptance_rate < 0.9


def test_mtp_head_is_exact(tmp_path):
    cfg = preset("tiny-llama", n_layers=2, vocab_size=300, nextn_layers=1)
    path = str(tmp_path / "mtp.gguf")
    synth_gguf(path, cfg, "F16", seed=3, norm_jitter=0.05)
    plain = LLM.from_gguf(path, EngineConfig(**EC), device="cpu")
    assert len(plain.weights.mtp) == 1 and len(plain.weights.layers) == 2
    want = [o.token_ids for o in plain.generate(PROMPTS, SP)]
    llm = LLM.from_gguf(path, EngineConfig(**EC), device="cpu")
    spec = attach_speculation(llm, None, k=2, use_mtp=True)
    got = [o.token_ids for o in llm.generate(PROMPTS, SP)]
    assert got == want and spec.stats.target_forwards > 0 and spec.stats.proposed > 0


def _first_token_histogram(accept_fn, V, trials, seed):
    """Draft one token from q, verify it against p, and count what comes out first; must be distributed as p."""
    rng = np.random.default_rng(seed)
    tl = rng.normal(0, 1.5, (2, V)).astype(np.float32)  # target rows 0 (verify) and 1 (bonus)
    dl = rng.normal(0, 1.5, (1, V)).astype(np.float32)
    T = 0.8
    from oxidize_b200.engine.sampler import probs_from_logits

    p, q = probs_from_logits(tl[0], T), probs_from_logits(dl[0], T)
    drafts = rng.choice(V, size=trials, p=q)
    uni = rng.random((trials, 3)).astype(np.float32)
    first, accepted = accept_fn(tl, dl, drafts, uni, T)
    hist = np.bincount(first, minlength=V).astype(np.float64)
    exp = p * trials
    chi2 = float(((hist - exp) ** 2 / np.maximum(exp, 1e-9)).sum())
    # acceptance probability of the rule: sum_v min(p, q)
    want_acc = float(np.minimum(p, q).sum())
    return chi2, accepted / trials, want_acc


def test_rejection_rule_preserves_the_target_distribution_on_host():
    from oxidize_b200.engine.sampler import probs_from_logits, speculative_accept

    V, trials = 17, 20000
    sp = SamplingParams(temperature=0.8)

    def host(tl, dl, drafts, uni, T):
        q = [probs_from_logits(dl[0], T)]
        first, acc = [], 0
        for d, u in zip(drafts, uni):
            out, n = speculative_accept([int(d)], q, tl, sp, [float(x) for x in u])
            first.append(out[0])
            acc += n
        return np.asarray(first), acc

    chi2, acc, want_acc = _first_token_histogram(host, V, trials, seed=4)
    assert chi2 < 45.0, chi2  # 16 degrees of freedom: p(chi2 > 45) < 2e-4
    assert abs(acc - want_acc) < 0.02


def test_sampled_speculation_runs_through_the_engine(target_path, tmp_path):
    """Temperature sampling with a draft model: drafts are sampled, verified with the rejection rule, every request gets
    its tokens; a draft identical to the target is accepted (p = q), a poor one is not, and requests whose sampling
    parameters the rule does not cover run without drafts."""
    sp = SamplingParams(temperature=0.9, max_tokens=20, ignore_eos=True, seed=11)
    llm = LLM.from_gguf(target_path, EngineConfig(**EC), device="cpu")
    spec = attach_speculation(llm, target_path, k=3)
    outs = llm.generate(PROMPTS, sp)
    assert all(len(o.token_ids) == 20 and all(0 <= t < 300 for t in o.token_ids) for o in outs)
    assert spec.stats.proposed > 0 and spec.stats.acceptance_rate > 0.9, spec.stats
    assert llm.pool.num_free == llm.pool.num_blocks and spec.proposer.pool.num_free == spec.proposer.pool.num_blocks

    dcfg = preset("tiny-llama", n_layers=1, vocab_size=300, hidden_size=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn_size=256)
    dpath = str(tmp_path / "draft_s.gguf")
    synth_gguf(dpath, dcfg, "F16", seed=7)
    llm2 = LLM.from_gguf(target_path, EngineConfig(**EC), device="cpu")
    spec2 = attach_speculation(llm2, dpath, k=3)
    outs2 = llm2.generate(PROMPTS, sp)
    assert all(len(o.token_ids) == 20 for o in outs2)
    assert spec2.stats.proposed > 0 and spec2.stats.acceptance_rate < spec.stats.acceptance_rate

    llm3 = LLM.from_gguf(target_path, EngineConfig(**EC), device="cpu")
    spec3 = attach_speculation(llm3, target_path, k=3)
    llm3.generate(PROMPTS, SamplingParams(temperature=0.9, top_k=5, max_tokens=8, ignore_eos=True, seed=1))
    assert spec3.stats.proposed == 0


def test_self_speculation_over_a_4bit_cache(tmp_path):
    """--quantspec: the model drafts for itself over a q4 copy of its cache; the output is the plain greedy output and
    nearly every draft is accepted (the draft is the target up to cache rounding)."""
    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.engine.sampler import SamplingParams
    from oxidize_b200.engine.spec import attach_speculation
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    path = str(tmp_path / "m.gguf")
    synth_gguf(path, preset("tiny-llama", n_layers=2, vocab_size=300, hidden_size=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn_size=256),
               "F32", seed=2, norm_jitter=0.1)
    ec = dict(max_model_len=128, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=32, max_num_batched_tokens=64)
    prompts = [[5, 9, 200, 31, 7], list(range(3, 40))]
    sp = SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)
    plain = [o.token_ids for o in LLM.from_gguf(path, EngineConfig(**ec), device="cpu").generate(prompts, sp)]
    llm = LLM.from_gguf(path, EngineConfig(**ec), device="cpu")
    spec = attach_speculation(llm, None, k=4, quantspec=True)
    assert spec.proposer.kv.spec.dtype_name == "q4" and spec.proposer.model.w is llm.weights
    assert [o.token_ids for o in llm.generate(prompts, sp)] == plain
    assert spec.stats.acceptance_rate > 0.7 and spec.stats.tokens_per_target_forward > 2.5
