"""Hidden-conditioned (DFlash-style) draft model: its batched, paged forward against a plain dense restatement of the
architecture, and exactness of speculative decoding with it."""
import numpy as np
import pytest
import torch

from oxidize_b200.engine.feature_draft import FeatureDraftProposer, feature_draft_config, load_feature_draft
from oxidize_b200.engine.llm import LLM, EngineConfig
from oxidize_b200.engine.sampler import SamplingParams
from oxidize_b200.engine.scheduler import Sequence
from oxidize_b200.engine.spec import attach_speculation
from oxidize_b200.formats.gguf import GGUFValueType, GGUFWriter, load_gguf
from oxidize_b200.models.config import preset
from oxidize_b200.ops import ref as opref
from oxidize_b200.utils.synth import synth_gguf

H, HEADS, KV, HD, FFN, LAYERS = 64, 4, 2, 16, 96, 2
TARGET_IDS = [0, 2]


def _draft_file(path, seed=0, scale=0.15):
    rng = np.random.default_rng(seed)
    w = GGUFWriter(path, arch="dflash-draft")
    U = GGUFValueType.UINT32
    for k, v in (("hidden_size", H), ("num_hidden_layers", LAYERS), ("num_attention_heads", HEADS), ("num_key_value_heads", KV),
                 ("intermediate_size", FFN), ("block_size", 16), ("mask_token_id", 7)):
        w.add(f"dflash-draft.{k}", v, U)
    w.add("dflash-draft.rope_theta", 10000.0, GGUFValueType.FLOAT32)
    w.add("dflash-draft.target_layer_ids", TARGET_IDS)
    t = {}

    def mat(name, o, i):
        t[name] = (rng.standard_normal((o, i)) * scale).astype(np.float32)
        w.add_tensor(name, t[name], (o, i), "F32")

    def vec(name, n):
        t[name] = (1.0 + 0.2 * rng.standard_normal(n)).astype(np.float32)
        w.add_tensor(name, t[name], (n,), "F32")

    mat("fc.weight", H, len(TARGET_IDS) * H)
    vec("hidden_norm.weight", H)
    for i in range(LAYERS):
        p = f"blk.{i}"
        vec(f"{p}.attn_norm.weight", H)
        mat(f"{p}.attn_q.weight", HEADS * HD, H)
        mat(f"{p}.attn_k.weight", KV * HD, H)
        mat(f"{p}.attn_v.weight", KV * HD, H)
        mat(f"{p}.attn_output.weight", H, HEADS * HD)
        vec(f"{p}.attn_q_norm.weight", HD)
        vec(f"{p}.attn_k_norm.weight", HD)
        vec(f"{p}.ffn_norm.weight", H)
        mat(f"{p}.ffn_gate.weight", FFN, H)
        mat(f"{p}.ffn_up.weight", FFN, H)
        mat(f"{p}.ffn_down.weight", H, FFN)
    vec("output_norm.weight", H)
    w.write()
    return {k: torch.from_numpy(v) for k, v in t.items()}


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    d = tmp_path_factory.mktemp("fd")
    target = str(d / "target.gguf")
    synth_gguf(target, preset("tiny-llama", n_layers=3, vocab_size=300, hidden_size=H, n_heads=4, n_kv_heads=2, head_dim=16,
                              ffn_size=96), "F32", seed=3, norm_jitter=0.1)
    draft = str(d / "draft.gguf")
    return target, draft, _draft_file(draft)


def _norm(x, w, eps=1e-5):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _dense_reference(t, embed, tokens, first_pos, feats_at):
    """The reference's token-by-token forward (dflash.rs:1119-1404) in plain torch: per layer a growing list of (k, v)
    entries; a token with target features first appends the entry of the context vector."""
    inv = opref.rope_inv_freq(HD, 10000.0)
    caches = [([], []) for _ in range(LAYERS)]
    out = None
    for j, tok in enumerate(tokens):
        pos = torch.tensor([first_pos + j])
        x = embed[tok].clone()
        ctx = None
        if j in feats_at:
            ctx = _norm(t["fc.weight"] @ feats_at[j], t["hidden_norm.weight"])
        for li in range(LAYERS):
            p = f"blk.{li}"
            n = _norm(x, t[f"{p}.attn_norm.weight"])
            q = (t[f"{p}.attn_q.weight"] @ n).reshape(1, HEADS, HD)
            ks, vs = caches[li]

            def key_of(vec_in):
                k = _norm((t[f"{p}.attn_k.weight"] @ vec_in).reshape(1, KV, HD), t[f"{p}.attn_k_norm.weight"])
                return opref.apply_rope(k, pos, inv)[0]

            if ctx is not None:
                ks.append(key_of(ctx))
                vs.append((t[f"{p}.attn_v.weight"] @ ctx).reshape(KV, HD))
            ks.append(key_of(n))
            vs.append((t[f"{p}.attn_v.weight"] @ n).reshape(KV, HD))
            q = opref.apply_rope(_norm(q, t[f"{p}.attn_q_norm.weight"]), pos, inv)[0]
            K, V = torch.stack(ks), torch.stack(vs)  # [L, KV, HD]
            g = HEADS // KV
            s = torch.einsum("kgd,lkd->kgl", q.reshape(KV, g, HD), K) * HD ** -0.5
            o = torch.einsum("kgl,lkd->kgd", torch.softmax(s, -1), V).reshape(HEADS * HD)
            x = x + t[f"{p}.attn_output.weight"] @ o
            n2 = _norm(x, t[f"{p}.ffn_norm.weight"])
            x = x + t[f"{p}.ffn_down.weight"] @ (torch.nn.functional.silu(t[f"{p}.ffn_gate.weight"] @ n2) * (t[f"{p}.ffn_up.weight"] @ n2))
        out = _norm(x, t["output_norm.weight"])
    return out


def test_config_and_loader(setup):
    target, draft, _ = setup
    fc = feature_draft_config(load_gguf(draft), 3)
    assert fc.target_layer_ids == TARGET_IDS and fc.block_size == 16 and fc.mask_token_id == 7
    m = fc.model
    assert (m.hidden_size, m.n_layers, m.n_heads, m.n_kv_heads, m.head_dim, m.ffn_size, m.qk_norm) == (H, LAYERS, HEADS, KV, HD, FFN, True)
    w = load_feature_draft(draft, "cpu", torch.float32, 3)
    assert w.embed is None and w.lm_head is None and w.fc.shape == (H, 2 * H) and len(w.layers) == LAYERS
    with pytest.raises(ValueError):
        feature_draft_config(load_gguf(draft), 2)  # layer 2 does not exist in a 2-layer target
    with pytest.raises(ValueError):
        feature_draft_config(load_gguf(target), 3)  # an ordinary checkpoint has no fc.weight


def test_paged_batched_forward_matches_the_dense_statement(setup):
    target, draft, t = setup
    llm = LLM.from_gguf(target, EngineConfig(max_model_len=128, max_num_seqs=4, num_kv_blocks=64), device="cpu")
    prop = FeatureDraftProposer(load_feature_draft(draft, "cpu", torch.float32, 3), llm.model, 3, 4, 128)
    embed = llm.model.w.embed.dense_cache()
    gen = torch.Generator().manual_seed(0)
    a, b = Sequence(list(range(5, 25)), SamplingParams(temperature=0.0)), Sequence([9, 8, 7], SamplingParams(temperature=0.0))
    fa, fb = torch.randn(2 * H, generator=gen), torch.randn(2 * H, generator=gen)
    from oxidize_b200.engine.feature_draft import _SeqState

    prop.state[a.seq_id], prop.state[b.seq_id] = _SeqState(), _SeqState()
    # catch-up pass for both (19 and 2 tokens), then one token each with a context entry, then one without
    prop._forward([a, b], [a.prompt[:-1], b.prompt[:-1]], [0, 0], [None, None])
    h1 = prop._forward([a, b], [[a.prompt[-1]], [b.prompt[-1]]], [19, 2], [fa, fb])
    h2 = prop._forward([a, b], [[77], [78]], [20, 3], [None, None])
    assert prop.state[a.seq_id].entries == 22 and prop.state[b.seq_id].entries == 5  # one extra entry each: the context
    want1a = _dense_reference(t, embed, a.prompt, 0, {19: fa})
    want2a = _dense_reference(t, embed, a.prompt + [77], 0, {19: fa})
    want2b = _dense_reference(t, embed, b.prompt + [78], 0, {2: fb})
    assert torch.allclose(h1[0], want1a, atol=2e-5) and torch.allclose(h2[0], want2a, atol=2e-5)
    assert torch.allclose(h2[1], want2b, atol=2e-5)
    # rollback drops the last token's entry and it can be fed again with the same result
    prop.rollback(a, 20)
    prop.rollback(b, 3)
    assert prop.state[a.seq_id].entries == 21 and prop.state[a.seq_id].seen == 20
    again = prop._forward([a, b], [[77], [78]], [20, 3], [None, None])
    assert torch.allclose(again, h2, atol=1e-6)


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_speculation_with_a_feature_draft_is_exact(setup, temperature):
    target, draft, _ = setup
    ec = dict(max_model_len=128, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=32, max_num_batched_tokens=64)
    prompts = [[5, 9, 200, 31, 7], list(range(3, 40))]
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    plain = [o.token_ids for o in LLM.from_gguf(target, EngineConfig(**ec), device="cpu").generate(prompts, sp)]
    llm = LLM.from_gguf(target, EngineConfig(**ec), device="cpu")
    spec = attach_speculation(llm, draft, k=3)
    assert isinstance(spec.proposer, FeatureDraftProposer) and llm.model.capture_layers == TARGET_IDS
    if temperature == 0.0:
        got = [o.token_ids for o in llm.generate(prompts, sp)]
        assert got == plain
        assert spec.stats.proposed > 0 and spec.stats.target_forwards > 0 and spec.proposer.context_entries > 0
        assert len(spec.proposer.features) == 0 and not spec.proposer.state  # released with their sequences
    else:
        # sampled requests: drafts are drawn from the draft's distribution and verified by rejection sampling; with a
        # seed the run is reproducible and every token is a valid vocabulary entry
        sps = SamplingParams(temperature=temperature, max_tokens=16, ignore_eos=True, seed=11)
        a = [o.token_ids for o in llm.generate(prompts, sps)]
        llm2 = LLM.from_gguf(target, EngineConfig(**ec), device="cpu")
        attach_speculation(llm2, draft, k=3)
        b = [o.token_ids for o in llm2.generate(prompts, sps)]
        assert a == b and all(len(x) == 16 and all(0 <= t < 300 for t in x) for x in a)


# --------------------------------------------------------------------------- EAGLE-3

DV = 100  # draft vocabulary; target id = 3 * draft id


def _eagle_file(path, seed=1, scale=0.15, norm_before_residual=False):
    rng = np.random.default_rng(seed)
    w = GGUFWriter(path, arch="eagle3")
    U = GGUFValueType.UINT32
    for k, v in (("hidden_size", H), ("num_attention_heads", HEADS), ("num_key_value_heads", KV), ("head_dim", HD)):
        w.add(f"eagle3.{k}", v, U)
    w.add("eagle3.extract_layers", [0, 1, 2])
    w.add("eagle3.norm_before_residual", bool(norm_before_residual))
    t = {}

    def mat(name, o, i):
        t[name] = (rng.standard_normal((o, i)) * scale).astype(np.float32)
        w.add_tensor(name, t[name], (o, i), "F32")

    def vec(name, n):
        t[name] = (1.0 + 0.2 * rng.standard_normal(n)).astype(np.float32)
        w.add_tensor(name, t[name], (n,), "F32")

    mat("fc.weight", H, 3 * H)
    w.add_tensor("d2t", (2 * np.arange(DV)).astype(np.int64), (DV,), "I64")
    p = "blk.0"
    vec(f"{p}.attn_norm.weight", H); vec(f"{p}.attn_norm_2.weight", H); vec(f"{p}.ffn_norm.weight", H)
    mat(f"{p}.attn_q.weight", HEADS * HD, 2 * H); mat(f"{p}.attn_k.weight", KV * HD, 2 * H); mat(f"{p}.attn_v.weight", KV * HD, 2 * H)
    mat(f"{p}.attn_output.weight", H, HEADS * HD)
    mat(f"{p}.ffn_gate.weight", FFN, H); mat(f"{p}.ffn_up.weight", FFN, H); mat(f"{p}.ffn_down.weight", H, FFN)
    vec("output_norm.weight", H)
    mat("output.weight", DV, H)
    w.write()
    return {k: torch.from_numpy(v) for k, v in t.items()}


def _eagle_dense(t, embed, tokens, first_pos, feats, norm_before_residual=False):
    """eagle3.rs:444-660 in plain torch: g = fc(features); per token [norm(embed) ; norm_2(g)] -> block -> g."""
    inv = opref.rope_inv_freq(HD, 10000.0)
    g = t["fc.weight"] @ feats
    ks, vs, out = [], [], []
    p = "blk.0"
    for j, tok in enumerate(tokens):
        pos = torch.tensor([first_pos + j])
        e = _norm(embed[tok], t[f"{p}.attn_norm.weight"])
        gn = _norm(g, t[f"{p}.attn_norm_2.weight"])
        x2 = torch.cat([e, gn])
        q = opref.apply_rope((t[f"{p}.attn_q.weight"] @ x2).reshape(1, HEADS, HD), pos, inv)[0]
        ks.append(opref.apply_rope((t[f"{p}.attn_k.weight"] @ x2).reshape(1, KV, HD), pos, inv)[0])
        vs.append((t[f"{p}.attn_v.weight"] @ x2).reshape(KV, HD))
        K, V = torch.stack(ks), torch.stack(vs)
        s = torch.einsum("kgd,lkd->kgl", q.reshape(KV, HEADS // KV, HD), K) * HD ** -0.5
        o = torch.einsum("kgl,lkd->kgd", torch.softmax(s, -1), V).reshape(HEADS * HD)
        hidden = t[f"{p}.attn_output.weight"] @ o + (gn if norm_before_residual else g)
        n2 = _norm(hidden, t[f"{p}.ffn_norm.weight"])
        hidden = hidden + t[f"{p}.ffn_down.weight"] @ (torch.nn.functional.silu(t[f"{p}.ffn_gate.weight"] @ n2) * (t[f"{p}.ffn_up.weight"] @ n2))
        g = hidden
        out.append((hidden, t["output.weight"] @ _norm(hidden, t["output_norm.weight"])))
    return out


@pytest.mark.parametrize("nbr", [False, True])
def test_eagle3_steps_match_the_dense_statement(setup, tmp_path, nbr):
    from oxidize_b200.engine.feature_draft import Eagle3Proposer, _EagleState, load_eagle3

    target, _, _ = setup
    path = str(tmp_path / "eagle.gguf")
    t = _eagle_file(path, norm_before_residual=nbr)
    llm = LLM.from_gguf(target, EngineConfig(max_model_len=128, max_num_seqs=4, num_kv_blocks=64), device="cpu")
    ew = load_eagle3(path, "cpu", torch.float32, 3, H)
    assert ew.extract_layers == [0, 1, 2] and ew.norm_before_residual == nbr and ew.model.vocab_size == DV and ew.embed is None
    prop = Eagle3Proposer(ew, llm.model, 3, 4, 128)
    assert llm.model.capture_layers == [0, 1, 2]
    embed = llm.model.w.embed.dense_cache()
    gen = torch.Generator().manual_seed(0)
    fa, fb = torch.randn(3 * H, generator=gen), torch.randn(3 * H, generator=gen)
    a, b = Sequence([1] * 20 + [41], SamplingParams(temperature=0.0)), Sequence([2, 3, 57], SamplingParams(temperature=0.0))
    for s, pos0 in ((a, 20), (b, 2)):
        prop.state[s.seq_id] = _EagleState(first=pos0)
    g = torch.stack([t["fc.weight"] @ fa, t["fc.weight"] @ fb])
    g1, l1 = prop._step([a, b], [41, 57], [20, 2], g)
    g2, l2 = prop._step([a, b], [77, 78], [21, 3], g1)
    wa = _eagle_dense(t, embed, [41, 77], 20, fa, nbr)
    wb = _eagle_dense(t, embed, [57, 78], 2, fb, nbr)
    assert torch.allclose(g1[0], wa[0][0], atol=2e-5) and torch.allclose(l2[0], wa[1][1], atol=2e-5)
    assert torch.allclose(g2[1], wb[1][0], atol=2e-5) and torch.allclose(l1[1], wb[0][1], atol=2e-5)
    assert prop._to_target_vocab(torch.tensor([0, 5, 99])).tolist() == [0, 15, 297]
    with pytest.raises(ValueError):
        load_eagle3(path, "cpu", torch.float32, 2, H)  # layer 2 of a 2-layer target
    with pytest.raises(ValueError):
        load_eagle3(path, "cpu", torch.float32, 3, H + 8)


def test_speculation_with_an_eagle3_head_is_exact(setup, tmp_path):
    from oxidize_b200.engine.feature_draft import Eagle3Proposer

    target, _, _ = setup
    path = str(tmp_path / "eagle.gguf")
    _eagle_file(path)
    ec = dict(max_model_len=128, max_num_seqs=4, num_kv_blocks=64, prefill_chunk_size=32, max_num_batched_tokens=64)
    prompts = [[5, 9, 200, 31, 7], list(range(3, 40))]
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    plain = [o.token_ids for o in LLM.from_gguf(target, EngineConfig(**ec), device="cpu").generate(prompts, sp)]
    llm = LLM.from_gguf(target, EngineConfig(**ec), device="cpu")
    spec = attach_speculation(llm, path, k=3)
    assert isinstance(spec.proposer, Eagle3Proposer)
    assert [o.token_ids for o in llm.generate(prompts, sp)] == plain
    assert spec.stats.proposed > 0 and not spec.proposer.state
    # sampled requests: reproducible with a seed, drafts come from the draft vocabulary's image in the target's
    sps = SamplingParams(temperature=0.8, max_tokens=12, ignore_eos=True, seed=5)
    llm2 = LLM.from_gguf(target, EngineConfig(**ec), device="cpu")
    attach_speculation(llm2, path, k=3)
    a = [o.token_ids for o in llm2.generate(prompts, sps)]
    llm3 = LLM.from_gguf(target, EngineConfig(**ec), device="cpu")
    attach_speculation(llm3, path, k=3)
    assert a == [o.token_ids for o in llm3.generate(prompts, sps)] and all(len(x) == 12 for x in a)
