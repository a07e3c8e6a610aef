"""Model semantics against an independent oracle: the Hugging Face `transformers` implementations, on CPU in float32.

A tiny random-init model of each family is saved as SafeTensors + config.json, converted to GGUF by this package's
converter, loaded by the engine and run through the ordinary serving path (chunked prefill, paged KV, greedy decode).
The logits after the prompt and the greedy continuation must agree with the oracle's.  This covers the converter's
tensor-name map and metadata, the loader, and every family-specific piece of layer math: q/k/v biases (Qwen2), per-head
QK-norm (Qwen3), fused qkv / gate-up tensors (Phi-3), softmax top-k routing (Mixtral, Qwen3-MoE), and for Gemma 1-3 the
scaled embeddings, GeGLU, norms on the branch outputs, (w + 1) norm weights, soft-capped scores and logits, the softmax
scale taken from query_pre_attn_scalar, and local / global layers with a window and two rotary bases; for DeepSeek-V2/V3
the latent attention (low-rank and full-rank queries, shared rotary key, interleaved rotary pairs, YaRN), softmax and
sigmoid group-limited routing with a selection bias, the shared expert and the leading dense layer; for LFM2 the gated
short-convolution layers, whose history lives in a second paged cache and crosses prefill chunks; for Mamba the selective
state-space recurrence with its per-sequence state carried across chunks and decode steps.
"""
import os

import pytest
import torch

T = pytest.importorskip("transformers")

from oxidize_b200.engine.llm import LLM, EngineConfig  # noqa: E402
from oxidize_b200.engine.sampler import SamplingParams  # noqa: E402
from oxidize_b200.formats.convert import convert_safetensors_to_gguf  # noqa: E402
from oxidize_b200.formats.gguf import load_gguf  # noqa: E402
from oxidize_b200.models.config import config_from_gguf  # noqa: E402

VOCAB = 199
COMMON = dict(vocab_size=VOCAB, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=256, attn_implementation="eager")


def _build(name: str):
    c = dict(COMMON)
    if name == "llama":
        return T.LlamaForCausalLM(T.LlamaConfig(**c))
    if name == "qwen2":
        return T.Qwen2ForCausalLM(T.Qwen2Config(**c))
    if name == "qwen3":
        return T.Qwen3ForCausalLM(T.Qwen3Config(**c, head_dim=32))
    if name == "phi3":
        return T.Phi3ForCausalLM(T.Phi3Config(**c, pad_token_id=0))
    if name == "mixtral":
        return T.MixtralForCausalLM(T.MixtralConfig(**c, num_local_experts=4, num_experts_per_tok=2))
    if name == "qwen3moe":
        return T.Qwen3MoeForCausalLM(T.Qwen3MoeConfig(**c, head_dim=32, num_experts=8, num_experts_per_tok=2,
                                                      moe_intermediate_size=48, norm_topk_prob=True))
    if name == "gemma":
        return T.GemmaForCausalLM(T.GemmaConfig(**c, head_dim=32))
    if name == "gemma2":
        # window 8 on every other layer, soft caps 50 / 30, softmax scale 24 ** -0.5 (not head_dim ** -0.5)
        return T.Gemma2ForCausalLM(T.Gemma2Config(**c, head_dim=32, sliding_window=8, query_pre_attn_scalar=24))
    if name == "gemma3":
        # 7 layers: five windowed (rotary base 1e4), the sixth global (base 1e6), the seventh windowed again
        c["num_hidden_layers"] = 7
        return T.Gemma3ForCausalLM(T.Gemma3TextConfig(**c, head_dim=32, sliding_window=8, query_pre_attn_scalar=40))
    if name == "llama31_rope":  # Llama-3.1 rule: low rotary frequencies divided by 8, high ones kept, a ramp between
        rp = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
              "original_max_position_embeddings": 32, "rope_theta": 10000.0}
        return T.LlamaForCausalLM(T.LlamaConfig(**c, rope_parameters=rp))
    if name == "phi3_longrope":  # LongRoPE: per-frequency factors, the long set (and its magnitude factor) beyond 32 tokens
        rp = {"rope_type": "longrope", "short_factor": [1.0 + 0.05 * i for i in range(8)], "long_factor": [1.5 + 0.4 * i for i in range(8)],
              "original_max_position_embeddings": 32, "rope_theta": 10000.0, "factor": 8.0}
        return T.Phi3ForCausalLM(T.Phi3Config(**c, pad_token_id=0, original_max_position_embeddings=32, rope_parameters=rp))
    if name == "mistral_swa":  # every layer windowed (8 tokens): the engine also returns pages that fell out of the window
        return T.MistralForCausalLM(T.MistralConfig(**c, sliding_window=8))
    if name == "qwen2moe":  # routed experts without renormalised weights + a sigmoid-gated shared expert, q/k/v biases
        return T.Qwen2MoeForCausalLM(T.Qwen2MoeConfig(**c, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=48,
                                                      shared_expert_intermediate_size=80, norm_topk_prob=False,
                                                      decoder_sparse_step=1, mlp_only_layers=[]))
    if name == "mamba":  # selective state-space layers only: convolution window of 4, 8-wide state, no attention, no MLP
        return T.MambaForCausalLM(T.MambaConfig(vocab_size=VOCAB, hidden_size=64, state_size=8, num_hidden_layers=3, conv_kernel=4,
                                                expand=2, time_step_rank=8))
    if name == "lfm2":  # convolution layers (kernel of 3 taps) around two attention layers with RMSNorm on q / k heads
        return T.Lfm2ForCausalLM(T.Lfm2Config(**c, conv_L_cache=3, block_auto_adjust_ff_dim=False,
                                              layer_types=["conv", "conv", "full_attention", "conv"]))
    if name == "lfm2moe":  # one dense layer, then 8 routed experts: sigmoid scores, a bias that only steers the choice, weights * 1.5
        m = T.Lfm2MoeForCausalLM(T.Lfm2MoeConfig(**c, conv_L_cache=3, moe_intermediate_size=48, num_experts=8, num_experts_per_tok=2,
                                                 num_dense_layers=1, use_expert_bias=True, routed_scaling_factor=1.5,
                                                 layer_types=["conv", "full_attention", "conv", "full_attention"]))
        with torch.no_grad():
            for layer in m.model.layers[1:]:
                layer.feed_forward.expert_bias.copy_(torch.randn(8) * 0.3)
        return m
    if name == "hunyuan_moe":  # norms on the rotated q / k heads, softmax routing over 8 experts + an always-on shared MLP, NTK-stretched base
        return T.HunYuanMoEV1ForCausalLM(T.HunYuanMoEV1Config(**c, head_dim=16, num_experts=8, moe_topk=2,
                                                              rope_parameters={"rope_type": "dynamic", "rope_theta": 10000.0, "alpha": 50.0, "factor": 1.0}))
    if name == "hunyuan_dense":
        return T.HunYuanDenseV1ForCausalLM(T.HunYuanDenseV1Config(**c, head_dim=16))
    if name == "qwen35":  # three gated-delta-rule layers (4 value heads over 2 key heads, 4 taps) to one gated attention layer
        return T.Qwen3_5ForCausalLM(T.Qwen3_5TextConfig(**c, head_dim=16, linear_conv_kernel_dim=4, linear_key_head_dim=8,
                                                        linear_value_head_dim=12, linear_num_key_heads=2, linear_num_value_heads=4,
                                                        layer_types=["linear_attention", "linear_attention", "full_attention",
                                                                     "linear_attention"]))
    if name == "qwen35moe":  # the same mixers in front of routed experts + a sigmoid-gated shared expert
        return T.Qwen3_5MoeForCausalLM(T.Qwen3_5MoeTextConfig(**{k: v for k, v in c.items() if k != "intermediate_size"}, head_dim=16,
                                                              linear_conv_kernel_dim=4, linear_key_head_dim=8, linear_value_head_dim=8,
                                                              linear_num_key_heads=2, linear_num_value_heads=2, num_experts=8,
                                                              num_experts_per_tok=2, moe_intermediate_size=48, shared_expert_intermediate_size=80,
                                                              layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"]))
    if name == "minimax_m2":  # q and k normalised over all heads at once, half of each head rotated, sigmoid routing with a bias
        m = T.MiniMaxM2ForCausalLM(T.MiniMaxM2Config(**c, head_dim=16, num_local_experts=8, num_experts_per_tok=2,
                                                     rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5}))
        with torch.no_grad():
            for layer in m.model.layers:
                layer.mlp.e_score_correction_bias.copy_(torch.randn(8) * 0.3)
        return m
    if name == "glm4":  # norms on both sides of both branches, fused gate-up, neighbouring values rotated over half of each head
        return T.Glm4ForCausalLM(T.Glm4Config(**c, head_dim=16, pad_token_id=0, attention_bias=True,
                                              rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5}))
    if name == "glm4moe":  # half of each head rotated, q/k/v biases, norms on q / k heads, DeepSeek-V3 style routing after a dense layer
        m = T.Glm4MoeForCausalLM(T.Glm4MoeConfig(**c, moe_intermediate_size=48, n_routed_experts=8, n_shared_experts=1,
                                                 num_experts_per_tok=2, first_k_dense_replace=1, n_group=2, topk_group=1,
                                                 routed_scaling_factor=1.5, norm_topk_prob=True, use_qk_norm=True, attention_bias=True,
                                                 rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5}))
        with torch.no_grad():
            for layer in m.model.layers[1:]:
                layer.mlp.gate.e_score_correction_bias.copy_(torch.randn(8) * 0.3)
        return m
    # DeepSeek: latent attention (32-wide latent, 16 position-free + 8 rotary query / key values per head, 24-wide values),
    # one dense layer then routed experts + a shared expert
    ds = dict(c, moe_intermediate_size=48, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2, first_k_dense_replace=1,
              kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=24, num_key_value_heads=4)
    if name == "deepseek_v2":  # softmax scores, plain top-k, weights not renormalised, scaled by 1.5
        return T.DeepseekV2ForCausalLM(T.DeepseekV2Config(**ds, q_lora_rank=48, n_group=1, topk_group=1, routed_scaling_factor=1.5,
                                                          topk_method="greedy"))
    if name == "deepseek_v3":  # sigmoid scores, 2 of 4 expert groups, low-rank queries
        return T.DeepseekV3ForCausalLM(T.DeepseekV3Config(**ds, q_lora_rank=48, n_group=4, topk_group=2, routed_scaling_factor=2.5,
                                                          norm_topk_prob=True))
    if name == "deepseek_v3_yarn":  # full-rank queries, YaRN-scaled rotary part (its magnitude term goes into the softmax scale)
        yarn = {"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 32, "mscale": 1.0, "mscale_all_dim": 1.0,
                "beta_fast": 32.0, "beta_slow": 1.0, "rope_theta": 10000.0}
        return T.DeepseekV3ForCausalLM(T.DeepseekV3Config(**ds, q_lora_rank=None, n_group=2, topk_group=1, rope_parameters=yarn))
    raise KeyError(name)


FAMILIES = ["llama", "qwen2", "qwen3", "phi3", "mixtral", "qwen3moe", "gemma", "gemma2", "gemma3", "deepseek_v2", "deepseek_v3",
            "deepseek_v3_yarn", "lfm2", "lfm2moe", "glm4", "glm4moe", "hunyuan_moe", "hunyuan_dense", "qwen35", "qwen35moe", "minimax_m2", "mamba", "mistral_swa", "qwen2moe",
            "llama31_rope", "phi3_longrope"]


@pytest.mark.parametrize("family", FAMILIES)
def test_logits_and_greedy_tokens_match_transformers(family, tmp_path):
    try:
        torch.manual_seed(0)
        ref = _build(family).eval().float()
    except (AttributeError, TypeError, KeyError) as e:  # a transformers build without this family
        pytest.skip(f"transformers cannot build {family}: {e}")
    with torch.no_grad():
        for pname, p in ref.named_parameters():
            if "norm" in pname:
                p.add_(torch.randn_like(p) * 0.3)  # norms away from their initial value, so that they matter
            elif p.ndim == 2:
                p.mul_(3.0)  # larger weights: logits with more spread than the 0.02-std init gives
    src = str(tmp_path / "hf")
    ref.save_pretrained(src, safe_serialization=True)
    path = convert_safetensors_to_gguf(src, str(tmp_path / "m.gguf"), "F32")
    cfg = config_from_gguf(load_gguf(path))
    if family == "gemma2":
        assert cfg.attn_softcap == 50.0 and cfg.final_softcap == 30.0 and cfg.sliding_window_pattern == 2 and cfg.post_norms
        assert abs(cfg.attn_scale - 24 ** -0.5) < 1e-6
    if family.startswith("deepseek"):
        assert cfg.is_mla and (cfg.kv_lora_rank, cfg.qk_nope_dim, cfg.rope_dim, cfg.v_head_dim, cfg.head_dim) == (32, 16, 8, 24, 24)
        assert cfg.rope_pairing == "adjacent" and cfg.n_shared_experts == 1 and cfg.leading_dense_blocks == 1
        assert cfg.expert_gating == ("softmax" if family == "deepseek_v2" else "sigmoid")
    if family == "mistral_swa":
        assert cfg.sliding_window == 8 and cfg.sliding_window_pattern == 0
    if family == "qwen2moe":
        assert cfg.n_shared_experts == 1 and cfg.shared_expert_gate and cfg.shared_expert_ffn_size == 80 and cfg.attn_bias
        assert not cfg.expert_weights_norm
    if family == "mamba":
        assert cfg.is_ssm and (cfg.ssm_d_inner, cfg.ssm_d_state, cfg.ssm_d_conv, cfg.ssm_dt_rank) == (128, 8, 4, 8)
    if family == "lfm2":
        assert cfg.conv_layers == [0, 1, 3] and cfg.conv_l_cache == 3 and cfg.qk_norm and cfg.n_kv_heads == 2
    if family.startswith("hunyuan"):
        assert cfg.qk_norm and cfg.qk_norm_after_rope
    if family == "hunyuan_moe":
        assert cfg.n_experts == 8 and cfg.n_shared_experts == 1 and not cfg.shared_expert_gate and cfg.expert_gating == "softmax"
        assert abs(cfg.rope_theta - 10000.0 * 50.0 ** (16 / 14)) < 1.0
    if family == "qwen35moe":
        assert cfg.gdn_layers == [0, 2] and cfg.n_experts == 8 and cfg.n_shared_experts == 1 and cfg.shared_expert_gate
    if family == "qwen35":
        assert cfg.gdn_layers == [0, 1, 3] and cfg.attn_out_gate and cfg.qk_norm and cfg.rope_dim == 4 and cfg.is_ssm
        assert (cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_k_dim, cfg.gdn_v_dim, cfg.gdn_conv) == (2, 4, 8, 12, 4)
    if family == "minimax_m2":
        assert cfg.qk_norm and cfg.qk_norm_full and cfg.expert_gating == "sigmoid" and cfg.rope_dim == 8 and cfg.n_experts == 8
    if family == "glm4":
        assert cfg.rope_pairing == "adjacent" and cfg.rope_dim == 8 and cfg.post_norms and cfg.attn_bias
    if family == "glm4moe":
        assert cfg.rope_dim == 8 and cfg.qk_norm and cfg.attn_bias and cfg.expert_gating == "sigmoid" and cfg.expert_group_count == 2
        assert cfg.n_shared_experts == 1 and cfg.leading_dense_blocks == 1
    if family == "lfm2moe":
        assert cfg.conv_layers == [0, 2] and cfg.n_experts == 8 and cfg.leading_dense_blocks == 1 and cfg.expert_gating == "sigmoid"
        assert cfg.expert_weights_scale == 1.5 and cfg.expert_ffn_size == 48
    if family == "gemma3":
        assert cfg.sliding_window_pattern == 6 and cfg.rope_theta_swa == 10000.0 and cfg.rope_theta == 1000000.0
        assert cfg.qk_norm and cfg.post_norms and cfg.ffn_act == "gelu_tanh" and cfg.embedding_scale == 8.0
    # prefill in chunks of 16 rows: prompts longer than that cross chunk (and window) boundaries
    llm = LLM.from_gguf(path, EngineConfig(kv_cache_dtype="f32", max_model_len=128, max_num_seqs=2, num_kv_blocks=32,
                                           prefill_chunk_size=16, max_num_batched_tokens=16, enable_prefix_cache=False),
                        device="cpu")
    llm.runner.keep_logits = True
    gen = torch.Generator().manual_seed(1)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    # (LongRoPE switches factor sets with the sequence length in the oracle and with the serving context here: compare
    # where both use the long set)
    for n_prompt in ((40, 50, 60) if family == "phi3_longrope" else (5, 19, 40)):
        ids = torch.randint(3, VOCAB, (n_prompt,), generator=gen).tolist()
        with torch.no_grad():
            want = ref(torch.tensor([ids])).logits[0, -1]
            want_tokens = ref.generate(torch.tensor([ids]), attention_mask=torch.ones(1, n_prompt, dtype=torch.long),
                                       max_new_tokens=6, do_sample=False, pad_token_id=0)[0, n_prompt:].tolist()
        llm.add_request(ids, sp)
        first, tokens = None, None
        while llm.has_unfinished:
            outs = llm.step()
            lg = llm.last_step[1].logits if llm.last_step is not None else None
            if first is None and lg is not None and lg.shape[0] == 1:
                first = lg.float()[0].clone()  # the step that finished the prompt
            for o in outs:
                if o.finished:
                    tokens = o.token_ids
        err = (first - want).abs().max().item() / want.abs().max().item()
        assert err < 2e-5, f"{family}, {n_prompt}-token prompt: logits differ by {err:.2e} of their range"
        # (the oracle stops when it emits its end-of-sequence id; the engine was told to carry on)
        assert tokens[: len(want_tokens)] == want_tokens and want_tokens, f"{family}, {n_prompt}-token prompt: {tokens} != {want_tokens}"
    assert os.path.getsize(path) > 0


@pytest.mark.parametrize("family", ["mamba", "qwen35"])
def test_state_space_model_through_the_scheduler(family, tmp_path):
    """A per-sequence recurrent state (Mamba; Qwen3.5's gated-delta-rule layers beside attention layers) under continuous batching: batched == one at a time, a pool small enough to preempt ==
    a roomy one (a restarted sequence recomputes its state from position 0), more sequential requests than state slots,
    no prefix sharing, no speculation."""
    torch.manual_seed(1)
    ref = _build(family).eval().float()
    with torch.no_grad():
        for pname, p in ref.named_parameters():
            if p.ndim == 2:
                p.mul_(2.0)
    src = str(tmp_path / "hf")
    ref.save_pretrained(src, safe_serialization=True)
    path = convert_safetensors_to_gguf(src, str(tmp_path / "m.gguf"), "F32")
    ec = dict(kv_cache_dtype="f32", max_model_len=128, max_num_seqs=4, prefill_chunk_size=16, max_num_batched_tokens=32)
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, VOCAB, (n,), generator=gen).tolist() for n in (5, 33, 18, 50, 7, 26)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    roomy = LLM.from_gguf(path, EngineConfig(**ec, num_kv_blocks=64), device="cpu")
    assert not roomy.scheduler.config.enable_prefix_cache
    one_by_one = [roomy.generate([p], sp)[0].token_ids for p in prompts]
    assert [o.token_ids for o in roomy.generate(prompts, sp)] == one_by_one
    with torch.no_grad():
        want0 = ref.generate(torch.tensor([prompts[1]]), attention_mask=torch.ones(1, len(prompts[1]), dtype=torch.long),
                             max_new_tokens=12, do_sample=False, pad_token_id=0)[0, len(prompts[1]):].tolist()
    assert one_by_one[1] == want0
    # short prompts that grow: all four are admitted, then the pool runs dry and the scheduler evicts and recomputes
    growers = [p[:14] for p in prompts if len(p) >= 14]
    long_sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    want_long = [o.token_ids for o in roomy.generate(growers, long_sp)]
    small = LLM.from_gguf(path, EngineConfig(**ec, num_kv_blocks=10), device="cpu")
    assert [o.token_ids for o in small.generate(growers, long_sp)] == want_long and small.scheduler.num_preemptions > 0
    # the same prompt twice in a row: identical (nothing of the first run's state leaks into the second)
    again = [roomy.generate([prompts[3]], sp)[0].token_ids for _ in range(2)]
    assert again[0] == again[1] == one_by_one[3]
    # more requests over time than one block of state slots
    for i in range(20):
        assert roomy.generate([prompts[i % 6]], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))[0].token_ids \
            == one_by_one[i % 6][:2]
    assert roomy.model._ssm_state.shape[0] <= 32
    # calls that bring a cache of their own (embeddings, scoring) give their state slots back
    n_keys = len(roomy.model._ssm_slots)
    for _ in range(40):
        roomy.embed([prompts[0]])
    lp = roomy.token_logprobs(prompts[1] + one_by_one[1], chunk=16)
    assert len(roomy.model._ssm_slots) == n_keys and roomy.model._ssm_state.shape[0] <= 32
    with torch.no_grad():
        full = torch.tensor([prompts[1] + one_by_one[1]])
        ref_lp = torch.log_softmax(ref(full).logits[0, :-1].double(), -1).gather(1, full[0, 1:, None])[:, 0]
    assert torch.allclose(torch.from_numpy(lp), ref_lp, atol=1e-4)
    from oxidize_b200.engine.spec import attach_speculation

    with pytest.raises(ValueError):
        attach_speculation(roomy, path, k=2)
