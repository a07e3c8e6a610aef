"""Model hyper-parameters read from GGUF metadata.

Mirrors ``InferenceConfig::from_gguf`` (``oxidize-core/src/model/inference.rs:363-697``): every
value comes from ``{arch}.*`` metadata with tensor-shape fallbacks, ``attention.key_length``
wins over ``hidden/heads`` (``:490-495``), the vocabulary axis of ``token_embd`` is the larger
one (``:425-428``), and the architecture string selects routing / norm conventions
(``:62-96``).  Named presets for the benchmark shapes live in :func:`preset`.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..formats.gguf import GGUFFile

# architecture strings accepted (reference arch-string map inference.rs:62-96)
# phi3: Llama layers with fused qkv / gate-up tensors.  gemma / gemma2 / gemma3: GeGLU, scaled embeddings, norms on the
# branch outputs, soft-capped logits, interleaved local / global attention with two rotary bases.
# lfm2 / lfm2moe: short-convolution mixers interleaved with grouped-query attention layers (lfm2moe: routed experts
# after the leading dense layers, sigmoid scores, a per-expert bias used for the choice only).
# glm4: Llama layers with norms on both branch outputs too, a fused gate-up tensor, and half of each head rotated over
# pairs of neighbouring values.
# hunyuan-dense / hunyuan-moe: RMSNorm on the q / k heads AFTER the rotation; the MoE form adds an always-on shared MLP.
# minimax-m2: q and k normalised over the whole projection (all heads at once) before the rotation, sigmoid routing with a
# correction bias.
# glm4moe: grouped-query attention over half-rotated heads, DeepSeek-V3 style routing (sigmoid scores, correction bias, groups).
# qwen35: three gated-delta-rule layers (linear attention with a per-sequence matrix state) to every attention layer, whose
# output passes a sigmoid gate computed beside the queries; norm weights stored as w - 1.
# mamba: selective state-space layers only (no attention, no feed-forward block).
DENSE_ARCHS = {"llama", "mistral", "qwen2", "qwen3", "deepseek", "phi3", "gemma", "gemma2", "gemma3", "lfm2", "mamba", "glm4",
               "qwen35", "qwen3_5", "qwen3_5_text", "qwen35_text",
               "hunyuan-dense", "hunyuan_dense"}
GEMMA_ARCHS = {"gemma", "gemma2", "gemma3"}
MOE_ARCHS = {"mixtral", "qwen2moe", "qwen3moe", "deepseek2", "deepseek-moe", "deepseek_moe", "lfm2moe", "glm4moe", "minimax-m2", "minimax_m2", "minimax", "qwen35moe", "qwen3_5_moe", "qwen3_5_moe_text",
             "hunyuan-moe", "hunyuan_moe"}
# Architectures whose layers need math this engine does not have (two attention geometries in one model,
# parallel attention / MLP blocks, recurrent or convolutional mixers): loading one would run it as
# a plain Llama and produce wrong tokens, so they are refused by name.
QWEN35_ARCHS = {"qwen35", "qwen3_5", "qwen3_5_text", "qwen35_text", "qwen35moe", "qwen3_5_moe", "qwen3_5_moe_text"}
UNSUPPORTED_ARCHS = {"gemma4", "phi", "phi2", "llama4", "mamba2", "jamba",
                     "falcon", "gpt2", "bert"}


class UnsupportedArchitecture(ValueError):
    pass


def check_architecture(arch: str) -> None:
    if arch in DENSE_ARCHS or arch in MOE_ARCHS:
        return
    if arch in UNSUPPORTED_ARCHS:
        raise UnsupportedArchitecture(f"architecture {arch!r} needs layer semantics this engine does not implement")
    raise UnsupportedArchitecture(f"unknown architecture {arch!r}; supported: {sorted(DENSE_ARCHS | MOE_ARCHS)}")


@dataclass
class RopeScaling:
    type: str = "none"  # none | linear | yarn
    factor: float = 1.0
    original_context_length: int = 0
    beta_fast: float = 32.0
    beta_slow: float = 1.0


@dataclass
class ModelConfig:
    arch: str = "llama"
    name: str = ""
    vocab_size: int = 32000
    hidden_size: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn_size: int = 14336
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_dim: int = 0  # 0 -> head_dim (full rotary)
    # Gated-delta-rule layers (Qwen3.5; the reference's run_mamba_layer, model/layer_wise/ssm.rs:82): which layers, key /
    # value head counts and widths, taps of the causal convolution in front of q / k / v
    gdn_layers: List[int] = field(default_factory=list)
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    gdn_k_dim: int = 0
    gdn_v_dim: int = 0
    gdn_conv: int = 4
    attn_out_gate: bool = False  # q_proj also yields a per-head gate; attention output * sigmoid(gate)
    qk_norm_full: bool = False  # MiniMax-M2: one RMSNorm over all of q (and of k), not one per head
    qk_norm_after_rope: bool = False  # Hunyuan: the per-head q / k norms act on the rotated vectors
    rope_pairing: str = "split_half"  # split_half (NeoX; what all reference engines do) | adjacent
    rope_attn_factor: float = 1.0  # magnitude factor that goes with the long LongRoPE frequency factors (Phi-3)
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    context_length: int = 8192
    sliding_window: int = 0
    # 0: a configured window applies to every layer (Mistral / Qwen style).  n > 0: every n-th layer attends over the
    # whole context and the others use the window (interleaved local / global attention; the reference's
    # ``layer_is_global``, oxidize-core/src/model/inference.rs:304-333).
    sliding_window_pattern: int = 0
    qk_norm: bool = False
    attn_bias: bool = False
    tie_embeddings: bool = False
    # Gemma-family layer semantics (the reference's ``embedding_scale`` / ``gelu_ffn`` / ``sandwich_norm`` /
    # ``rope_theta_swa``, oxidize-core/src/model/inference.rs:604-636)
    embedding_scale: float = 1.0  # the embedding rows are multiplied by this (Gemma: sqrt(hidden_size))
    ffn_act: str = "silu"  # silu (SwiGLU) | gelu_tanh (GeGLU)
    post_norms: bool = False  # RMSNorm on the attention and FFN branch outputs before they join the residual stream
    attn_softcap: float = 0.0  # scores = cap * tanh(scores / cap) before the softmax (Gemma-2); 0 = off
    final_softcap: float = 0.0  # the same on the output logits
    rope_theta_swa: float = 0.0  # rotary base of the windowed layers (Gemma-3: 10000, unscaled); 0 = same as rope_theta
    attn_scale: float = 0.0  # softmax scale; 0 = head_dim ** -0.5
    # Multi-head latent attention (DeepSeek-V2/V3; the reference's ``deepseek_mla_layer``,
    # oxidize-core/src/model/inference/layers.rs:1547).  head_dim is the query / key width per head
    # (qk_nope_dim + rope_dim); keys and values are rebuilt from one shared latent of kv_lora_rank values per token.
    kv_lora_rank: int = 0  # > 0: the attention layers are latent-attention layers
    q_lora_rank: int = 0  # 0: one full query projection; > 0: down-projection, norm, up-projection
    qk_nope_dim: int = 0  # part of every query / key head that carries no position
    v_head_dim: int = 0  # value width per head
    yarn_log_multiplier: float = 0.0  # YaRN: the scores are scaled by (1 + this * ln(factor)) ** 2
    # Short-convolution mixer layers (LFM2; the reference's short-conv layer, model/inference/layers.rs:313): in those
    # layers a gated depthwise causal convolution over the last conv_l_cache positions takes the place of attention.
    conv_layers: List[int] = field(default_factory=list)  # indices of the convolution layers
    conv_l_cache: int = 0  # kernel length
    # Selective state-space layers (Mamba; the reference's SSM layer, model/inference/layers.rs:377): every layer is
    # norm -> mixer -> residual; the mixer keeps a convolution window and a [d_inner, d_state] state per sequence.
    ssm_d_inner: int = 0  # > 0: the layers are state-space layers
    ssm_d_state: int = 0
    ssm_d_conv: int = 0
    ssm_dt_rank: int = 0
    # MoE
    n_experts: int = 0
    n_experts_used: int = 0
    expert_ffn_size: int = 0
    expert_gating: str = "softmax"  # softmax | sigmoid
    expert_weights_scale: float = 1.0
    expert_weights_norm: bool = True
    expert_group_count: int = 0
    expert_group_used_count: int = 0
    leading_dense_blocks: int = 0
    n_shared_experts: int = 0
    shared_expert_ffn_size: int = 0
    shared_expert_gate: bool = False
    router_bias: bool = False
    # multi-token prediction (in-GGUF nextn layers appended after the decoder stack)
    nextn_layers: int = 0

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def is_ssm(self) -> bool:
        return self.ssm_d_inner > 0 or bool(self.gdn_layers)

    @property
    def rotary_dim(self) -> int:
        return self.rope_dim or self.head_dim

    @property
    def q_size(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.n_kv_heads * self.head_dim

    def layer_sliding_window(self, layer: int) -> int:
        """Attention window of one layer: 0 = the whole context."""
        if self.sliding_window <= 0:
            return 0
        if self.sliding_window_pattern > 0 and (layer + 1) % self.sliding_window_pattern == 0:
            return 0
        return self.sliding_window

    def layer_is_moe(self, layer: int) -> bool:
        return self.is_moe and layer >= self.leading_dense_blocks

    def param_count(self) -> int:
        h = self.hidden_size
        attn = h * self.q_size * 2 + h * self.kv_size * 2
        dense = 3 * h * self.ffn_size
        n = 0
        for i in range(self.n_layers):
            n += attn + 2 * h
            if self.layer_is_moe(i):
                n += self.n_experts * 3 * h * self.expert_ffn_size + h * self.n_experts
                n += self.n_shared_experts * 3 * h * (self.shared_expert_ffn_size or self.expert_ffn_size)
            else:
                n += dense
        n += self.vocab_size * h * (1 if self.tie_embeddings else 2) + h
        return n

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


def _scalar(v, default):
    if v is None:
        return default
    if isinstance(v, (list, tuple)):
        return v[0] if v else default
    return v


def config_from_gguf(g: GGUFFile) -> ModelConfig:
    arch = g.architecture
    check_architecture(arch)
    a = g.arch_get
    c = ModelConfig(arch=arch, name=str(g.get("general.name", "")))
    emb = g.tensors.get("token_embd.weight")
    c.hidden_size = int(_scalar(a("embedding_length"), emb.dims[0] if emb else c.hidden_size))
    if emb is not None:
        rows = emb.n_elements // emb.dims[0]
        # vocab axis is "the larger one"
        c.vocab_size = max(rows, emb.dims[0]) if rows != emb.dims[0] and emb.dims[0] == c.hidden_size else rows
    c.vocab_size = int(_scalar(a("vocab_size"), c.vocab_size))
    toks = g.get("tokenizer.ggml.tokens")
    if a("vocab_size") is None and emb is None and toks:
        c.vocab_size = len(toks)
    c.n_layers = int(_scalar(a("block_count"), c.n_layers))
    if arch == "mamba":
        c.ssm_d_inner = int(_scalar(a("ssm.inner_size"), g.tensors["blk.0.ssm_in.weight"].shape[0] // 2))
        c.ssm_d_state = int(_scalar(a("ssm.state_size"), g.tensors["blk.0.ssm_a"].shape[-1]))
        c.ssm_d_conv = int(_scalar(a("ssm.conv_kernel"), g.tensors["blk.0.ssm_conv1d.weight"].shape[-1]))
        c.ssm_dt_rank = int(_scalar(a("ssm.time_step_rank"), g.tensors["blk.0.ssm_dt.weight"].shape[-1]))
        c.rms_eps = float(_scalar(a("attention.layer_norm_rms_epsilon"), 1e-5))
        c.context_length = int(_scalar(a("context_length"), 1 << 20))
        c.n_heads = c.n_kv_heads = 1
        c.head_dim = 32  # no attention: only sizes a token cache that is never written
        c.ffn_size = 0
        c.tie_embeddings = not g.has_tensor("output.weight")
        return c
    c.nextn_layers = int(_scalar(a("nextn_predict_layers"), 0))
    c.n_heads = int(_scalar(a("attention.head_count"), c.n_heads))
    kvh = a("attention.head_count_kv")
    if isinstance(kvh, (list, tuple)):
        nz = [int(x) for x in kvh if int(x) > 0]
        kvh = nz[0] if nz else c.n_heads
    c.n_kv_heads = int(kvh if kvh is not None else c.n_heads)
    key_len = a("attention.key_length")
    c.head_dim = int(key_len) if key_len else c.hidden_size // c.n_heads
    ffn = a("feed_forward_length")
    if isinstance(ffn, (list, tuple)):
        nz = [int(x) for x in ffn if int(x) > 0]
        ffn = nz[0] if nz else None
    if ffn is None:
        t = g.tensors.get("blk.0.ffn_gate.weight") or g.tensors.get("blk.0.ffn_up.weight")
        ffn = t.shape[0] if t is not None else 0
    c.ffn_size = int(ffn)
    c.rms_eps = float(_scalar(a("attention.layer_norm_rms_epsilon"), 1e-5))
    c.rope_theta = float(_scalar(a("rope.freq_base"), 10000.0))
    c.rope_dim = int(_scalar(a("rope.dimension_count"), 0))
    if c.rope_dim >= c.head_dim:
        c.rope_dim = 0
    stype = a("rope.scaling.type")
    if stype:
        c.rope_scaling = RopeScaling(
            type=str(stype),
            factor=float(_scalar(a("rope.scaling.factor"), 1.0)),
            original_context_length=int(_scalar(a("rope.scaling.original_context_length"), 0)),
        )
    elif a("rope.scaling.original_context_length"):
        # LongRoPE files: no scaling rule, only the context length up to which the short frequency factors apply
        c.rope_scaling = RopeScaling(original_context_length=int(_scalar(a("rope.scaling.original_context_length"), 0)))
    c.context_length = int(_scalar(a("context_length"), 8192))
    c.sliding_window = int(_scalar(a("attention.sliding_window"), 0))
    c.sliding_window_pattern = int(_scalar(a("attention.sliding_window_pattern"), 0))
    c.qk_norm = g.has_tensor("blk.0.attn_q_norm.weight")
    c.attn_bias = g.has_tensor("blk.0.attn_q.bias") or g.has_tensor("blk.0.attn_qkv.bias")
    c.rope_attn_factor = float(_scalar(a("rope.scaling.attn_factor"), 1.0))
    c.tie_embeddings = not g.has_tensor("output.weight")
    if g.has_tensor("blk.0.attn_kv_a_mqa.weight"):
        # latent attention.  Two metadata conventions exist: key_length / value_length are the per-head widths
        # (nope + rope, v) and head_count_kv = heads; or they describe the cached latent (kv_lora + rope, kv_lora) with one
        # KV head, and key_length_mla / value_length_mla carry the per-head widths.
        c.kv_lora_rank = int(_scalar(a("attention.kv_lora_rank"), g.tensors["blk.0.attn_kv_a_norm.weight"].shape[-1]))
        c.q_lora_rank = int(_scalar(a("attention.q_lora_rank"), 0)) if g.has_tensor("blk.0.attn_q_a.weight") else 0
        rope = int(_scalar(a("rope.dimension_count"), 0)) or g.tensors["blk.0.attn_kv_a_mqa.weight"].shape[0] - c.kv_lora_rank
        qk = int(_scalar(a("attention.key_length_mla"), 0)) or int(key_len or 0)
        vd = int(_scalar(a("attention.value_length_mla"), 0)) or int(_scalar(a("attention.value_length"), 0))
        if g.has_tensor("blk.0.attn_kv_b.weight") and (qk <= rope or vd <= 0):
            per_head = g.tensors["blk.0.attn_kv_b.weight"].shape[0] // c.n_heads  # nope + v, equal in all released models
            qk, vd = qk if qk > rope else per_head // 2 + rope, vd or per_head // 2
        c.head_dim, c.rope_dim, c.qk_nope_dim, c.v_head_dim = qk, rope, qk - rope, vd
        c.n_kv_heads = c.n_heads
        c.rope_pairing = "adjacent"  # the rotary part is stored with interleaved pairs and files keep that order
        c.yarn_log_multiplier = float(_scalar(a("rope.scaling.yarn_log_multiplier"), 0.0))
    if arch in ("lfm2", "lfm2moe"):
        c.conv_l_cache = int(_scalar(a("shortconv.l_cache"), 3))
        c.conv_layers = [i for i in range(c.n_layers) if g.has_tensor(f"blk.{i}.shortconv.conv.weight")]
        first_attn = next((i for i in range(c.n_layers) if i not in c.conv_layers), 0)
        c.qk_norm = g.has_tensor(f"blk.{first_attn}.attn_q_norm.weight")
        c.tie_embeddings = not g.has_tensor("output.weight")
    qn = g.tensors.get("blk.0.attn_q_norm.weight")
    c.qk_norm_full = qn is not None and qn.n_elements > c.head_dim
    if arch in QWEN35_ARCHS:
        c.gdn_layers = [i for i in range(c.n_layers) if g.has_tensor(f"blk.{i}.ssm_alpha.weight")]
        c.attn_out_gate = True
        attn = next((i for i in range(c.n_layers) if i not in c.gdn_layers), None)
        if attn is not None:
            c.qk_norm = g.has_tensor(f"blk.{attn}.attn_q_norm.weight")
        if c.gdn_layers:
            i0 = c.gdn_layers[0]
            c.gdn_conv = int(_scalar(a("ssm.conv_kernel"), g.tensors[f"blk.{i0}.ssm_conv1d.weight"].shape[-1]))
            c.gdn_v_heads = int(_scalar(a("ssm.time_step_rank"), g.tensors[f"blk.{i0}.ssm_a"].n_elements))
            inner = int(_scalar(a("ssm.inner_size"), g.tensors[f"blk.{i0}.attn_gate.weight"].shape[0]))
            c.gdn_v_dim = inner // c.gdn_v_heads
            c.gdn_k_dim = int(_scalar(a("ssm.state_size"), c.gdn_v_dim))
            kdim = (g.tensors[f"blk.{i0}.attn_qkv.weight"].shape[0] - inner) // 2
            c.gdn_k_heads = int(_scalar(a("ssm.group_count"), kdim // c.gdn_k_dim))
    if arch.startswith("hunyuan"):
        c.qk_norm_after_rope = c.qk_norm
    if arch == "glm4":
        c.rope_pairing = "adjacent"
        c.post_norms = g.has_tensor("blk.0.post_attention_norm.weight")
    if arch in GEMMA_ARCHS:
        c.embedding_scale = float(c.hidden_size) ** 0.5
        c.ffn_act = "gelu_tanh"
        c.post_norms = g.has_tensor("blk.0.post_attention_norm.weight")
        if arch == "gemma2":
            # llama.cpp's defaults when a Gemma-2 file does not carry the keys
            c.attn_softcap = float(_scalar(a("attn_logit_softcapping"), 50.0))
            c.final_softcap = float(_scalar(a("final_logit_softcapping"), 30.0))
        if c.sliding_window > 0 and c.sliding_window_pattern <= 0:
            c.sliding_window_pattern = 2 if arch == "gemma2" else 6 if arch == "gemma3" else 0
        if arch == "gemma3":
            c.rope_theta_swa = float(_scalar(a("rope.freq_base_swa"), 10000.0))
        scale = a("attention.scale")
        if scale is not None and float(scale) > 0:
            c.attn_scale = float(scale)
        elif (arch, c.n_layers) in (("gemma2", 46), ("gemma3", 62)):
            # the 27B models scale the scores by (hidden_size / heads) ** -0.5 instead of head_dim ** -0.5; the file
            # format has no key for it, llama.cpp keys it on the model size as well
            c.attn_scale = float(c.hidden_size // c.n_heads) ** -0.5
    # MoE
    c.n_experts = int(_scalar(a("expert_count"), 0))
    c.n_experts_used = int(_scalar(a("expert_used_count"), 0))
    c.leading_dense_blocks = int(_scalar(a("leading_dense_block_count"), 0))
    if c.n_experts:
        eff = a("expert_feed_forward_length")
        if eff is None:
            for i in range(c.n_layers):
                t = g.tensors.get(f"blk.{i}.ffn_gate_exps.weight")
                if t is not None:
                    eff = t.shape[-2]
                    break
        c.expert_ffn_size = int(eff or c.ffn_size)
        gating = int(_scalar(a("expert_gating_func"), 1))
        c.expert_gating = "sigmoid" if gating == 2 else "softmax"
        c.expert_weights_scale = float(_scalar(a("expert_weights_scale"), 1.0)) or 1.0
        c.expert_weights_norm = bool(_scalar(a("expert_weights_norm"), True))
        c.expert_group_count = int(_scalar(a("expert_group_count"), 0))
        c.expert_group_used_count = int(_scalar(a("expert_group_used_count"), 0))
        for i in range(c.n_layers):
            t = g.tensors.get(f"blk.{i}.ffn_gate_shexp.weight")
            if t is not None:
                c.shared_expert_ffn_size = int(t.shape[0])
                c.n_shared_experts = max(1, int(_scalar(a("expert_shared_count"), 1)))
                c.shared_expert_gate = g.has_tensor(f"blk.{i}.ffn_gate_inp_shexp.weight")
                c.router_bias = g.has_tensor(f"blk.{i}.exp_probs_b.bias")
                break
    return c


_PRESETS: Dict[str, Dict[str, Any]] = {
    # CPU tiny Llama: 512 d, 8 L, 8/2 heads (hd 64), FFN 1408, vocab 32000
    "tiny-llama": dict(arch="llama", vocab_size=32000, hidden_size=512, n_layers=8, n_heads=8, n_kv_heads=2,
                       head_dim=64, ffn_size=1408, rms_eps=1e-5, rope_theta=10000.0, context_length=2048),
    "llama3-8b": dict(arch="llama", vocab_size=128256, hidden_size=4096, n_layers=32, n_heads=32, n_kv_heads=8,
                      head_dim=128, ffn_size=14336, rope_theta=500000.0, context_length=8192),
    "llama3-70b": dict(arch="llama", vocab_size=128256, hidden_size=8192, n_layers=80, n_heads=64, n_kv_heads=8,
                       head_dim=128, ffn_size=28672, rope_theta=500000.0, context_length=8192),
    "mixtral-8x7b": dict(arch="mixtral", vocab_size=32000, hidden_size=4096, n_layers=32, n_heads=32, n_kv_heads=8,
                         head_dim=128, ffn_size=14336, rope_theta=1000000.0, context_length=32768,
                         n_experts=8, n_experts_used=2, expert_ffn_size=14336),
    "qwen3-30b-a3b": dict(arch="qwen3moe", vocab_size=151936, hidden_size=2048, n_layers=48, n_heads=32, n_kv_heads=4,
                          head_dim=128, ffn_size=6144, rope_theta=1000000.0, context_length=32768, qk_norm=True,
                          n_experts=128, n_experts_used=8, expert_ffn_size=768),
    # Gemma-3-27B: 5 windowed layers (1024 tokens, rotary base 1e4) to every global one (base 1e6, positions / 8)
    "gemma3-27b": dict(arch="gemma3", vocab_size=262208, hidden_size=5376, n_layers=62, n_heads=32, n_kv_heads=16,
                       head_dim=128, ffn_size=21504, rms_eps=1e-6, rope_theta=1000000.0, rope_theta_swa=10000.0,
                       rope_scaling=RopeScaling(type="linear", factor=8.0), context_length=131072, sliding_window=1024,
                       sliding_window_pattern=6, qk_norm=True, post_norms=True, ffn_act="gelu_tanh",
                       embedding_scale=5376 ** 0.5, attn_scale=168 ** -0.5, tie_embeddings=True),
    # DeepSeek-V3: latent attention (512-wide latent + 64 rotary values cached per token), 3 dense layers, then 256 routed
    # experts (8 of them per token, out of 4 of 8 groups) and a shared expert
    "deepseek-v3": dict(arch="deepseek2", vocab_size=129280, hidden_size=7168, n_layers=61, n_heads=128, n_kv_heads=128,
                        head_dim=192, rope_dim=64, qk_nope_dim=128, v_head_dim=128, kv_lora_rank=512, q_lora_rank=1536,
                        ffn_size=18432, rms_eps=1e-6, rope_theta=10000.0, rope_pairing="adjacent", context_length=163840,
                        rope_scaling=RopeScaling(type="yarn", factor=40.0, original_context_length=4096),
                        yarn_log_multiplier=0.1, n_experts=256, n_experts_used=8, expert_ffn_size=2048,
                        expert_gating="sigmoid", expert_weights_scale=2.5, expert_group_count=8, expert_group_used_count=4,
                        leading_dense_blocks=3, n_shared_experts=1, shared_expert_ffn_size=2048, router_bias=True),
    "qwen-draft-0.5b": dict(arch="qwen2", vocab_size=151936, hidden_size=896, n_layers=24, n_heads=14, n_kv_heads=2,
                            head_dim=64, ffn_size=4864, rope_theta=1000000.0, context_length=32768,
                            tie_embeddings=True),
}


def preset(name: str, **overrides) -> ModelConfig:
    if name not in _PRESETS:
        raise KeyError(f"unknown preset {name!r}; have {sorted(_PRESETS)}")
    kw = dict(_PRESETS[name])
    kw.update(overrides)
    return ModelConfig(name=name, **kw)


def preset_names() -> List[str]:
    return sorted(_PRESETS)
