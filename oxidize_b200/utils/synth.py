"""Random-init models of a named shape: GGUF files for small shapes, direct device weights
for the large benchmark shapes.

There is no network for checkpoints, so every benchmark runs on N(0, 0.02) weights of the
architecture named in the config.  Files carry a trivial ``gpt2``-style vocabulary because the
reference's C engine refuses to run a GGUF without tokenizer metadata
(``oxidize-c/src/cli/commands.c:709-715``).
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ..formats.gguf import GGUFValueType, GGUFWriter, ggml_type
from ..models.config import ModelConfig
from ..models.weights import (ExpertWeights, LayerWeights, LinearWeight, ModelWeights, QTensor, shard_range)
from ..quant import ref as qref

WEIGHT_STD = 0.02


def q4_k_m_type(name: str, layer: int, n_layers: int) -> str:
    """llama.cpp-style Q4_K_M mix: Q6_K for the output head, and for attn_v / ffn_down in the
    first and last eighth of the layers and every third layer in between; Q4_K elsewhere."""
    if name == "output":
        return "Q6_K"
    if name in ("attn_v", "ffn_down"):
        more = layer < n_layers // 8 or layer >= 7 * n_layers // 8 or (layer - n_layers // 8) % 3 == 2
        return "Q6_K" if more else "Q4_K"
    return "Q4_K"


def pick_type(policy: str, name: str, layer: int, n_layers: int, in_features: int) -> str:
    policy = policy.upper()
    t = q4_k_m_type(name, layer, n_layers) if policy == "Q4_K_M" else policy
    if t in ("F32", "F16", "BF16"):
        return t
    bs = ggml_type(t).block_size
    if in_features % bs:
        # k-quants need whole 256-value super-blocks per row; fall back to a 32-block type
        # the way llama.cpp-style quantizers do (e.g. FFN 1408 = 5.5 × 256 → Q8_0).
        for alt in ("Q8_0",):
            if in_features % ggml_type(alt).block_size == 0:
                return alt
        return "F16"
    return t


def minimal_vocab(n: int):
    base = [f"<{i}>" for i in range(n)]
    base[0] = "<unk>"
    if n > 1:
        base[1] = "<s>"
    if n > 2:
        base[2] = "</s>"
    # printable single-byte pieces so that text round-trips through the byte-level BPE
    from ..formats.tokenizer import gpt2_byte_table

    b2u = gpt2_byte_table()
    j = 3
    for b in range(256):
        if j >= n:
            break
        base[j] = b2u[b]
        j += 1
    return base


def add_minimal_tokenizer(w: GGUFWriter, vocab_size: int) -> None:
    toks = minimal_vocab(vocab_size)
    w.add("tokenizer.ggml.model", "gpt2")
    w.add("tokenizer.ggml.tokens", toks, GGUFValueType.ARRAY, GGUFValueType.STRING)
    types = [1] * vocab_size
    for i in range(min(3, vocab_size)):
        types[i] = 3
    w.add("tokenizer.ggml.token_type", types, GGUFValueType.ARRAY, GGUFValueType.INT32)
    w.add("tokenizer.ggml.merges", [], GGUFValueType.ARRAY, GGUFValueType.STRING)
    w.add("tokenizer.ggml.unknown_token_id", 0, GGUFValueType.UINT32)
    w.add("tokenizer.ggml.bos_token_id", min(1, vocab_size - 1), GGUFValueType.UINT32)
    w.add("tokenizer.ggml.eos_token_id", min(2, vocab_size - 1), GGUFValueType.UINT32)
    w.add("tokenizer.ggml.add_bos_token", False)


def write_config_metadata(w: GGUFWriter, cfg: ModelConfig) -> None:
    a = cfg.arch
    U = GGUFValueType.UINT32
    w.add("general.name", cfg.name or "synthetic")
    w.add(f"{a}.vocab_size", cfg.vocab_size, U)
    w.add(f"{a}.embedding_length", cfg.hidden_size, U)
    w.add(f"{a}.block_count", cfg.n_layers, U)
    w.add(f"{a}.context_length", cfg.context_length, U)
    w.add(f"{a}.feed_forward_length", cfg.ffn_size, U)
    w.add(f"{a}.attention.head_count", cfg.n_heads, U)
    w.add(f"{a}.attention.head_count_kv", cfg.n_kv_heads, U)
    w.add(f"{a}.attention.key_length", cfg.head_dim, U)
    w.add(f"{a}.attention.value_length", cfg.v_head_dim if cfg.is_mla else cfg.head_dim, U)
    if cfg.is_mla:
        w.add(f"{a}.attention.kv_lora_rank", cfg.kv_lora_rank, U)
        if cfg.q_lora_rank:
            w.add(f"{a}.attention.q_lora_rank", cfg.q_lora_rank, U)
        if cfg.yarn_log_multiplier:
            w.add(f"{a}.rope.scaling.yarn_log_multiplier", float(cfg.yarn_log_multiplier), GGUFValueType.FLOAT32)
    w.add(f"{a}.attention.layer_norm_rms_epsilon", float(cfg.rms_eps), GGUFValueType.FLOAT32)
    w.add(f"{a}.rope.freq_base", float(cfg.rope_theta), GGUFValueType.FLOAT32)
    w.add(f"{a}.rope.dimension_count", cfg.rotary_dim, U)
    if cfg.sliding_window:
        w.add(f"{a}.attention.sliding_window", cfg.sliding_window, U)
        if cfg.sliding_window_pattern:
            w.add(f"{a}.attention.sliding_window_pattern", cfg.sliding_window_pattern, U)
    F = GGUFValueType.FLOAT32
    if cfg.rope_theta_swa > 0:
        w.add(f"{a}.rope.freq_base_swa", float(cfg.rope_theta_swa), F)
    if cfg.attn_scale > 0:
        w.add(f"{a}.attention.scale", float(cfg.attn_scale), F)
    if a == "gemma2":
        w.add(f"{a}.attn_logit_softcapping", float(cfg.attn_softcap), F)
        w.add(f"{a}.final_logit_softcapping", float(cfg.final_softcap), F)
    if cfg.rope_scaling.type != "none":
        w.add(f"{a}.rope.scaling.type", cfg.rope_scaling.type)
        w.add(f"{a}.rope.scaling.factor", float(cfg.rope_scaling.factor), GGUFValueType.FLOAT32)
        w.add(f"{a}.rope.scaling.original_context_length", cfg.rope_scaling.original_context_length, U)
    if cfg.n_experts:
        w.add(f"{a}.expert_count", cfg.n_experts, U)
        w.add(f"{a}.expert_used_count", cfg.n_experts_used, U)
        w.add(f"{a}.expert_feed_forward_length", cfg.expert_ffn_size, U)
        w.add(f"{a}.expert_gating_func", 2 if cfg.expert_gating == "sigmoid" else 1, U)
        w.add(f"{a}.expert_weights_scale", float(cfg.expert_weights_scale), GGUFValueType.FLOAT32)
        w.add(f"{a}.expert_weights_norm", bool(cfg.expert_weights_norm))
        if cfg.expert_group_count:
            w.add(f"{a}.expert_group_count", cfg.expert_group_count, U)
            w.add(f"{a}.expert_group_used_count", cfg.expert_group_used_count, U)
        if cfg.leading_dense_blocks:
            w.add(f"{a}.leading_dense_block_count", cfg.leading_dense_blocks, U)
    if cfg.nextn_layers:
        w.add(f"{a}.nextn_predict_layers", cfg.nextn_layers, U)


def synth_gguf(path: str, cfg: ModelConfig, quant: str = "Q4_K_M", seed: int = 0, tokenizer: bool = True,
               norm_jitter: float = 0.0, device=None, embed_type: Optional[str] = None, fused_layout: bool = False,
               rope_freqs: Optional[np.ndarray] = None) -> str:
    """Write a random-init GGUF of shape ``cfg``; matrices N(0, 0.02) encoded per ``quant``
    (``Q4_K_M`` = llama.cpp-style Q4_K/Q6_K mix), norms f32 ones.

    With ``device`` (a CUDA device) the matrices are drawn and block-encoded there with the torch
    encoders and only the packed bytes cross to the host, which turns the minutes a NumPy encode of a
    multi-billion-parameter shape takes into the time of the file write.  ``embed_type`` stores the
    token-embedding table in another type than ``quant`` picks (the reference's CUDA backend has no row
    lookup for a bf16 / f16 table: ``oxidize-c/src/backends/cuda.cu`` ``cuda_embed`` hands every "packed"
    table to ``oc_cuda_mmq_get_row``, which knows the block-quantized types only).  ``fused_layout`` writes the
    Phi-3 tensor layout (one ``attn_qkv`` and one gate-then-up ``ffn_up`` tensor per layer) with the SAME values a
    plain file of the same seed holds; ``rope_freqs`` adds a ``rope_freqs.weight`` tensor of per-pair divisors."""
    rng = np.random.default_rng(seed)
    dev = torch.device(device) if device is not None else None
    tgen = None
    if dev is not None:
        tgen = torch.Generator(device=dev)
        tgen.manual_seed(seed)
    w = GGUFWriter(path, arch=cfg.arch)
    write_config_metadata(w, cfg)
    if tokenizer:
        add_minimal_tokenizer(w, cfg.vocab_size)
    h, hd = cfg.hidden_size, cfg.head_dim
    L = cfg.n_layers

    def mat(gname: str, kind: str, layer: int, out_f: int, in_f: int, n_exp: int = 0, add: bool = True):
        t = pick_type(quant, kind, layer, L, in_f)
        if kind == "token_embd" and embed_type:
            t = embed_type.upper()
        shape = (n_exp, out_f, in_f) if n_exp else (out_f, in_f)
        n = int(np.prod(shape))
        sd = int(rng.integers(0, 2**63 - 1))

        def gen(n=n, sd=sd, t=t, in_f=in_f):
            if dev is not None and t in ("BF16", "F16", "F32", "Q8_0", "Q4_K", "Q6_K", "NVFP4"):
                q = _rand_matrix(n // in_f, in_f, t, dev, tgen).data
                return q.contiguous().view(torch.uint8).reshape(-1).cpu().numpy()
            x = np.random.default_rng(sd).standard_normal(n, dtype=np.float32) * WEIGHT_STD
            return qref.quantize(t, x)

        if add:
            w.add_tensor(gname, gen, shape, t)
        return gen, t

    def fused(gname: str, pieces, in_f: int):
        """One tensor whose rows are the rows of `pieces` [(gen, type, out_f)] one after the other."""
        types = {t for _, t, _ in pieces}
        if len(types) != 1:
            raise ValueError(f"{gname}: the fused pieces have different encodings {sorted(types)}")
        gens = [g_ for g_, _, _ in pieces]
        w.add_tensor(gname, lambda gens=gens: np.concatenate([np.asarray(g_()).reshape(-1).view(np.uint8) for g_ in gens]),
                     (sum(o for _, _, o in pieces), in_f), types.pop())

    def vec(gname: str, n: int):
        v = np.ones(n, dtype=np.float32)
        if norm_jitter:
            v = v + rng.standard_normal(n).astype(np.float32) * norm_jitter
        w.add_tensor(gname, v, (n,), "F32")

    mat("token_embd.weight", "token_embd", 0, cfg.vocab_size, h)
    for i in range(L + cfg.nextn_layers):
        p = f"blk.{i}"
        vec(f"{p}.attn_norm.weight", h)
        if cfg.is_mla:  # latent attention: low-rank (or full) queries, shared latent + rotary key, per-head up-projection
            if cfg.q_lora_rank:
                mat(f"{p}.attn_q_a.weight", "attn_q", i, cfg.q_lora_rank, h)
                vec(f"{p}.attn_q_a_norm.weight", cfg.q_lora_rank)
                mat(f"{p}.attn_q_b.weight", "attn_q", i, cfg.q_size, cfg.q_lora_rank)
            else:
                mat(f"{p}.attn_q.weight", "attn_q", i, cfg.q_size, h)
            mat(f"{p}.attn_kv_a_mqa.weight", "attn_k", i, cfg.kv_lora_rank + cfg.rotary_dim, h)
            vec(f"{p}.attn_kv_a_norm.weight", cfg.kv_lora_rank)
            mat(f"{p}.attn_kv_b.weight", "attn_v", i, cfg.n_heads * (cfg.qk_nope_dim + cfg.v_head_dim), cfg.kv_lora_rank)
        else:
            gq = mat(f"{p}.attn_q.weight", "attn_q", i, cfg.q_size, h, add=not fused_layout)
            gk = mat(f"{p}.attn_k.weight", "attn_k", i, cfg.kv_size, h, add=not fused_layout)
            gv = mat(f"{p}.attn_v.weight", "attn_v", i, cfg.kv_size, h, add=not fused_layout)
            if fused_layout:
                fused(f"{p}.attn_qkv.weight", [(*gq, cfg.q_size), (*gk, cfg.kv_size), (*gv, cfg.kv_size)], h)
        if cfg.attn_bias:  # Qwen2-style q/k/v projection biases
            for nm, nb in (("attn_q", cfg.q_size), ("attn_k", cfg.kv_size), ("attn_v", cfg.kv_size)):
                w.add_tensor(f"{p}.{nm}.bias", (rng.standard_normal(nb) * 0.1).astype(np.float32), (nb,), "F32")
        mat(f"{p}.attn_output.weight", "attn_output", i, h, cfg.n_heads * cfg.v_head_dim if cfg.is_mla else cfg.q_size)
        if cfg.qk_norm:
            vec(f"{p}.attn_q_norm.weight", hd)
            vec(f"{p}.attn_k_norm.weight", hd)
        vec(f"{p}.ffn_norm.weight", h)
        if cfg.post_norms:  # Gemma-2/3: norms on the branch outputs
            vec(f"{p}.post_attention_norm.weight", h)
            vec(f"{p}.post_ffw_norm.weight", h)
        if cfg.layer_is_moe(min(i, L - 1)):
            w.add_tensor(f"{p}.ffn_gate_inp.weight",
                         (rng.standard_normal((cfg.n_experts, h)) * WEIGHT_STD).astype(np.float32),
                         (cfg.n_experts, h), "F32")
            ef = cfg.expert_ffn_size
            mat(f"{p}.ffn_gate_exps.weight", "ffn_gate", i, ef, h, cfg.n_experts)
            mat(f"{p}.ffn_up_exps.weight", "ffn_up", i, ef, h, cfg.n_experts)
            mat(f"{p}.ffn_down_exps.weight", "ffn_gate", i, h, ef, cfg.n_experts)
            if cfg.router_bias:
                w.add_tensor(f"{p}.exp_probs_b.bias", (rng.standard_normal(cfg.n_experts) * 0.01).astype(np.float32),
                             (cfg.n_experts,), "F32")
            if cfg.n_shared_experts:
                sf = cfg.shared_expert_ffn_size or ef
                mat(f"{p}.ffn_gate_shexp.weight", "ffn_gate", i, sf, h)
                mat(f"{p}.ffn_up_shexp.weight", "ffn_up", i, sf, h)
                mat(f"{p}.ffn_down_shexp.weight", "ffn_gate", i, h, sf)
                if cfg.shared_expert_gate:
                    w.add_tensor(f"{p}.ffn_gate_inp_shexp.weight",
                                 (rng.standard_normal((1, h)) * WEIGHT_STD).astype(np.float32), (1, h), "F32")
        else:
            gg = mat(f"{p}.ffn_gate.weight", "ffn_gate", i, cfg.ffn_size, h, add=not fused_layout)
            gu = mat(f"{p}.ffn_up.weight", "ffn_up", i, cfg.ffn_size, h, add=not fused_layout)
            if fused_layout:
                fused(f"{p}.ffn_up.weight", [(*gg, cfg.ffn_size), (*gu, cfg.ffn_size)], h)
            mat(f"{p}.ffn_down.weight", "ffn_down", i, h, cfg.ffn_size)
        if i >= L:
            q = f"{p}.nextn"
            vec(f"{q}.enorm.weight", h)
            vec(f"{q}.hnorm.weight", h)
            mat(f"{q}.eh_proj.weight", "attn_q", i, h, 2 * h)
            vec(f"{q}.shared_head_norm.weight", h)
    vec("output_norm.weight", h)
    if rope_freqs is not None:
        w.add_tensor("rope_freqs.weight", np.asarray(rope_freqs, dtype=np.float32), (len(rope_freqs),), "F32")
    if not cfg.tie_embeddings:
        mat("output.weight", "output", 0, cfg.vocab_size, h)
    w.write()
    return path


# --------------------------------------------------------------------------- direct device init


def _rand_matrix(out_f: int, in_f: int, qtype: str, device, gen: torch.Generator) -> QTensor:
    """N(0, 0.02) weight generated on the device and encoded there (no host round trip)."""
    qtype = qtype.upper()
    if qtype in ("BF16", "F16", "F32"):
        dt = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32}[qtype]
        w = torch.empty(out_f, in_f, dtype=dt, device=device)
        step = max(1, (1 << 28) // max(in_f, 1))
        for r in range(0, out_f, step):
            w[r : r + step].normal_(0.0, WEIGHT_STD, generator=gen)
        return QTensor(qtype, w, (out_f, in_f))
    from ..quant import torch_quant

    return torch_quant.random_quantized(out_f, in_f, qtype, device, gen, WEIGHT_STD)


def synth_weights(cfg: ModelConfig, device, quant: str = "BF16", seed: int = 0, tp_rank: int = 0, tp_size: int = 1,
                  ep_rank: int = 0, ep_size: int = 1, layer_range=None, expert_quant: Optional[str] = None) -> ModelWeights:
    """Build this rank's shard of a random-init model directly on ``device``.

    Every rank draws its own shard from a rank-specific stream; replicated tensors (norms,
    embedding, router) use a shared stream so that all ranks hold identical copies."""
    device = torch.device(device)
    shared = torch.Generator(device=device)
    shared.manual_seed(seed)
    own = torch.Generator(device=device)
    own.manual_seed(seed * 1000003 + 7919 * (tp_rank + 1) + 104729 * (ep_rank + 1))
    h, hd, L = cfg.hidden_size, cfg.head_dim, cfg.n_layers
    kv_rep = max(1, tp_size // cfg.n_kv_heads)
    nq = cfg.n_heads // tp_size
    nkv = max(1, cfg.n_kv_heads // tp_size)
    ones = lambda n: torch.ones(n, dtype=torch.float32, device=device)
    l0, l1 = layer_range if layer_range is not None else (0, L)
    layers = []
    for i in range(l0, l1):
        tq = pick_type(quant, "attn_q", i, L, h)
        tv = pick_type(quant, "attn_v", i, L, h)
        if tq == tv:
            qkv = [_rand_matrix((nq + 2 * nkv) * hd, h, tq, device, own)]
        else:
            qkv = [_rand_matrix((nq + nkv) * hd, h, tq, device, own), _rand_matrix(nkv * hd, h, tv, device, own)]
        lw = LayerWeights(attn_norm=ones(h), wqkv=LinearWeight(qkv),
                          wo=LinearWeight([_rand_matrix(h, nq * hd, pick_type(quant, "attn_output", i, L, nq * hd), device, own)]),
                          ffn_norm=ones(h))
        if cfg.qk_norm:
            lw.q_norm, lw.k_norm = ones(hd), ones(hd)
        if cfg.post_norms:
            lw.post_attn_norm, lw.post_ffn_norm = ones(h), ones(h)
        if cfg.layer_is_moe(i):
            lw.router = _rand_matrix(cfg.n_experts, h, "F32" if device.type == "cpu" else "BF16", device, shared)
            e0, e1 = shard_range(cfg.n_experts, ep_rank, ep_size)
            ef = cfg.expert_ffn_size
            tg = pick_type(expert_quant or quant, "ffn_gate", i, L, h)
            td = pick_type(expert_quant or quant, "ffn_gate", i, L, ef)
            lw.experts = ExpertWeights([_rand_matrix(2 * ef, h, tg, device, own) for _ in range(e0, e1)],
                                       [_rand_matrix(h, ef, td, device, own) for _ in range(e0, e1)], e0)
        else:
            f = cfg.ffn_size // tp_size
            lw.w_gate_up = LinearWeight([_rand_matrix(2 * f, h, pick_type(quant, "ffn_gate", i, L, h), device, own)])
            lw.w_down = LinearWeight([_rand_matrix(h, f, pick_type(quant, "ffn_down", i, L, f), device, own)])
        layers.append(lw)
    emb_t = pick_type(quant, "token_embd", 0, L, h)
    embed = _rand_matrix(cfg.vocab_size, h, emb_t, device, shared)
    v0, v1 = shard_range(cfg.vocab_size, tp_rank, tp_size) if cfg.vocab_size % tp_size == 0 else (0, cfg.vocab_size)
    if cfg.tie_embeddings:
        head = embed.rows(v0, v1)
    else:
        head = _rand_matrix(v1 - v0, h, pick_type(quant, "output", 0, L, h), device, own)
    return ModelWeights(cfg, embed, layers, ones(h), LinearWeight([head]), [], tp_rank, tp_size, ep_rank, ep_size, l0, v0)


def _main(argv=None) -> int:
    """``python -m oxidize_b200.utils.synth --preset llama3-8b --quant Q4_K_M --out model.gguf``"""
    import argparse

    from ..models.config import preset, preset_names

    ap = argparse.ArgumentParser(description="write a random-init GGUF of a named shape")
    ap.add_argument("--preset", required=True, choices=preset_names())
    ap.add_argument("--quant", default="Q4_K_M")
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count")
    ap.add_argument("--context", type=int, default=0, help="override the advertised context length")
    ap.add_argument("--embed-type", default=None, help="store the token embedding table in this type")
    ap.add_argument("--device", default="auto", help="cuda device used to draw and encode the weights; 'cpu' = NumPy")
    a = ap.parse_args(argv)
    cfg = preset(a.preset)
    if a.layers:
        cfg.n_layers = a.layers
    if a.context:
        cfg.context_length = a.context
    dev = a.device
    if dev == "auto":
        dev = "cuda" if torch.cuda.is_available() else "cpu"
    synth_gguf(a.out, cfg, a.quant, seed=a.seed, device=None if dev == "cpu" else dev, embed_type=a.embed_type)
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
