"""HF SafeTensors directory (``config.json`` + ``*.safetensors``) → GGUF, optionally quantizing.

Counterpart of the reference's converter (``oxidize-core/src/format/safetensors_to_gguf.rs``:
architecture metadata written from ``config.json`` ``:446-560``, tensor-name mapping via
``map_hf_decoder_name``, per-expert tensors stacked into ``ffn_*_exps``).  Also usable as
``python -m oxidize_b200.formats.convert SRC_DIR OUT.gguf --quant Q4_K_M``.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from ..quant import ref as qref
from ..utils.synth import pick_type
from .gguf import GGUFValueType, GGUFWriter, map_hf_tensor_name
from .safetensors_io import SafeTensorsFile

_ARCH = {"LlamaForCausalLM": "llama", "MistralForCausalLM": "llama", "MixtralForCausalLM": "mixtral",
         "Qwen2ForCausalLM": "qwen2", "Qwen3ForCausalLM": "qwen3", "Qwen3MoeForCausalLM": "qwen3moe",
         "Qwen2MoeForCausalLM": "qwen2moe", "DeepseekV2ForCausalLM": "deepseek2", "DeepseekV3ForCausalLM": "deepseek2",
         "Phi3ForCausalLM": "phi3", "GemmaForCausalLM": "gemma", "Gemma2ForCausalLM": "gemma2",
         "Gemma3ForCausalLM": "gemma3", "Gemma3ForConditionalGeneration": "gemma3", "Lfm2ForCausalLM": "lfm2",
         "Lfm2MoeForCausalLM": "lfm2moe", "Glm4MoeForCausalLM": "glm4moe", "Glm4ForCausalLM": "glm4", "MiniMaxM2ForCausalLM": "minimax-m2",
         "Qwen3_5ForCausalLM": "qwen35", "Qwen3_5ForConditionalGeneration": "qwen35",
         "Qwen3_5MoeForCausalLM": "qwen35moe", "Qwen3_5MoeForConditionalGeneration": "qwen35moe",
         "HunYuanMoEV1ForCausalLM": "hunyuan-moe", "HunYuanDenseV1ForCausalLM": "hunyuan-dense", "MambaForCausalLM": "mamba"}
GEMMA = ("gemma", "gemma2", "gemma3")


def arch_from_config(cfg: Dict[str, Any]) -> str:
    for a in cfg.get("architectures") or []:
        if a in _ARCH:
            return _ARCH[a]
    mt = str(cfg.get("model_type", "llama")).lower()
    return {"mistral": "llama", "qwen3_moe": "qwen3moe", "qwen2_moe": "qwen2moe", "deepseek_v2": "deepseek2",
            "deepseek_v3": "deepseek2", "gemma3_text": "gemma3"}.get(mt, mt)


def _rope_settings(c: Dict[str, Any]) -> Tuple[float, float, Dict[str, Any]]:
    """(rotary base, rotary base of the windowed layers or 0, scaling dict) from either config layout: the flat keys
    (``rope_theta``, ``rope_local_base_freq``, ``rope_scaling``) or the nested ``rope_parameters`` (per attention kind
    for models with local and global layers)."""
    rp = c.get("rope_parameters") or {}
    if "full_attention" in rp or "sliding_attention" in rp:
        full, local = rp.get("full_attention") or {}, rp.get("sliding_attention") or {}
        return float(full.get("rope_theta", 10000.0)), float(local.get("rope_theta", 0.0)), full
    theta = float(rp.get("rope_theta") or c.get("rope_theta") or 10000.0)
    if rp.get("rope_type") == "dynamic" and rp.get("alpha") and str(c.get("model_type", "")).startswith("hunyuan"):
        # Hunyuan's fixed NTK stretch: the base grows by alpha ** (d / (d - 2)); files carry the grown base
        hd = int(c.get("head_dim") or int(c["hidden_size"]) // int(c["num_attention_heads"]))
        return theta * float(rp["alpha"]) ** (hd / (hd - 2)), 0.0, {}
    return theta, float(c.get("rope_local_base_freq") or 0.0), (rp if rp.get("rope_type") else c.get("rope_scaling") or {})


def rope_factor_tensors(c: Dict[str, Any]) -> Dict[str, np.ndarray]:
    """Per-frequency divisors that a checkpoint's rotary scaling implies, as the tensors files carry them:
    ``rope_freqs.weight`` for the Llama-3.1 rule (low frequencies divided by ``factor``, high ones kept, a smooth ramp
    between), ``rope_factors_short / _long.weight`` for LongRoPE (Phi-3)."""
    import math

    _, _, rs = _rope_settings(c)
    kind = str(rs.get("rope_type") or rs.get("type") or "")
    if kind not in ("llama3", "longrope", "su", "yarn_long"):
        return {}
    heads = int(c["num_attention_heads"])
    hd = int(c.get("head_dim") or int(c["hidden_size"]) // heads)
    rot = int(hd * float(c.get("partial_rotary_factor", 1.0)))
    if kind == "llama3":
        theta = float(rs.get("rope_theta") or c.get("rope_theta") or 10000.0)
        factor, lo, hi = float(rs.get("factor", 8.0)), float(rs.get("low_freq_factor", 1.0)), float(rs.get("high_freq_factor", 4.0))
        orig = float(rs.get("original_max_position_embeddings", 8192))
        out = []
        for i in range(0, rot, 2):
            wavelen = 2 * math.pi * theta ** (i / rot)
            if wavelen < orig / hi:
                out.append(1.0)
            elif wavelen > orig / lo:
                out.append(factor)
            else:
                smooth = (orig / wavelen - lo) / (hi - lo)
                out.append(1.0 / ((1.0 - smooth) / factor + smooth))
        return {"rope_freqs.weight": np.asarray(out, dtype=np.float32)}
    if kind in ("longrope", "su", "yarn_long") and rs.get("short_factor") is not None:
        return {"rope_factors_short.weight": np.asarray(rs["short_factor"], dtype=np.float32),
                "rope_factors_long.weight": np.asarray(rs["long_factor"], dtype=np.float32)}
    return {}


def write_mamba_metadata(w: GGUFWriter, c: Dict[str, Any]) -> None:
    U, F = GGUFValueType.UINT32, GGUFValueType.FLOAT32
    hidden = int(c["hidden_size"])
    w.add("general.name", str(c.get("_name_or_path") or "mamba"))
    w.add("mamba.vocab_size", int(c["vocab_size"]), U)
    w.add("mamba.embedding_length", hidden, U)
    w.add("mamba.block_count", int(c["num_hidden_layers"]), U)
    w.add("mamba.context_length", int(c.get("max_position_embeddings", 1 << 20)), U)
    w.add("mamba.ssm.conv_kernel", int(c.get("conv_kernel", 4)), U)
    w.add("mamba.ssm.inner_size", int(c.get("intermediate_size") or int(c.get("expand", 2)) * hidden), U)
    w.add("mamba.ssm.state_size", int(c.get("state_size", 16)), U)
    rank = c.get("time_step_rank", "auto")
    w.add("mamba.ssm.time_step_rank", -(-hidden // 16) if rank == "auto" else int(rank), U)
    w.add("mamba.attention.layer_norm_rms_epsilon", float(c.get("layer_norm_epsilon", 1e-5)), F)


def write_hf_metadata(w: GGUFWriter, arch: str, c: Dict[str, Any]) -> None:
    U, F = GGUFValueType.UINT32, GGUFValueType.FLOAT32
    if arch == "mamba":
        return write_mamba_metadata(w, c)
    heads = int(c["num_attention_heads"])
    hidden = int(c["hidden_size"])
    w.add("general.name", str(c.get("_name_or_path") or c.get("model_type") or "converted"))
    w.add(f"{arch}.vocab_size", int(c["vocab_size"]), U)
    w.add(f"{arch}.embedding_length", hidden, U)
    w.add(f"{arch}.block_count", int(c["num_hidden_layers"]), U)
    w.add(f"{arch}.context_length", int(c.get("max_position_embeddings", 4096)), U)
    ffn = int(c.get("intermediate_size", 0))
    if arch == "lfm2" and c.get("block_auto_adjust_ff_dim"):
        # the checkpoint's MLP width is derived from intermediate_size (two thirds, scaled, rounded up to a multiple)
        ffn = int(2 * ffn / 3)
        if c.get("block_ffn_dim_multiplier"):
            ffn = int(float(c["block_ffn_dim_multiplier"]) * ffn)
        mult = int(c.get("block_multiple_of", 256))
        ffn = mult * ((ffn + mult - 1) // mult)
    w.add(f"{arch}.feed_forward_length", ffn, U)
    w.add(f"{arch}.attention.head_count", heads, U)
    kvh = int(c.get("num_key_value_heads", heads))
    if arch in ("lfm2", "lfm2moe"):
        # one entry per layer, 0 for the convolution layers (as llama.cpp's converter writes it)
        kinds = c.get("layer_types") or []
        w.add(f"{arch}.attention.head_count_kv", [kvh if k == "full_attention" else 0 for k in kinds] or kvh)
        w.add(f"{arch}.shortconv.l_cache", int(c.get("conv_L_cache", 3)), U)
    else:
        w.add(f"{arch}.attention.head_count_kv", kvh, U)
    hd = int(c.get("head_dim") or hidden // heads)
    if c.get("kv_lora_rank"):
        # latent attention: per-head query / key width (position-free + rotary part) and value width
        hd = int(c["qk_nope_head_dim"]) + int(c["qk_rope_head_dim"])
        w.add(f"{arch}.attention.kv_lora_rank", int(c["kv_lora_rank"]), U)
        if c.get("q_lora_rank"):
            w.add(f"{arch}.attention.q_lora_rank", int(c["q_lora_rank"]), U)
    w.add(f"{arch}.attention.key_length", hd, U)
    w.add(f"{arch}.attention.value_length", int(c.get("v_head_dim") or hd), U)
    w.add(f"{arch}.attention.layer_norm_rms_epsilon", float(c.get("rms_norm_eps") or c.get("norm_eps") or 1e-5), F)
    theta, theta_swa, rs = _rope_settings(c)
    w.add(f"{arch}.rope.freq_base", theta, F)
    w.add(f"{arch}.rope.dimension_count",
          int(c["qk_rope_head_dim"]) if c.get("kv_lora_rank") else int(c["rotary_dim"]) if c.get("rotary_dim") else int(hd * float(c.get("partial_rotary_factor") or (c.get("rope_parameters") or {}).get("partial_rotary_factor") or 1.0)), U)
    if arch in ("qwen35", "qwen35moe"):
        vh, vd = int(c.get("linear_num_value_heads", 0)), int(c.get("linear_value_head_dim", 0))
        w.add(f"{arch}.ssm.conv_kernel", int(c.get("linear_conv_kernel_dim", 4)), U)
        w.add(f"{arch}.ssm.state_size", int(c.get("linear_key_head_dim", vd)), U)
        w.add(f"{arch}.ssm.group_count", int(c.get("linear_num_key_heads", vh)), U)
        w.add(f"{arch}.ssm.time_step_rank", vh, U)
        w.add(f"{arch}.ssm.inner_size", vh * vd, U)
        kinds = c.get("layer_types") or []
        if "full_attention" in kinds:
            w.add(f"{arch}.full_attention_interval", kinds.index("full_attention") + 1, U)
    if c.get("sliding_window"):
        w.add(f"{arch}.attention.sliding_window", int(c["sliding_window"]), U)
    if arch in GEMMA:
        if theta_swa > 0:
            w.add(f"{arch}.rope.freq_base_swa", theta_swa, F)
        kinds = c.get("layer_types") or []
        if "full_attention" in kinds and "sliding_attention" in kinds:
            # every n-th layer attends over the whole context
            w.add(f"{arch}.attention.sliding_window_pattern", kinds.index("full_attention") + 1, U)
        elif c.get("sliding_window_pattern"):
            w.add(f"{arch}.attention.sliding_window_pattern", int(c["sliding_window_pattern"]), U)
        if arch == "gemma2":
            w.add(f"{arch}.attn_logit_softcapping", float(c.get("attn_logit_softcapping") or 0.0), F)
            w.add(f"{arch}.final_logit_softcapping", float(c.get("final_logit_softcapping") or 0.0), F)
        if c.get("query_pre_attn_scalar"):
            w.add(f"{arch}.attention.scale", float(c["query_pre_attn_scalar"]) ** -0.5, F)
    if rs.get("type") or rs.get("rope_type"):
        kind = str(rs.get("type") or rs.get("rope_type"))
        if kind in ("longrope", "su") and rs.get("short_factor") is not None:
            # LongRoPE: the factor tensors carry the scaling; the metadata says where the long set takes over and by how
            # much the rotated vectors are magnified then
            import math

            orig = int(rs.get("original_max_position_embeddings") or c.get("original_max_position_embeddings")
                       or c.get("max_position_embeddings", 0))
            scale = float(c.get("max_position_embeddings", orig)) / max(orig, 1)
            w.add(f"{arch}.rope.scaling.original_context_length", orig, U)
            att = rs.get("attention_factor")
            w.add(f"{arch}.rope.scaling.attn_factor",
                  float(att) if att else (math.sqrt(1 + math.log(scale) / math.log(orig)) if scale > 1 else 1.0), F)
        if kind in ("linear", "yarn"):
            w.add(f"{arch}.rope.scaling.type", kind)
            w.add(f"{arch}.rope.scaling.factor", float(rs.get("factor", 1.0)), F)
            w.add(f"{arch}.rope.scaling.original_context_length",
                  int(rs.get("original_max_position_embeddings", c.get("max_position_embeddings", 0))), U)
            if kind == "yarn" and c.get("kv_lora_rank"):
                w.add(f"{arch}.rope.scaling.yarn_log_multiplier", 0.1 * float(rs.get("mscale_all_dim") or 0.0), F)
    n_exp = int(c.get("num_local_experts") or c.get("num_experts") or c.get("n_routed_experts") or 0)
    if n_exp > 1 or (n_exp and not arch.startswith("hunyuan")):
        w.add(f"{arch}.expert_count", n_exp, U)
        w.add(f"{arch}.expert_used_count", int(c.get("num_experts_per_tok") or c.get("moe_topk") or 2), U)
        w.add(f"{arch}.expert_feed_forward_length", int(c.get("moe_intermediate_size") or c.get("intermediate_size")), U)
        # DeepSeek-V3 configs often omit scoring_func: that model always scores with a sigmoid
        sigmoid = c.get("scoring_func") == "sigmoid" or (c.get("scoring_func") is None
                                                         and c.get("model_type") in ("deepseek_v3", "lfm2_moe", "glm4_moe", "minimax_m2"))
        w.add(f"{arch}.expert_gating_func", 2 if sigmoid else 1, U)
        w.add(f"{arch}.expert_weights_scale", float(c.get("routed_scaling_factor", 1.0)), F)
        w.add(f"{arch}.expert_weights_norm", bool(c.get("norm_topk_prob", True)))
        if c.get("n_group"):
            w.add(f"{arch}.expert_group_count", int(c["n_group"]), U)
            w.add(f"{arch}.expert_group_used_count", int(c.get("topk_group", 1)), U)
        if c.get("n_shared_experts"):
            w.add(f"{arch}.expert_shared_count", int(c["n_shared_experts"]), U)
        dense = c.get("first_k_dense_replace") or c.get("num_dense_layers")
        if dense:
            w.add(f"{arch}.leading_dense_block_count", int(dense), U)


def _kind_of(gname: str) -> str:
    base = gname.split(".")[-2] if gname.count(".") >= 2 else gname.split(".")[0]
    return {"token_embd": "token_embd", "output": "output"}.get(base, base.replace("_exps", "").replace("_shexp", ""))


def convert_safetensors_to_gguf(src_dir: str, out_path: str, quant: str = "F16", tokenizer_metadata: Dict = None) -> str:
    with open(os.path.join(src_dir, "config.json")) as f:
        cfg = json.load(f)
    if "text_config" in cfg:
        # multimodal wrapper (LLaVA, Gemma-3 with vision): the language model's settings are nested and only its tensors
        # are converted; the vision tower goes into a projector file of its own (vision.convert_vision_tower)
        wrapper = cfg
        cfg = dict(wrapper["text_config"])
        if cfg.get("model_type") == "gemma3_text" or "Gemma3" in "".join(wrapper.get("architectures") or []):
            cfg.setdefault("architectures", ["Gemma3ForCausalLM"])
    arch = arch_from_config(cfg)
    files = [SafeTensorsFile(p) for p in sorted(glob.glob(os.path.join(src_dir, "*.safetensors")))]
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {src_dir}")
    w = GGUFWriter(out_path, arch=arch)
    write_hf_metadata(w, arch, cfg)
    for k, v in (tokenizer_metadata or {}).items():
        w.add(k, v)
    L = int(cfg.get("num_hidden_layers") or cfg.get("n_layer"))
    plain: List[Tuple[str, SafeTensorsFile, str]] = []
    experts: Dict[str, Dict[int, Tuple[SafeTensorsFile, str]]] = {}
    for f in files:
        for name in f.keys():
            m = map_hf_tensor_name(name, arch)
            if m is None:
                continue
            gname, e = m
            if e is None:
                plain.append((gname, f, name))
            else:
                experts.setdefault(gname, {})[e] = (f, name)

    def layer_of(gname: str) -> int:
        parts = gname.split(".")
        return int(parts[1]) if parts[0] == "blk" else 0

    def encode(gname: str, arr_f32: np.ndarray):
        if (arr_f32.ndim == 1 or "norm" in gname or gname.endswith(".bias") or "ffn_gate_inp" in gname or gname.endswith("ssm_d")
                or "ssm_alpha" in gname or "ssm_beta" in gname):
            if (arch in GEMMA or (arch in ("qwen35", "qwen35moe") and not gname.endswith("ssm_norm.weight"))) and gname.endswith("norm.weight"):
                arr_f32 = arr_f32 + 1.0  # Gemma and Qwen3.5 store w - 1; files carry the multiplier itself (as llama.cpp's do)
            return arr_f32.astype(np.float32), "F32"
        t = pick_type(quant, _kind_of(gname), layer_of(gname), L, arr_f32.shape[-1])
        return qref.quantize(t, arr_f32.reshape(-1)), t

    for gname, f, name in plain:
        shape = f.shape(name)
        if gname.endswith("ssm_a"):  # the checkpoint stores log(-A); files carry A itself
            w.add_tensor(gname, (lambda f=f, name=name: (-np.exp(f.tensor_f32(name))).astype(np.float32)), shape, "F32")
            continue
        if gname.endswith(("ssm_conv1d.weight", "shortconv.conv.weight")):  # [channels, 1, taps] -> [channels, taps], kept in f32
            shape = (shape[0], shape[-1])
            w.add_tensor(gname, (lambda f=f, name=name, shape=shape: f.tensor_f32(name).reshape(shape).astype(np.float32)),
                         shape, "F32")
            continue

        def gen(f=f, name=name, gname=gname):
            return encode(gname, f.tensor_f32(name))[0]

        t = encode(gname, np.zeros(shape[-1:] if len(shape) == 1 else (1, shape[-1]), dtype=np.float32))[1]
        w.add_tensor(gname, gen, shape, t)
    for tname, arr in rope_factor_tensors(cfg).items():
        w.add_tensor(tname, arr, arr.shape, "F32")
    for gname, per in experts.items():
        n = max(per) + 1
        f0, n0 = per[0]
        rows, cols = f0.shape(n0)

        def gen_e(per=per, n=n, gname=gname):
            return np.concatenate([np.ascontiguousarray(encode(gname, per[e][0].tensor_f32(per[e][1]))[0]).view(np.uint8)
                                   .reshape(-1) for e in range(n)])

        t = pick_type(quant, _kind_of(gname), layer_of(gname), L, cols)
        w.add_tensor(gname, gen_e, (n, rows, cols), t)
    w.write()
    return out_path


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="HF SafeTensors → GGUF")
    ap.add_argument("src")
    ap.add_argument("out")
    ap.add_argument("--quant", default="F16")
    a = ap.parse_args()
    print(convert_safetensors_to_gguf(a.src, a.out, a.quant, tokenizer_metadata_from_hf(a.src)))


def tokenizer_metadata_from_hf(src_dir: str) -> Dict[str, Any]:
    """GGUF tokenizer metadata from a Hugging Face directory's ``tokenizer.json`` (+ ``tokenizer_config.json`` for the
    special tokens and the chat template): byte-level BPE becomes ``tokenizer.ggml.model = gpt2`` (tokens, merges), a
    Unigram model becomes ``llama`` (tokens, scores).  Other tokenizer kinds give an empty mapping: the model then loads
    without a tokenizer and wants token ids, or ``--tokenizer-model`` with a GGUF that has one."""
    tj = os.path.join(src_dir, "tokenizer.json")
    if not os.path.isfile(tj):
        return {}
    with open(tj, encoding="utf-8") as f:
        t = json.load(f)
    model = t.get("model") or {}
    kind = model.get("type")
    added = {int(a["id"]): a for a in t.get("added_tokens") or []}

    def uses_byte_level(node) -> bool:
        if isinstance(node, dict):
            return node.get("type") == "ByteLevel" or any(uses_byte_level(v) for v in node.values())
        if isinstance(node, list):
            return any(uses_byte_level(v) for v in node)
        return False

    md: Dict[str, Any] = {}
    if kind == "BPE" and uses_byte_level(t.get("pre_tokenizer")) and not model.get("byte_fallback"):
        vocab = model.get("vocab") or {}
        n = max(list(vocab.values()) + list(added) + [-1]) + 1
        tokens = [f"[PAD{i}]" for i in range(n)]
        for tok, i in vocab.items():
            tokens[int(i)] = tok
        for i, a in added.items():
            tokens[i] = a["content"]
        merges = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges") or []]
        types = [3 if (i in added and added[i].get("special")) else 1 for i in range(n)]
        md = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": merges,
              "tokenizer.ggml.token_type": types}
    elif kind == "Unigram":
        pieces = model.get("vocab") or []
        tokens = [p[0] for p in pieces]
        scores = [float(p[1]) for p in pieces]
        for i, a in added.items():
            if i < len(tokens):
                tokens[i] = a["content"]
        types = [3 if (i in added and added[i].get("special")) else 1 for i in range(len(tokens))]
        md = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.scores": scores,
              "tokenizer.ggml.token_type": types}
        if model.get("unk_id") is not None:
            md["tokenizer.ggml.unknown_token_id"] = int(model["unk_id"])
    if not md:
        return {}
    ids = {tok: i for i, tok in enumerate(md["tokenizer.ggml.tokens"])}
    cfgp = os.path.join(src_dir, "tokenizer_config.json")
    if os.path.isfile(cfgp):
        with open(cfgp, encoding="utf-8") as f:
            tc = json.load(f)
        for key, name in (("bos_token", "bos_token_id"), ("eos_token", "eos_token_id"), ("unk_token", "unknown_token_id"),
                          ("pad_token", "padding_token_id")):
            v = tc.get(key)
            v = v.get("content") if isinstance(v, dict) else v
            if isinstance(v, str) and v in ids:
                md[f"tokenizer.ggml.{name}"] = ids[v]
        if isinstance(tc.get("chat_template"), str):
            md["tokenizer.chat_template"] = tc["chat_template"]
        if tc.get("add_bos_token") is not None:
            md["tokenizer.ggml.add_bos_token"] = bool(tc["add_bos_token"])
    return md
