"""LoRA / QLoRA supervised fine-tuning on the CPU path, self-training rounds, per-round checkpoints with resume, and export
(the reference's ``oxidize-finetuning`` crate: ``src/trainer.rs``, ``lora.rs``, ``qlora.rs``, ``self_train.rs``,
``export.rs``).

The trainer has a dense, differentiable forward of its own over whole sequences (no paged cache): RMSNorm, fused qkv with
optional biases and per-head QK-norm, rotary embedding, causal grouped-query attention with an optional window, SwiGLU or
GeGLU, tied or separate head, for the dense decoder families the engine serves.  It reads the same ``ModelWeights`` the
engine loads, so the frozen base can stay in its checkpoint encoding (QLoRA: a quantized matrix is decoded each time it is
used and never kept as float) and the test suite checks its logits against the engine's.  Only the low-rank pairs train.
Adapters are written in the PEFT layout (``adapter_model.safetensors`` + ``adapter_config.json``), which
``oxidize lora-merge`` folds into a GGUF.

    python -m oxidize_b200.offline.finetune --model base.gguf --data sft.jsonl --output out_dir --steps 200 \\
        [--qlora] [--resume-from out_dir/round-0003] [--self-train-rounds 2 --prompts prompts.txt] [--merge-output merged.gguf]
        [--dpo-data prefs.jsonl --dpo-beta 0.1]

Preference training (``dpo.rs`` in the reference) is direct preference optimisation with the adapter-free base as the
reference policy.  Data: JSON lines with ``{"prompt": ..., "completion": ...}`` (loss on the completion only), ``{"text": ...}`` (loss on
every token) or ``{"messages": [...]}`` (rendered with the model's chat template; loss on the last assistant turn).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
from dataclasses import asdict, dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..formats.gguf import load_gguf
from ..formats.safetensors_io import SafeTensorsFile, save_file
from ..models.config import ModelConfig, config_from_gguf
from ..models.weights import LinearWeight, ModelWeights, load_weights
from ..ops import ref as opref

TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "lm_head")
_HF_MODULE = {"q_proj": "self_attn.q_proj", "k_proj": "self_attn.k_proj", "v_proj": "self_attn.v_proj",
              "o_proj": "self_attn.o_proj", "gate_proj": "mlp.gate_proj", "up_proj": "mlp.up_proj", "down_proj": "mlp.down_proj"}


@dataclass
class LoraConfig:
    r: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    targets: Tuple[str, ...] = ("q_proj", "v_proj")

    @property
    def scale(self) -> float:
        return self.alpha / self.r


@dataclass
class TrainConfig:
    steps: int = 100
    batch_size: int = 4
    lr: float = 2e-4
    weight_decay: float = 0.0
    warmup_steps: int = 0
    max_seq_len: int = 512
    grad_clip: float = 1.0
    seed: int = 0
    qlora: bool = False  # keep quantized base matrices encoded; decode per use
    checkpoint_every: int = 0  # steps; 0 = only at the end of a round


@dataclass
class Example:
    tokens: List[int]
    loss_from: int  # first position whose token is a training target


class LoraModel(torch.nn.Module):
    """Frozen base (``ModelWeights`` on the CPU in float32 or in its quantized encoding) + trainable low-rank pairs."""

    def __init__(self, weights: ModelWeights, lora: LoraConfig, qlora: bool = False, seed: int = 0):
        super().__init__()
        cfg = weights.cfg
        if cfg.is_moe or cfg.is_mla or cfg.is_ssm or cfg.conv_layers or cfg.qk_norm_after_rope:
            raise NotImplementedError("the trainer covers the dense grouped-query decoder families")
        if weights.tp_size != 1 or weights.first_layer != 0:
            raise ValueError("the trainer wants the whole model on one rank")
        bad = [t for t in lora.targets if t not in TARGETS]
        if bad:
            raise ValueError(f"unknown LoRA targets {bad}; choose from {TARGETS}")
        self.w, self.cfg, self.lora, self.qlora = weights, cfg, lora, qlora
        self.inv_freq = opref.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta, cfg.rope_scaling, freq_factors=weights.rope_freq_factors)
        self.inv_freq_swa = (opref.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta_swa, None)
                             if cfg.rope_theta_swa > 0 and cfg.sliding_window > 0 else None)
        self.mscale = opref.rope_mscale(cfg.rope_scaling)
        gen = torch.Generator().manual_seed(seed)
        dims = {"q_proj": (cfg.q_size, cfg.hidden_size), "k_proj": (cfg.kv_size, cfg.hidden_size),
                "v_proj": (cfg.kv_size, cfg.hidden_size), "o_proj": (cfg.hidden_size, cfg.q_size),
                "gate_proj": (cfg.ffn_size, cfg.hidden_size), "up_proj": (cfg.ffn_size, cfg.hidden_size),
                "down_proj": (cfg.hidden_size, cfg.ffn_size)}
        self.A = torch.nn.ParameterDict()
        self.B = torch.nn.ParameterDict()
        if "lm_head" in lora.targets:
            if cfg.tie_embeddings:
                raise ValueError("lm_head cannot be a LoRA target when the head is tied to the embedding table")
            a = (torch.rand(lora.r, cfg.hidden_size, generator=gen) * 2 - 1) / math.sqrt(cfg.hidden_size)
            self.A["head"] = torch.nn.Parameter(a)
            self.B["head"] = torch.nn.Parameter(torch.zeros(cfg.vocab_size, lora.r))
        for i in range(len(weights.layers)):
            for t in lora.targets:
                if t == "lm_head":
                    continue
                out_f, in_f = dims[t]
                bound = 1.0 / math.sqrt(in_f)
                a = (torch.rand(lora.r, in_f, generator=gen) * 2 - 1) * bound
                self.A[f"{i}_{t}"] = torch.nn.Parameter(a)
                self.B[f"{i}_{t}"] = torch.nn.Parameter(torch.zeros(out_f, lora.r))  # zero: training starts at the base model

    # ------------------------------------------------------------------ pieces
    def _dense(self, w: LinearWeight) -> torch.Tensor:
        parts = [opref.dequantize_weight(p) if self.qlora else p.dense_cache() for p in w.parts]
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)

    @staticmethod
    def _hf_base(key: str) -> str:
        if key == "head":
            return "base_model.model.lm_head"
        i, t = key.split("_", 1)
        return f"base_model.model.model.layers.{i}.{_HF_MODULE[t]}"

    adapters_on = True  # False: the forward is the frozen base model (the reference policy of preference training)

    def _delta(self, layer: int, target: str, x: torch.Tensor) -> Optional[torch.Tensor]:
        key = f"{layer}_{target}"
        if key not in self.A or not self.adapters_on:
            return None
        if self.training and self.lora.dropout > 0:
            x = F.dropout(x, self.lora.dropout)
        return (x @ self.A[key].t()) @ self.B[key].t() * self.lora.scale

    def _linear(self, layer: int, w: LinearWeight, x: torch.Tensor, targets: Sequence[Tuple[str, int]]) -> torch.Tensor:
        """x W^T (+ bias) + the low-rank terms of the projections that W's rows consist of: ``targets`` lists them in row
        order with their row counts."""
        y = x @ self._dense(w).t()
        if w.bias is not None:
            y = y + w.bias
        deltas, any_delta = [], False
        for t, rows in targets:
            d = self._delta(layer, t, x)
            any_delta = any_delta or d is not None
            deltas.append(d if d is not None else x.new_zeros(*x.shape[:-1], rows))
        return y + torch.cat(deltas, dim=-1) if any_delta else y

    @staticmethod
    def _norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def _rope(self, x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, mscale: float) -> torch.Tensor:
        b, s, h, d = x.shape
        y = opref.apply_rope(x.reshape(b * s, h, d), positions.repeat(b), inv_freq, self.cfg.rope_pairing, mscale)
        return y.reshape(b, s, h, d)

    # ------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, S] int64 → logits [B, S, vocab] float32 (right-padded batches: the padding comes after every real
        token, so causal attention never lets it reach one)."""
        cfg, w = self.cfg, self.w
        B, S = tokens.shape
        emb = w.embed.dense_cache() if not self.qlora else opref.dequantize_weight(w.embed)
        x = emb[tokens] * cfg.embedding_scale
        pos = torch.arange(S)
        nh, nkv, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        scale = cfg.attn_scale if cfg.attn_scale > 0 else hd ** -0.5
        qpos, kpos = pos[:, None], pos[None, :]
        for i, lw in enumerate(w.layers):
            h = self._norm(x, lw.attn_norm, cfg.rms_eps)
            qkv = self._linear(i, lw.wqkv, h, [("q_proj", cfg.q_size), ("k_proj", cfg.kv_size), ("v_proj", cfg.kv_size)])
            q = qkv[..., : cfg.q_size].reshape(B, S, nh, hd)
            k = qkv[..., cfg.q_size : cfg.q_size + cfg.kv_size].reshape(B, S, nkv, hd)
            v = qkv[..., cfg.q_size + cfg.kv_size :].reshape(B, S, nkv, hd)
            if lw.q_norm is not None:
                q, k = self._norm(q, lw.q_norm, cfg.rms_eps), self._norm(k, lw.k_norm, cfg.rms_eps)
            window = cfg.layer_sliding_window(i)
            inv, ms = (self.inv_freq_swa, 1.0) if (window > 0 and self.inv_freq_swa is not None) else (self.inv_freq, self.mscale)
            q, k = self._rope(q, pos, inv, ms), self._rope(k, pos, inv, ms)
            g = nh // nkv
            qg = q.reshape(B, S, nkv, g, hd)
            s = torch.einsum("bqkgd,blkd->bkgql", qg, k) * scale
            if cfg.attn_softcap > 0:
                s = torch.tanh(s / cfg.attn_softcap) * cfg.attn_softcap
            mask = kpos <= qpos
            if window > 0:
                mask = mask & (kpos > qpos - window)
            s = s.masked_fill(~mask, float("-inf"))
            o = torch.einsum("bkgql,blkd->bqkgd", torch.softmax(s, dim=-1), v).reshape(B, S, nh * hd)
            a = self._linear(i, lw.wo, o, [("o_proj", cfg.hidden_size)])
            if lw.post_attn_norm is not None:
                a = self._norm(a, lw.post_attn_norm, cfg.rms_eps)
            x = x + a
            h = self._norm(x, lw.ffn_norm, cfg.rms_eps)
            gu = self._linear(i, lw.w_gate_up, h, [("gate_proj", cfg.ffn_size), ("up_proj", cfg.ffn_size)])
            gate, up = gu[..., : cfg.ffn_size], gu[..., cfg.ffn_size :]
            act = F.gelu(gate, approximate="tanh") if cfg.ffn_act == "gelu_tanh" else F.silu(gate)
            f = self._linear(i, lw.w_down, act * up, [("down_proj", cfg.hidden_size)])
            if lw.post_ffn_norm is not None:
                f = self._norm(f, lw.post_ffn_norm, cfg.rms_eps)
            x = x + f
        x = self._norm(x, w.out_norm, cfg.rms_eps)
        logits = x @ self._dense(w.lm_head).t()
        if "head" in self.A and self.adapters_on:
            logits = logits + (x @ self.A["head"].t()) @ self.B["head"].t() * self.lora.scale
        if cfg.final_softcap > 0:
            logits = torch.tanh(logits / cfg.final_softcap) * cfg.final_softcap
        return logits

    # ------------------------------------------------------------------ adapters on disk
    def adapter_tensors(self) -> Dict[str, np.ndarray]:
        out = {}
        for key in self.A:
            base = self._hf_base(key)
            out[f"{base}.lora_A.weight"] = self.A[key].detach().numpy().copy()
            out[f"{base}.lora_B.weight"] = self.B[key].detach().numpy().copy()
        return out

    def save_adapter(self, directory: str) -> str:
        os.makedirs(directory, exist_ok=True)
        save_file(self.adapter_tensors(), os.path.join(directory, "adapter_model.safetensors"), {"format": "pt"})
        with open(os.path.join(directory, "adapter_config.json"), "w") as f:
            json.dump({"peft_type": "LORA", "r": self.lora.r, "lora_alpha": self.lora.alpha, "lora_dropout": self.lora.dropout,
                       "target_modules": list(self.lora.targets), "bias": "none", "task_type": "CAUSAL_LM"}, f, indent=1)
        return directory

    def load_adapter(self, directory: str) -> None:
        st = SafeTensorsFile(os.path.join(directory, "adapter_model.safetensors"))
        with torch.no_grad():
            for key in self.A:
                base = self._hf_base(key)
                self.A[key].copy_(torch.from_numpy(st.tensor_f32(f"{base}.lora_A.weight").copy()))
                self.B[key].copy_(torch.from_numpy(st.tensor_f32(f"{base}.lora_B.weight").copy()))


# --------------------------------------------------------------------------- data


def load_examples(path: str, tokenizer, chat_template: Optional[str], max_seq_len: int) -> List[Example]:
    from ..formats.tokenizer import render_chat_template

    out: List[Example] = []
    with open(path) as f:
        for ln, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            try:
                rec = json.loads(line)
            except ValueError as e:
                raise ValueError(f"{path}:{ln}: not JSON ({e})") from None
            if "messages" in rec:
                msgs = rec["messages"]
                if not msgs or msgs[-1].get("role") != "assistant":
                    raise ValueError(f"{path}:{ln}: the last message must be the assistant turn to learn")
                prompt = render_chat_template(chat_template, msgs[:-1], True)
                completion = str(msgs[-1]["content"])
            elif "prompt" in rec and "completion" in rec:
                prompt, completion = str(rec["prompt"]), str(rec["completion"])
            elif "text" in rec:
                prompt, completion = "", str(rec["text"])
            else:
                raise ValueError(f"{path}:{ln}: want prompt+completion, text, or messages")
            p = tokenizer.encode(prompt) if prompt else []
            c = tokenizer.encode(completion)
            eos = tokenizer.special_tokens.eos
            if eos is not None and eos >= 0:
                c = c + [eos]
            toks = (p + c)[:max_seq_len]
            if len(toks) - len(p) < 1 or len(toks) < 2:
                continue  # nothing left to learn after truncation
            out.append(Example(toks, max(1, len(p))))
    if not out:
        raise ValueError(f"{path}: no usable examples")
    return out


def batch_loss(model: LoraModel, batch: Sequence[Example]) -> torch.Tensor:
    """Mean next-token cross-entropy over the target positions of a right-padded batch."""
    S = max(len(e.tokens) for e in batch)
    toks = torch.zeros(len(batch), S, dtype=torch.int64)
    tgt = torch.full((len(batch), S), -100, dtype=torch.int64)
    for b, e in enumerate(batch):
        n = len(e.tokens)
        toks[b, :n] = torch.tensor(e.tokens)
        tgt[b, e.loss_from - 1 : n - 1] = torch.tensor(e.tokens[e.loss_from :])  # position p predicts token p + 1
    logits = model(toks)
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), tgt.reshape(-1), ignore_index=-100)


# --------------------------------------------------------------------------- preference pairs (DPO)


@dataclass
class PreferencePair:
    chosen: Example
    rejected: Example


def load_preference_pairs(path: str, tokenizer, max_seq_len: int) -> List[PreferencePair]:
    """JSON lines ``{"prompt": ..., "chosen": ..., "rejected": ...}``."""
    out: List[PreferencePair] = []
    eos = tokenizer.special_tokens.eos
    tail = [eos] if eos is not None and eos >= 0 else []
    with open(path) as f:
        for ln, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            if not all(k in rec for k in ("prompt", "chosen", "rejected")):
                raise ValueError(f"{path}:{ln}: want prompt, chosen and rejected")
            p = tokenizer.encode(str(rec["prompt"]))
            pair = []
            for key in ("chosen", "rejected"):
                toks = (p + tokenizer.encode(str(rec[key])) + tail)[:max_seq_len]
                if len(toks) <= len(p):
                    break
                pair.append(Example(toks, max(1, len(p))))
            if len(pair) == 2:
                out.append(PreferencePair(*pair))
    if not out:
        raise ValueError(f"{path}: no usable preference pairs")
    return out


def sequence_logprobs(model: "LoraModel", examples: Sequence[Example]) -> torch.Tensor:
    """Sum of the target tokens' log-probabilities of every example, [len(examples)] (right-padded batch)."""
    S = max(len(e.tokens) for e in examples)
    toks = torch.zeros(len(examples), S, dtype=torch.int64)
    tgt = torch.zeros(len(examples), S, dtype=torch.int64)
    mask = torch.zeros(len(examples), S)
    for b, e in enumerate(examples):
        n = len(e.tokens)
        toks[b, :n] = torch.tensor(e.tokens)
        tgt[b, e.loss_from - 1 : n - 1] = torch.tensor(e.tokens[e.loss_from :])
        mask[b, e.loss_from - 1 : n - 1] = 1.0
    lp = torch.log_softmax(model(toks), dim=-1).gather(2, tgt[:, :, None]).squeeze(2)
    return (lp * mask).sum(dim=1)


def dpo_loss(model: "LoraModel", pairs: Sequence[PreferencePair], beta: float = 0.1) -> Tuple[torch.Tensor, float]:
    """Direct preference optimisation (Rafailov et al. 2023): -log sigmoid(beta * ((pi_w - pi_l) - (ref_w - ref_l))) with
    the adapter-free base model as the reference policy.  Returns (loss, fraction of pairs the policy already ranks right)."""
    ex = [p.chosen for p in pairs] + [p.rejected for p in pairs]
    pol = sequence_logprobs(model, ex)
    model.adapters_on = False
    try:
        with torch.no_grad():
            ref = sequence_logprobs(model, ex)
    finally:
        model.adapters_on = True
    n = len(pairs)
    margin = (pol[:n] - pol[n:]) - (ref[:n] - ref[n:])
    return -F.logsigmoid(beta * margin).mean(), float((margin > 0).float().mean())


# --------------------------------------------------------------------------- training


@dataclass
class TrainState:
    step: int = 0
    round: int = 0
    losses: List[float] = field(default_factory=list)


class Trainer:
    def __init__(self, model: LoraModel, cfg: TrainConfig):
        self.model, self.cfg = model, cfg
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.opt = torch.optim.AdamW(self.params, lr=cfg.lr, weight_decay=cfg.weight_decay)
        self.state = TrainState()
        self.rng = np.random.default_rng(cfg.seed)

    def _lr(self, step: int) -> float:
        c = self.cfg
        if c.warmup_steps > 0 and step < c.warmup_steps:
            return c.lr * (step + 1) / c.warmup_steps
        return c.lr

    def train(self, examples: Sequence, steps: Optional[int] = None, checkpoint_dir: Optional[str] = None,
              dpo_beta: Optional[float] = None) -> List[float]:
        """``examples``: supervised :class:`Example` s, or with ``dpo_beta`` :class:`PreferencePair` s."""
        c = self.cfg
        self.model.train()
        done: List[float] = []
        for _ in range(steps if steps is not None else c.steps):
            idx = self.rng.choice(len(examples), size=min(c.batch_size, len(examples)), replace=False)
            for gp in self.opt.param_groups:
                gp["lr"] = self._lr(self.state.step)
            self.opt.zero_grad(set_to_none=True)
            batch = [examples[i] for i in idx]
            loss = dpo_loss(self.model, batch, dpo_beta)[0] if dpo_beta is not None else batch_loss(self.model, batch)
            loss.backward()
            if c.grad_clip > 0:
                torch.nn.utils.clip_grad_norm_(self.params, c.grad_clip)
            self.opt.step()
            self.state.step += 1
            self.state.losses.append(float(loss.detach()))
            done.append(float(loss.detach()))
            if checkpoint_dir and c.checkpoint_every and self.state.step % c.checkpoint_every == 0:
                self.save_checkpoint(os.path.join(checkpoint_dir, f"step-{self.state.step:06d}"))
        self.model.eval()
        return done

    # adapter + optimizer + counters + the sampling stream: resuming continues the exact run
    def save_checkpoint(self, directory: str) -> str:
        self.model.save_adapter(directory)
        torch.save({"optimizer": self.opt.state_dict(), "state": asdict(self.state), "rng": self.rng.bit_generator.state,
                    "train_config": asdict(self.cfg), "lora": asdict(self.model.lora)},
                   os.path.join(directory, "trainer_state.pt"))
        return directory

    def load_checkpoint(self, directory: str) -> None:
        self.model.load_adapter(directory)
        blob = torch.load(os.path.join(directory, "trainer_state.pt"), weights_only=False)
        if blob["lora"]["r"] != self.model.lora.r or tuple(blob["lora"]["targets"]) != tuple(self.model.lora.targets):
            raise ValueError("the checkpoint was trained with a different LoRA rank or target set")
        self.opt.load_state_dict(blob["optimizer"])
        self.state = TrainState(**blob["state"])
        self.rng.bit_generator.state = blob["rng"]


def generate_with_adapter(model: LoraModel, prompt_tokens: Sequence[int], max_new: int, eos: Optional[int] = None) -> List[int]:
    """Greedy continuation with the trainer's own forward (whole-sequence recompute per token: for the short texts of
    self-training rounds and tests, not a serving path)."""
    toks = list(prompt_tokens)
    out: List[int] = []
    model.eval()
    with torch.no_grad():
        for _ in range(max_new):
            nxt = int(model(torch.tensor([toks]))[0, -1].argmax())
            out.append(nxt)
            toks.append(nxt)
            if eos is not None and nxt == eos:
                break
    return out


def self_train_round(trainer: Trainer, tokenizer, prompts: Sequence[str], max_new: int, steps: int, min_tokens: int = 4,
                     must_match: Optional[str] = None, log_path: Optional[str] = None) -> Dict[str, object]:
    """One round of self-training: the current model answers ``prompts`` greedily, answers that are long enough (and match
    ``must_match`` if given) become training examples, and the adapter trains on them for ``steps`` steps.  The accepted
    pairs are appended to ``log_path`` as JSON lines."""
    import re

    eos = tokenizer.special_tokens.eos
    accepted: List[Example] = []
    records = []
    for p in prompts:
        ids = tokenizer.encode(p)
        gen = generate_with_adapter(trainer.model, ids, max_new, eos)
        body = [t for t in gen if t != eos]
        text = tokenizer.decode_without_special_tokens(body)
        if len(body) < min_tokens or (must_match and not re.search(must_match, text)):
            continue
        accepted.append(Example(ids + gen, len(ids)))
        records.append({"prompt": p, "completion": text})
    losses = trainer.train(accepted, steps) if accepted else []
    trainer.state.round += 1
    if log_path and records:
        with open(log_path, "a") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")
    return {"round": trainer.state.round, "generated": len(prompts), "accepted": len(accepted),
            "loss_first": losses[0] if losses else None, "loss_last": losses[-1] if losses else None}


# --------------------------------------------------------------------------- command line


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oxidize finetune", description="LoRA / QLoRA fine-tuning of a GGUF checkpoint on the CPU")
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", help="JSONL training set")
    ap.add_argument("--output", required=True, help="directory for adapters, checkpoints and logs")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--lr", type=float, default=2e-4)
    ap.add_argument("--warmup-steps", type=int, default=0)
    ap.add_argument("--max-seq-len", type=int, default=512)
    ap.add_argument("--rank", type=int, default=8)
    ap.add_argument("--alpha", type=float, default=16.0)
    ap.add_argument("--dropout", type=float, default=0.0)
    ap.add_argument("--targets", default="q_proj,v_proj", help=",".join(TARGETS))
    ap.add_argument("--qlora", action="store_true", help="keep the quantized base encoded; decode each matrix per use")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--checkpoint-every", type=int, default=0)
    ap.add_argument("--resume-from", help="checkpoint directory written by an earlier run")
    ap.add_argument("--self-train-rounds", type=int, default=0)
    ap.add_argument("--prompts", help="text file, one prompt per line (self-training)")
    ap.add_argument("--self-train-max-new", type=int, default=64)
    ap.add_argument("--self-train-match", help="regular expression an answer must match to be kept")
    ap.add_argument("--dpo-data", help="JSONL of prompt / chosen / rejected: preference training (DPO) after any --data pass")
    ap.add_argument("--dpo-beta", type=float, default=0.1)
    ap.add_argument("--merge-output", help="also write the base with the adapter folded in, as a GGUF")
    a = ap.parse_args(argv)
    try:
        from ..formats.tokenizer import chat_template_from_metadata, load_tokenizer_from_metadata

        g = load_gguf(a.model)
        cfg: ModelConfig = config_from_gguf(g)
        weights = load_weights(g, cfg, "cpu", torch.float32)
        tok = load_tokenizer_from_metadata(g.metadata)
        lora = LoraConfig(a.rank, a.alpha, a.dropout, tuple(t for t in a.targets.split(",") if t))
        tc = TrainConfig(a.steps, a.batch_size, a.lr, 0.0, a.warmup_steps, a.max_seq_len, 1.0, a.seed, a.qlora, a.checkpoint_every)
        trainer = Trainer(LoraModel(weights, lora, a.qlora, a.seed), tc)
        if a.resume_from:
            trainer.load_checkpoint(a.resume_from)
            print(f"resumed from {a.resume_from} at step {trainer.state.step}, round {trainer.state.round}")
        os.makedirs(a.output, exist_ok=True)
        if a.data:
            ex = load_examples(a.data, tok, chat_template_from_metadata(g.metadata), a.max_seq_len)
            losses = trainer.train(ex, a.steps, a.output)
            print(f"trained {len(losses)} steps on {len(ex)} examples: loss {losses[0]:.4f} -> {losses[-1]:.4f}")
            trainer.save_checkpoint(os.path.join(a.output, f"round-{trainer.state.round:04d}"))
        if a.dpo_data:
            pairs = load_preference_pairs(a.dpo_data, tok, a.max_seq_len)
            losses = trainer.train(pairs, a.steps, a.output, dpo_beta=a.dpo_beta)
            trainer.state.round += 1
            print(f"preference training, {len(losses)} steps on {len(pairs)} pairs: loss {losses[0]:.4f} -> {losses[-1]:.4f}")
            trainer.save_checkpoint(os.path.join(a.output, f"round-{trainer.state.round:04d}"))
        if a.self_train_rounds:
            if not a.prompts:
                raise ValueError("--self-train-rounds needs --prompts")
            with open(a.prompts) as f:
                prompts = [l.strip() for l in f if l.strip()]
            for _ in range(a.self_train_rounds):
                rep = self_train_round(trainer, tok, prompts, a.self_train_max_new, a.steps, must_match=a.self_train_match,
                                       log_path=os.path.join(a.output, "self_train.jsonl"))
                print(json.dumps(rep))
                trainer.save_checkpoint(os.path.join(a.output, f"round-{trainer.state.round:04d}"))
        final = trainer.model.save_adapter(os.path.join(a.output, "adapter"))
        print(f"adapter: {final}")
        if a.merge_output:
            from .lora import merge_lora_gguf

            merge_lora_gguf(a.model, final, a.merge_output)
            print(f"merged checkpoint: {a.merge_output}")
    except (ValueError, OSError, NotImplementedError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
