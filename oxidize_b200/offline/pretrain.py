"""Train every weight of a small decoder from scratch (or continue from a GGUF) on the CPU and write the result as a GGUF
that the engine serves: the reference's stand-alone GPT trainer (``oxidize-training/src/train_gpt.c``) and the full-weight
mode of its C++ port's trainer (``oxidize-cpp`` "LoRA/full trainer with autograd"), on the fine-tuning module's dense
differentiable forward.

    python -m oxidize_b200.formats.tokenizer_train corpus.txt --vocab-size 1024 --output tok.json
    python -m oxidize_b200.offline.pretrain --corpus corpus.txt --tokenizer tok.json --output tiny.gguf \\
        --hidden 128 --layers 4 --heads 4 --kv-heads 2 --ffn 384 --seq-len 128 --steps 500
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List, Optional

import numpy as np
import torch

from ..formats.gguf import GGUFWriter
from ..models.config import ModelConfig
from ..models.weights import LinearWeight, ModelWeights
from .finetune import Example, LoraConfig, LoraModel, TrainConfig, Trainer


class FullModel(LoraModel):
    """The fine-tuning forward with every matrix, norm and the embedding table as a trainable parameter (no adapters)."""

    def __init__(self, weights: ModelWeights):
        super().__init__(weights, LoraConfig(r=1, targets=()), qlora=False)
        self._params: Dict[int, torch.nn.Parameter] = {}
        self.plist = torch.nn.ParameterList()

        def own(t: torch.Tensor) -> torch.nn.Parameter:
            p = torch.nn.Parameter(t.detach().float().clone())
            self.plist.append(p)
            return p

        w = weights
        self.embed_p = own(w.embed.dense_cache())
        for lw in w.layers:
            for lin in (lw.wqkv, lw.wo, lw.w_gate_up, lw.w_down):
                self._params[id(lin)] = own(torch.cat([p.dense_cache() for p in lin.parts], dim=0))
            lw.attn_norm, lw.ffn_norm = own(lw.attn_norm), own(lw.ffn_norm)
            if lw.q_norm is not None:
                lw.q_norm, lw.k_norm = own(lw.q_norm), own(lw.k_norm)
        w.out_norm = own(w.out_norm)
        self.tied = w.cfg.tie_embeddings
        if not self.tied:
            self._params[id(w.lm_head)] = own(torch.cat([p.dense_cache() for p in w.lm_head.parts], dim=0))

    def _dense(self, w: LinearWeight) -> torch.Tensor:
        if self.tied and w is self.w.lm_head:
            return self.embed_p
        return self._params[id(w)]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        # the parent's forward reads the embedding through the weight container: point it at the parameter for this call
        emb = self.w.embed
        saved = emb._dense
        emb._dense = self.embed_p
        try:
            return super().forward(tokens)
        finally:
            emb._dense = saved

    # ------------------------------------------------------------------ export
    def export_gguf(self, path: str, tokenizer_metadata: Optional[Dict[str, object]] = None, quant: str = "F32") -> str:
        from ..quant import ref as qref
        from ..utils.synth import pick_type, write_config_metadata

        cfg: ModelConfig = self.cfg
        w = GGUFWriter(path, arch=cfg.arch)
        write_config_metadata(w, cfg)
        for k, v in (tokenizer_metadata or {}).items():
            w.add(k, v)
        L = cfg.n_layers

        def put(name: str, t: torch.Tensor, kind: Optional[str] = None, layer: int = 0):
            a = t.detach().float().numpy()
            if kind is None:
                w.add_tensor(name, np.ascontiguousarray(a), a.shape, "F32")
                return
            ty = pick_type(quant, kind, layer, L, a.shape[-1])
            w.add_tensor(name, a if ty == "F32" else qref.quantize(ty, a.reshape(-1)), a.shape, ty)

        put("token_embd.weight", self.embed_p, "token_embd")
        q, kv, f = cfg.q_size, cfg.kv_size, cfg.ffn_size
        for i, lw in enumerate(self.w.layers):
            p = f"blk.{i}"
            put(f"{p}.attn_norm.weight", lw.attn_norm)
            qkv = self._params[id(lw.wqkv)]
            put(f"{p}.attn_q.weight", qkv[:q], "attn_q", i)
            put(f"{p}.attn_k.weight", qkv[q : q + kv], "attn_k", i)
            put(f"{p}.attn_v.weight", qkv[q + kv :], "attn_v", i)
            put(f"{p}.attn_output.weight", self._params[id(lw.wo)], "attn_output", i)
            if lw.q_norm is not None:
                put(f"{p}.attn_q_norm.weight", lw.q_norm)
                put(f"{p}.attn_k_norm.weight", lw.k_norm)
            put(f"{p}.ffn_norm.weight", lw.ffn_norm)
            gu = self._params[id(lw.w_gate_up)]
            put(f"{p}.ffn_gate.weight", gu[:f], "ffn_gate", i)
            put(f"{p}.ffn_up.weight", gu[f:], "ffn_up", i)
            put(f"{p}.ffn_down.weight", self._params[id(lw.w_down)], "ffn_down", i)
        put("output_norm.weight", self.w.out_norm)
        if not self.tied:
            put("output.weight", self._params[id(self.w.lm_head)], "output")
        w.write()
        return path


def windows(ids: List[int], seq_len: int) -> List[Example]:
    """Non-overlapping training windows of ``seq_len`` tokens; every token after a window's first is a target."""
    out = [Example(ids[i : i + seq_len], 1) for i in range(0, len(ids) - 1, seq_len)]
    return [e for e in out if len(e.tokens) >= 2]


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oxidize pretrain", description="Train a small decoder from scratch on the CPU")
    ap.add_argument("--corpus", required=True)
    ap.add_argument("--tokenizer", required=True, help="JSON of GGUF tokenizer metadata (oxidize train-tokenizer)")
    ap.add_argument("--output", required=True, help="GGUF to write")
    ap.add_argument("--init", help="continue from this GGUF instead of a random initialisation")
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--ffn", type=int, default=384)
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--warmup-steps", type=int, default=20)
    ap.add_argument("--weight-decay", type=float, default=0.01)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--quant", default="F32", help="encoding of the exported matrices")
    a = ap.parse_args(argv)
    try:
        from ..formats.tokenizer import load_tokenizer_from_metadata

        with open(a.tokenizer, encoding="utf-8") as f:
            tmd = json.load(f)
        tok = load_tokenizer_from_metadata(tmd)
        with open(a.corpus, encoding="utf-8") as f:
            ids = tok.encode(f.read())
        if a.init:
            from ..formats.gguf import load_gguf
            from ..models.config import config_from_gguf
            from ..models.weights import load_weights

            g = load_gguf(a.init)
            cfg = config_from_gguf(g)
            weights = load_weights(g, cfg, "cpu", torch.float32)
        else:
            from ..utils.synth import synth_weights

            if a.hidden % a.heads or a.heads % a.kv_heads:
                raise ValueError("hidden must divide into heads, heads into kv-heads")
            cfg = ModelConfig(arch="llama", name="pretrained", vocab_size=len(tmd["tokenizer.ggml.tokens"]), hidden_size=a.hidden,
                              n_layers=a.layers, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.hidden // a.heads,
                              ffn_size=a.ffn, context_length=max(a.seq_len, 512), tie_embeddings=True)
            weights = synth_weights(cfg, "cpu", "F32", seed=a.seed)
        model = FullModel(weights)
        data = windows(ids, a.seq_len)
        if not data:
            raise ValueError("the corpus is shorter than two tokens")
        tc = TrainConfig(a.steps, a.batch_size, a.lr, a.weight_decay, a.warmup_steps, a.seq_len, 1.0, a.seed)
        losses = Trainer(model, tc).train(data, a.steps)
        print(f"trained {len(losses)} steps on {len(data)} windows of {a.seq_len} tokens: loss {losses[0]:.4f} -> {losses[-1]:.4f}")
        model.export_gguf(a.output, tmd, a.quant)
        print(f"wrote {a.output}")
    except (ValueError, OSError, NotImplementedError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
