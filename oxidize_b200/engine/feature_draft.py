"""Hidden-conditioned draft model ("DFlash"-style; the same mechanism serves EAGLE-3-style heads): a small decoder whose
attention also sees a *context entry* computed from the target model's hidden states.

Architecture as in the reference (``oxidize-core/src/model/dflash.rs``: config ``:11-27``, tensor names ``:860-925``,
forward ``:1119-1404``): the hidden states of a few target layers at the last verified token are concatenated, projected
by ``fc`` (+ bias) and normalised (``hidden_norm``) into a context vector.  Every draft layer projects that vector with
its own K / V projections (K normalised and rotated like a token's key) and appends the pair to its cache in front of the
token's own entry; the token stream itself is an ordinary pre-norm decoder (per-head QK-norm, rotary embedding, SwiGLU).
Embedding table and output head come from the draft file or, when it has none, from the target.

Here the draft runs on the engine's operators and a paged cache of its own, batched over sequences; tokens the draft has
not seen yet (the prompt, tokens the target corrected) are caught up in one multi-row pass per round.  Verification by
the target keeps the output exact whatever the draft proposes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq

import numpy as np
import torch

from .. import ops
from ..formats.gguf import GGUFFile, load_gguf
from ..models.config import ModelConfig
from ..models.transformer import BatchMeta, RopeState
from ..models.weights import GGUFWeightSource, LayerWeights, LinearWeight, QTensor, _load_layer
from ..ops import ref as opref
from .kv_pool import KVCache, KVCacheSpec, make_block_pool
from .scheduler import Sequence

PAGE = 16


@dataclass
class FeatureDraftConfig:
    model: ModelConfig
    target_layer_ids: List[int] = field(default_factory=list)
    block_size: int = 16
    mask_token_id: int = 0


def feature_draft_config(g: GGUFFile, n_target_layers: int) -> FeatureDraftConfig:
    """Metadata under the file's architecture name, ``dflash`` or ``dflash-draft``, in either naming scheme (``hidden_size``
    / ``embedding_length`` ...), as the reference reads it (``dflash.rs:54-200``)."""
    spaces = [g.architecture, "dflash", "dflash-draft"]

    def get(*names, default=None):
        for ns in spaces:
            for n in names:
                v = g.metadata.get(f"{ns}.{n}")
                if v is not None:
                    return v
        return default

    fc = next((g.tensors[n] for n in ("fc.weight", "dflash_fc.weight", "model.fc.weight") if n in g.tensors), None)
    if fc is None:
        raise ValueError("not a hidden-conditioned draft file: no fc.weight")
    hidden = int(get("hidden_size", "embedding_length", default=fc.shape[0]))
    heads = int(get("num_attention_heads", "attention.head_count", default=32))
    qn = g.tensors.get("blk.0.attn_q_norm.weight")
    head_dim = int(get("head_dim", "attention.key_length", default=(qn.shape[-1] if qn is not None else hidden // heads)))
    layers = int(get("num_hidden_layers", "block_count", default=8))
    ffn = g.tensors.get("blk.0.ffn_gate.weight")
    cfg = ModelConfig(arch="llama", name="feature-draft", hidden_size=hidden, n_layers=layers, n_heads=heads,
                      n_kv_heads=int(get("num_key_value_heads", "attention.head_count_kv", default=heads)), head_dim=head_dim,
                      ffn_size=int(get("intermediate_size", "feed_forward_length", default=(ffn.shape[0] if ffn is not None else 0))),
                      rms_eps=float(get("rms_norm_eps", "attention.layer_norm_rms_epsilon", default=1e-5)),
                      rope_theta=float(get("rope_theta", "rope.freq_base", default=10000.0)),
                      vocab_size=int(get("vocab_size", default=0)), qk_norm=qn is not None)
    ids = get("target_layer_ids", default=None)
    n_feat = fc.shape[1] // hidden if fc.shape[1] % hidden == 0 else 0
    if ids is None:
        # evenly spread over the target's depth, first and last layers left out (the reference's default spacing)
        n = max(1, n_feat)
        ids = [1 + i * max(1, (n_target_layers - 3)) // max(1, n - 1) for i in range(n)] if n > 1 else [n_target_layers // 2]
    ids = [int(i) for i in ids]
    if any(i < 0 or i >= n_target_layers for i in ids):
        raise ValueError(f"target_layer_ids {ids} outside the target's {n_target_layers} layers")
    return FeatureDraftConfig(cfg, ids, int(get("block_size", default=16)), int(get("mask_token_id", default=0)))


@dataclass
class FeatureDraftWeights:
    cfg: FeatureDraftConfig
    fc: QTensor
    fc_bias: Optional[torch.Tensor]
    hidden_norm: Optional[torch.Tensor]
    layers: List[LayerWeights]
    out_norm: torch.Tensor
    embed: Optional[QTensor]
    lm_head: Optional[LinearWeight]


def load_feature_draft(path: str, device, act_dtype: torch.dtype, n_target_layers: int) -> FeatureDraftWeights:
    g = load_gguf(path)
    fcfg = feature_draft_config(g, n_target_layers)
    src = GGUFWeightSource(g, device, act_dtype)

    def first(*names):
        return next((n for n in names if src.has(n)), None)

    layers = []
    for i in range(fcfg.model.n_layers):
        if not src.has(f"blk.{i}.ffn_norm.weight") and src.has(f"blk.{i}.post_attention_norm.weight"):
            # files converted with the norm in front of the MLP under its original name
            g.tensors[f"blk.{i}.ffn_norm.weight"] = g.tensors.pop(f"blk.{i}.post_attention_norm.weight")
        layers.append(_load_layer(src, fcfg.model, i, 0, 1, 0, 1))
    fc_name = first("fc.weight", "dflash_fc.weight", "model.fc.weight")
    hn = first("hidden_norm.weight", "dflash_hidden_norm.weight", "model.hidden_norm.weight")
    on = first("output_norm.weight", "norm.weight", "model.norm.weight")
    if on is None:
        raise ValueError("draft file has no final norm")
    emb = first("token_embd.weight", "model.embed_tokens.weight", "tok_embeddings.weight")
    head = first("output.weight", "lm_head.weight")
    bias = first("fc.bias", "dflash_fc.bias", "model.fc.bias")
    embed = src.matrix(emb) if emb else None
    return FeatureDraftWeights(fcfg, src.matrix(fc_name), src.vector(bias) if bias else None, src.vector(hn) if hn else None,
                               layers, src.vector(on), embed,
                               LinearWeight([src.matrix(head)]) if head else (LinearWeight([embed]) if embed is not None else None))


@dataclass
class _SeqState:
    blocks: List[int] = field(default_factory=list)
    seen: int = 0  # target tokens whose entries are in the cache
    entries: int = 0  # cache entries in use (a token with a context entry takes two)
    entry_end: List[int] = field(default_factory=list)  # entry_end[t] = entries after token t went in


class FeatureDraftProposer:
    def __init__(self, weights: FeatureDraftWeights, target_model, k: int, max_seqs: int, max_model_len: int):
        self.k, self.w, self.m = k, weights, target_model
        cfg = weights.cfg.model
        dev = target_model.device
        self.cfg, self.dev = cfg, dev
        if cfg.hidden_size != target_model.cfg.hidden_size and (weights.embed is None or weights.lm_head is None):
            raise ValueError("a draft without its own embedding table and head must have the target's hidden size")
        self.embed_table = weights.embed if weights.embed is not None else target_model.w.embed
        self.head = weights.lm_head if weights.lm_head is not None else target_model.w.lm_head
        if self.head.out_features != target_model.cfg.vocab_size:
            raise ValueError(f"draft vocabulary {self.head.out_features} != target vocabulary {target_model.cfg.vocab_size}")
        n_feat = len(weights.cfg.target_layer_ids)
        if weights.fc.in_features != n_feat * target_model.cfg.hidden_size:
            raise ValueError(f"fc expects {weights.fc.in_features} features, the target gives {n_feat} x "
                             f"{target_model.cfg.hidden_size}")
        target_model.capture_layers = list(weights.cfg.target_layer_ids)  # the target now records these layers' outputs
        self.rope = RopeState(opref.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta, None, device=dev), cfg.rope_pairing, 1.0,
                              cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
        self.scale = cfg.head_dim ** -0.5
        # every token can take two entries (its own and a context entry)
        per_seq = (2 * max_model_len + PAGE - 1) // PAGE + 1
        kvd = "bf16" if dev.type == "cuda" else "f32"
        self.kv = KVCache(KVCacheSpec(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, PAGE, kvd), max_seqs * per_seq, dev)
        self.pool = make_block_pool(max_seqs * per_seq, PAGE, enable_prefix_cache=False)
        self.max_blocks = per_seq
        self.state: Dict[int, _SeqState] = {}
        self.features: Dict[int, torch.Tensor] = {}
        self.draft_logits: Dict[int, torch.Tensor] = {}
        self.act = target_model.act_dtype
        self.context_entries = 0  # context entries written so far (a gauge: 0 means the target's features never arrived)

    # ------------------------------------------------------------------ SpecDecoder protocol
    def observe_features(self, seq: Sequence, feats: torch.Tensor) -> None:
        """Concatenated hidden states of the target's capture layers at the last accepted token."""
        self.features[seq.seq_id] = feats

    def release(self, seq: Sequence) -> None:
        st = self.state.pop(seq.seq_id, None)
        if st is not None:
            self.pool.release_all(st.blocks)
        self.features.pop(seq.seq_id, None)
        self.draft_logits.pop(seq.seq_id, None)

    def rollback(self, seq: Sequence, n_valid_tokens: int) -> None:
        st = self.state.get(seq.seq_id)
        if st is not None and st.seen > n_valid_tokens:
            st.seen = n_valid_tokens
            st.entry_end = st.entry_end[:n_valid_tokens]
            st.entries = st.entry_end[-1] if st.entry_end else 0

    # ------------------------------------------------------------------ forward
    def _context(self, feats: torch.Tensor) -> torch.Tensor:
        c = ops.linear(feats.to(self.act), self.w.fc)
        if self.w.fc_bias is not None:
            c = (c.float() + self.w.fc_bias).to(c.dtype)
        return ops.rmsnorm(c, self.w.hidden_norm, self.cfg.rms_eps) if self.w.hidden_norm is not None else c

    def _forward(self, seqs: Seq[Sequence], tokens: List[List[int]], first_pos: List[int],
                 ctx: List[Optional[torch.Tensor]]) -> torch.Tensor:
        """Feed ``tokens[i]`` (consecutive positions from ``first_pos[i]``) of sequence i; with ``ctx[i]`` given (only for
        single-token feeds) a context entry goes into the cache in front of the token's.  Returns the final-norm hidden
        state of each sequence's LAST fed token, [len(seqs), hidden]."""
        cfg, dev = self.cfg, self.dev
        i32 = dict(dtype=torch.int32, device=dev)
        tok_ids, pos, slots, is_ctx, q_start, seq_lens = [], [], [], [], [0], []
        for s, toks, p0, c in zip(seqs, tokens, first_pos, ctx):
            st = self.state[s.seq_id]
            n_new = len(toks) + (1 if c is not None else 0)
            while len(st.blocks) * PAGE < st.entries + n_new:
                st.blocks.append(self.pool.allocate())
            e = st.entries
            if c is not None:
                tok_ids.append(toks[0]); pos.append(p0); is_ctx.append(True)
                slots.append(st.blocks[e // PAGE] * PAGE + e % PAGE)
                e += 1
                self.context_entries += 1
            for j, t in enumerate(toks):
                tok_ids.append(t); pos.append(p0 + j); is_ctx.append(False)
                slots.append(st.blocks[e // PAGE] * PAGE + e % PAGE)
                e += 1
                st.entry_end.append(e)
            st.entries = e
            st.seen += len(toks)
            q_start.append(q_start[-1] + len(toks))
            seq_lens.append(e)
        R = len(tok_ids)
        ctx_rows = torch.tensor(is_ctx, dtype=torch.bool, device=dev)
        tok_rows = (~ctx_rows).nonzero(as_tuple=True)[0]
        positions, slot_map = torch.tensor(pos, **i32), torch.tensor(slots, **i32)
        x = ops.embed(torch.tensor(tok_ids, **i32)[tok_rows], self.embed_table, self.act)
        ctx_mat = None
        if bool(ctx_rows.any()):
            ctx_mat = torch.cat([self._context(c[None, :]) for c in ctx if c is not None], dim=0)
        bt = torch.zeros(len(seqs), self.max_blocks, **i32)
        for i, s in enumerate(seqs):
            bl = self.state[s.seq_id].blocks
            bt[i, : len(bl)] = torch.tensor(bl, **i32)
        meta = BatchMeta(torch.tensor(tok_ids, **i32)[tok_rows], positions[tok_rows], slot_map[tok_rows],
                         torch.tensor(q_start, **i32), torch.tensor(seq_lens, **i32), bt, None,
                         max(len(t) for t in tokens), max(seq_lens), len(seqs))
        nq, nkv, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        for li, lw in enumerate(self.w.layers):
            normed = ops.rmsnorm(x, lw.attn_norm, cfg.rms_eps)
            qkv = ops.linear(normed, lw.wqkv)
            if ctx_mat is not None:
                # context rows: K and V straight from the context vector (their query part is computed and dropped)
                rows = torch.empty(R, qkv.shape[1], dtype=qkv.dtype, device=dev)
                rows[tok_rows] = qkv
                rows[ctx_rows] = ops.linear(ctx_mat, lw.wqkv)
            else:
                rows = qkv
            q = ops.qk_rope_kv_write(rows, positions, slot_map, self.kv, li, self.rope, lw.q_norm, lw.k_norm, cfg.rms_eps)
            q = q[tok_rows] if ctx_mat is not None else q
            attn = ops.paged_attention(q.contiguous(), self.kv, li, meta, self.scale, 0)
            x = x + ops.linear(attn.reshape(attn.shape[0], nq * hd), lw.wo)
            h = ops.rmsnorm(x, lw.ffn_norm, cfg.rms_eps)
            x = x + ops.linear(ops.silu_mul(ops.linear(h, lw.w_gate_up)), lw.w_down)
        last = torch.tensor([q_start[i + 1] - 1 for i in range(len(seqs))], dtype=torch.int64, device=dev)
        return ops.rmsnorm(x.index_select(0, last), self.w.out_norm, cfg.rms_eps)

    def propose(self, seqs: List[Sequence]) -> Dict[int, List[int]]:
        drafts: Dict[int, List[int]] = {s.seq_id: [] for s in seqs}
        if not seqs:
            return drafts
        for s in seqs:
            self.state.setdefault(s.seq_id, _SeqState())
        # catch-up: every token the draft has not seen except the newest one, in one multi-row pass
        behind = [s for s in seqs if len(s.all_tokens) - 1 > self.state[s.seq_id].seen]
        if behind:
            self._forward(behind, [s.all_tokens[self.state[s.seq_id].seen : -1] for s in behind],
                          [self.state[s.seq_id].seen for s in behind], [None] * len(behind))
        toks = [[s.all_tokens[-1]] for s in seqs]
        pos = [len(s.all_tokens) - 1 for s in seqs]
        ctx: List[Optional[torch.Tensor]] = [self.features.get(s.seq_id) for s in seqs]
        sampled = [not s.params.is_greedy for s in seqs]
        rows: Dict[int, List[torch.Tensor]] = {s.seq_id: [] for s, smp in zip(seqs, sampled) if smp}
        for it in range(self.k):
            hidden = self._forward(seqs, toks, pos, ctx)
            logits = ops.linear(hidden, self.head).float()
            if any(sampled):
                from .sampler import probs_from_logits

                nxt = []
                for i, s in enumerate(seqs):
                    if sampled[i]:
                        # drafts of a sampled request are drawn from the draft's own distribution at the request's temperature
                        p = torch.from_numpy(probs_from_logits(logits[i].cpu().numpy(), s.params.temperature))
                        nxt.append(int(torch.searchsorted(torch.cumsum(p, 0), torch.tensor(s.rng.next())).clamp(max=p.numel() - 1)))
                        rows[s.seq_id].append(logits[i].cpu())
                    else:
                        nxt.append(int(ops.argmax(logits[i : i + 1])[0]))
            else:
                nxt = ops.argmax(logits).tolist()
            for i, s in enumerate(seqs):
                drafts[s.seq_id].append(int(nxt[i]))
            toks = [[int(t)] for t in nxt]
            pos = [p + 1 for p in pos]
            ctx = [None] * len(seqs)  # target features exist for verified tokens only
        for sid, r in rows.items():
            self.draft_logits[sid] = torch.stack(r).to(self.dev)
        # the drafted tokens are not part of the sequence yet: their entries are dropped again (kept ones are re-fed with
        # the catch-up pass of the next round, now possibly with context)
        for s in seqs:
            self.rollback(s, len(s.all_tokens))
        return drafts


# --------------------------------------------------------------------------- EAGLE-3


@dataclass
class Eagle3Weights:
    model: ModelConfig
    extract_layers: List[int]
    norm_before_residual: bool
    fc: QTensor
    layer: LayerWeights  # q / k / v take [norm(embedding) ; norm(g)]: 2 x hidden inputs
    attn_norm_2: torch.Tensor
    out_norm: torch.Tensor
    head: LinearWeight  # [draft vocabulary, hidden]
    d2t: Optional[torch.Tensor]  # target id = draft id + d2t[draft id]
    embed: Optional[QTensor]


def default_eagle3_extract_layers(n_target_layers: int) -> List[int]:
    """Early, middle and late layer of the target (the reference's default, ``eagle3.rs:266-276``)."""
    return [0, 0, 0] if n_target_layers < 4 else [2, n_target_layers // 2, max(0, n_target_layers - 3)]


def load_eagle3(path: str, device, act_dtype: torch.dtype, n_target_layers: int, target_hidden: int) -> Eagle3Weights:
    """EAGLE-3 draft head from a GGUF file (``eagle3.rs:663-770``: ``fc``, ``d2t``, one block ``blk.0.*`` with a second
    input norm ``attn_norm_2``, ``output_norm``, ``output`` over the draft vocabulary, optional ``token_embd``)."""
    g = load_gguf(path)
    spaces = [g.architecture, "eagle3"]

    def get(*names, default=None):
        for ns in spaces:
            for n in names:
                v = g.metadata.get(f"{ns}.{n}")
                if v is not None:
                    return v
        return default

    if "fc.weight" not in g.tensors or "blk.0.attn_norm_2.weight" not in g.tensors:
        raise ValueError("not an EAGLE-3 draft file: fc.weight / blk.0.attn_norm_2.weight missing")
    fc = g.tensors["fc.weight"]
    hidden = int(get("hidden_size", "embedding_length", default=fc.shape[0]))
    heads = int(get("num_attention_heads", "attention.head_count", default=32))
    q = g.tensors["blk.0.attn_q.weight"]
    head_dim = int(get("head_dim", "attention.key_length", default=q.shape[0] // heads))
    kvh = int(get("num_key_value_heads", "attention.head_count_kv", default=g.tensors["blk.0.attn_k.weight"].shape[0] // head_dim))
    cfg = ModelConfig(arch="llama", name="eagle3", hidden_size=hidden, n_layers=1, n_heads=heads, n_kv_heads=kvh, head_dim=head_dim,
                      ffn_size=int(g.tensors["blk.0.ffn_gate.weight"].shape[0]),
                      rms_eps=float(get("rms_norm_eps", "attention.layer_norm_rms_epsilon", default=1e-5)),
                      rope_theta=float(get("rope_theta", "rope.freq_base", default=10000.0)),
                      vocab_size=int(g.tensors["output.weight"].shape[0]))
    layers = get("extract_layers", "target_layers", default=None)
    layers = [int(i) for i in layers] if layers is not None else default_eagle3_extract_layers(n_target_layers)
    if any(i < 0 or i >= n_target_layers for i in layers):
        raise ValueError(f"extract_layers {layers} outside the target's {n_target_layers} layers")
    if fc.shape[1] != len(layers) * target_hidden:
        raise ValueError(f"fc expects {fc.shape[1]} features, the target gives {len(layers)} x {target_hidden}")
    src = GGUFWeightSource(g, device, act_dtype)
    d2t = None
    if src.has("d2t"):
        d2t = torch.from_numpy(np.asarray(g.tensor("d2t")).astype(np.int64).reshape(-1).copy()).to(src.device)
    return Eagle3Weights(cfg, layers, bool(get("norm_before_residual", default=False)), src.matrix("fc.weight"),
                         _load_layer(src, cfg, 0, 0, 1, 0, 1), src.vector("blk.0.attn_norm_2.weight"),
                         src.vector("output_norm.weight"), LinearWeight([src.matrix("output.weight")]), d2t,
                         src.matrix("token_embd.weight") if src.has("token_embd.weight") else None)


@dataclass
class _EagleState:
    blocks: List[int] = field(default_factory=list)
    first: int = -1  # index (in the sequence) of the first token that has a cache entry
    entries: int = 0


class Eagle3Proposer:
    """EAGLE-3 drafting (``eagle3.rs:444-660``): ``g = fc(target features)`` at the last verified position; every draft step
    feeds ``[norm(embed(token)) ; norm_2(g)]`` to one decoder block whose output becomes the next step's ``g`` and, through
    ``output_norm`` and the draft head, the next token (mapped to the target vocabulary by ``d2t``).  The block's cache holds
    the tokens fed so far in this and earlier rounds (verified ones only survive a round); the prompt itself is not
    replayed through the draft."""

    def __init__(self, weights: Eagle3Weights, target_model, k: int, max_seqs: int, max_model_len: int):
        self.k, self.w, self.m = k, weights, target_model
        cfg = weights.model
        dev = target_model.device
        self.cfg, self.dev, self.act = cfg, dev, target_model.act_dtype
        if weights.embed is None and cfg.hidden_size != target_model.cfg.hidden_size:
            raise ValueError("a draft head without its own embedding table must have the target's hidden size")
        self.embed_table = weights.embed if weights.embed is not None else target_model.w.embed
        target_model.capture_layers = list(weights.extract_layers)
        self.rope = RopeState(opref.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta, None, device=dev), cfg.rope_pairing, 1.0,
                              cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
        self.scale = cfg.head_dim ** -0.5
        per_seq = (max_model_len + PAGE - 1) // PAGE + 1
        kvd = "bf16" if dev.type == "cuda" else "f32"
        self.kv = KVCache(KVCacheSpec(1, cfg.n_kv_heads, cfg.head_dim, PAGE, kvd), max_seqs * per_seq, dev)
        self.pool = make_block_pool(max_seqs * per_seq, PAGE, enable_prefix_cache=False)
        self.max_blocks = per_seq
        self.state: Dict[int, _EagleState] = {}
        self.features: Dict[int, torch.Tensor] = {}
        self.draft_logits: Dict[int, torch.Tensor] = {}
        self.vocab = target_model.cfg.vocab_size

    def observe_features(self, seq: Sequence, feats: torch.Tensor) -> None:
        self.features[seq.seq_id] = feats

    def release(self, seq: Sequence) -> None:
        st = self.state.pop(seq.seq_id, None)
        if st is not None:
            self.pool.release_all(st.blocks)
        self.features.pop(seq.seq_id, None)
        self.draft_logits.pop(seq.seq_id, None)

    def rollback(self, seq: Sequence, n_valid_tokens: int) -> None:
        st = self.state.get(seq.seq_id)
        if st is not None and st.first >= 0:
            st.entries = max(0, min(st.entries, n_valid_tokens - st.first))

    def _step(self, seqs: Seq[Sequence], toks: List[int], pos: List[int], g: torch.Tensor):
        """One decoder step for one token per sequence; returns (hidden [B, h], logits over the draft vocabulary)."""
        cfg, dev, lw = self.cfg, self.dev, self.w.layer
        i32 = dict(dtype=torch.int32, device=dev)
        B = len(seqs)
        slots, lens = [], []
        bt = torch.zeros(B, self.max_blocks, **i32)
        for i, s in enumerate(seqs):
            st = self.state[s.seq_id]
            while len(st.blocks) * PAGE < st.entries + 1:
                st.blocks.append(self.pool.allocate())
            slots.append(st.blocks[st.entries // PAGE] * PAGE + st.entries % PAGE)
            st.entries += 1
            lens.append(st.entries)
            bt[i, : len(st.blocks)] = torch.tensor(st.blocks, **i32)
        tok_t, pos_t = torch.tensor(toks, **i32), torch.tensor(pos, **i32)
        e = ops.rmsnorm(ops.embed(tok_t, self.embed_table, self.act), lw.attn_norm, cfg.rms_eps)
        gn = ops.rmsnorm(g, self.w.attn_norm_2, cfg.rms_eps)
        residual = gn if self.w.norm_before_residual else g
        qkv = ops.linear(torch.cat([e, gn], dim=-1), lw.wqkv)
        q = ops.qk_rope_kv_write(qkv, pos_t, torch.tensor(slots, **i32), self.kv, 0, self.rope, None, None, cfg.rms_eps)
        meta = BatchMeta(tok_t, pos_t, torch.tensor(slots, **i32), torch.arange(B + 1, **i32), torch.tensor(lens, **i32), bt,
                         None, 1, max(lens), B)
        attn = ops.paged_attention(q.contiguous(), self.kv, 0, meta, self.scale, 0)
        hidden = ops.linear(attn.reshape(B, -1), lw.wo) + residual
        h2 = ops.rmsnorm(hidden, lw.ffn_norm, cfg.rms_eps)
        hidden = hidden + ops.linear(ops.silu_mul(ops.linear(h2, lw.w_gate_up)), lw.w_down)
        logits = ops.linear(ops.rmsnorm(hidden, self.w.out_norm, cfg.rms_eps), self.w.head).float()
        return hidden, logits

    def _to_target_vocab(self, draft_ids: torch.Tensor) -> torch.Tensor:
        return draft_ids if self.w.d2t is None else draft_ids + self.w.d2t[draft_ids.long()].to(draft_ids.dtype)

    def propose(self, seqs: List[Sequence]) -> Dict[int, List[int]]:
        drafts: Dict[int, List[int]] = {s.seq_id: [] for s in seqs}
        ready = [s for s in seqs if s.seq_id in self.features]
        if not ready:
            return drafts
        g = ops.linear(torch.stack([self.features[s.seq_id] for s in ready]).to(self.act), self.w.fc)
        for s in ready:
            st = self.state.setdefault(s.seq_id, _EagleState())
            n = len(s.all_tokens)
            if st.first < 0 or st.first + st.entries < n - 1 - 1:
                # nothing cached yet, or more than one verified token was never fed: start the cache at the newest token
                st.first, st.entries = n - 1, 0
        # a verified token that was never fed (the last draft of a fully accepted round) goes in first, with this round's g
        gap = [s for s in ready if self.state[s.seq_id].first + self.state[s.seq_id].entries == len(s.all_tokens) - 2]
        if gap:
            idx = [ready.index(s) for s in gap]
            self._step(gap, [s.all_tokens[-2] for s in gap], [len(s.all_tokens) - 2 for s in gap], g[idx])
        toks = [s.all_tokens[-1] for s in ready]
        pos = [len(s.all_tokens) - 1 for s in ready]
        sampled = [not s.params.is_greedy for s in ready]
        rows: Dict[int, List[torch.Tensor]] = {s.seq_id: [] for s, smp in zip(ready, sampled) if smp}
        for _ in range(self.k):
            g, logits = self._step(ready, toks, pos, g)
            nxt = torch.argmax(logits, dim=-1)
            if any(sampled):
                from .sampler import probs_from_logits

                for i, s in enumerate(ready):
                    if sampled[i]:
                        full = torch.full((self.vocab,), float("-inf"))
                        ids = self._to_target_vocab(torch.arange(logits.shape[1], device=self.dev)).cpu()
                        full[ids] = logits[i].cpu()
                        p = torch.from_numpy(probs_from_logits(full.numpy(), s.params.temperature))
                        t = int(torch.searchsorted(torch.cumsum(p, 0), torch.tensor(s.rng.next())).clamp(max=p.numel() - 1))
                        nxt[i] = int((ids == t).nonzero()[0]) if bool((ids == t).any()) else nxt[i]
                        rows[s.seq_id].append(full)
            tgt = self._to_target_vocab(nxt)
            for i, s in enumerate(ready):
                drafts[s.seq_id].append(int(tgt[i]))
            toks = [int(t) for t in tgt]
            pos = [p + 1 for p in pos]
        for sid, r in rows.items():
            self.draft_logits[sid] = torch.stack(r).to(self.dev)
        for s in ready:
            self.rollback(s, len(s.all_tokens))  # drafted tokens are not verified yet
        return drafts
