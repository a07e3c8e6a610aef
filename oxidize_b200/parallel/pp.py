"""Pipeline parallelism: contiguous layer ranges per stage, activations handed from stage to
stage with point-to-point sends (NCCL on GPUs, gloo on CPU ranks).

The reference's one real multi-process path is a two-node pipeline over TCP: the head runs layers
``[0, L/2)`` and ships an f16 hidden state per position, the tail runs the rest plus the final norm,
lm_head and argmax and ships the token back (``oxidize-cli/src/pipeline.rs:1-23,223-259,302,471``);
its mesh variant splits layers contiguously with the remainder spread over the first stages
(``oxidize-core/src/mesh/sharding.rs:75-91``).  Here the same shape generalises to N stages and to
whole micro-batches: each stage loads only its own layers, the wire format is one contiguous tensor
``[tokens, hidden]`` (+ residual) per micro-batch, and sends are issued asynchronously so that a
stage starts the next micro-batch while its previous output is still on the link.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def split_layers(n_layers: int, n_stages: int) -> List[Tuple[int, int]]:
    """Contiguous ranges; the first ``n_layers % n_stages`` stages take one extra layer."""
    if n_stages < 1 or n_stages > max(n_layers, 1):
        raise ValueError("need 1 <= stages <= layers")
    base, rem = divmod(n_layers, n_stages)
    out, s = [], 0
    for i in range(n_stages):
        e = s + base + (1 if i < rem else 0)
        out.append((s, e))
        s = e
    return out


@dataclass
class StageIO:
    """Tensor hand-off between neighbouring stages and the token broadcast from the last stage.

    ``rank`` / ``world`` count pipeline stages.  With tensor parallelism inside every stage the job has
    ``world * tp_size`` processes laid out stage-major (global rank = stage * tp_size + tp_rank): a process talks to
    the process with the same ``tp_rank`` in the neighbouring stage, and ``group`` (the processes that share this
    ``tp_rank``) carries the token broadcast."""

    rank: int
    world: int
    group: Optional[object] = None
    tp_size: int = 1
    tp_rank: int = 0

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.world - 1

    def _global(self, stage: int) -> int:
        return stage * self.tp_size + self.tp_rank

    def send_next(self, t: torch.Tensor):
        return dist.isend(t.contiguous(), self._global(self.rank + 1))

    def recv_prev(self, shape, dtype, device) -> torch.Tensor:
        buf = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(buf, self._global(self.rank - 1))
        return buf

    def send_tokens_to_first(self, toks: torch.Tensor):
        return dist.isend(toks.contiguous(), self._global(0))

    def recv_tokens_from_last(self, n: int, device) -> torch.Tensor:
        buf = torch.empty(n, dtype=torch.int32, device=device)
        dist.recv(buf, self._global(self.world - 1))
        return buf

    def broadcast_tokens(self, toks: torch.Tensor) -> torch.Tensor:
        """Every stage obtains the tokens the last stage sampled (all stages run the same scheduler and need them)."""
        dist.broadcast(toks, src=self._global(self.world - 1), group=self.group)
        return toks

    def broadcast_object(self, obj):
        box = [obj]
        dist.broadcast_object_list(box, src=self._global(self.world - 1), group=self.group)
        return box[0]


def make_pipeline_groups(world_size: int, rank: int, tp_size: int, pp_size: int):
    """Process groups of a stage-major pp x tp job.  Returns (StageIO or None, tp_group or None); every process must
    call this (group creation is collective)."""
    if tp_size * pp_size != world_size:
        raise ValueError(f"tp_size ({tp_size}) x pp_size ({pp_size}) must equal the number of processes ({world_size})")
    tp_group = pp_group = None
    if pp_size > 1 and tp_size > 1:
        for st in range(pp_size):
            g = dist.new_group([st * tp_size + j for j in range(tp_size)])
            if rank // tp_size == st:
                tp_group = g
        for j in range(tp_size):
            g = dist.new_group([st * tp_size + j for st in range(pp_size)])
            if rank % tp_size == j:
                pp_group = g
    io = StageIO(rank // tp_size, pp_size, pp_group, tp_size, rank % tp_size) if pp_size > 1 else None
    return io, tp_group


class PipelineStage:
    """One stage of an N-stage pipeline over a :class:`Transformer` that holds only this
    stage's layers (``load_weights(..., layer_range=...)``)."""

    def __init__(self, model, io: StageIO):
        self.model = model
        self.io = io
        self.pending: list = []

    def forward_microbatch(self, meta, kv, tie: str = "lowest") -> Optional[torch.Tensor]:
        """Run this stage on one micro-batch.  The first stage embeds, the last one returns the
        sampled tokens (and sends them back to the first stage); the others return ``None``."""
        m, io = self.model, self.io
        T = int(meta.token_ids.shape[0])
        H = m.cfg.hidden_size
        if io.is_first:
            h, residual = m.embed(meta.token_ids), None
        else:
            both = io.recv_prev((2, T, H), m.act_dtype, m.device)
            h, residual = both[0], both[1]
        h, residual = m.run_layers(h, residual, meta, kv)
        if not io.is_last:
            if residual is None:
                residual = torch.zeros_like(h)
            self.pending.append(io.send_next(torch.stack([h, residual])))
            return None
        logits = m.head(h, residual, meta.logits_indices)
        from .. import ops

        toks = ops.argmax(logits, tie)
        if io.world > 1:
            self.pending.append(io.send_tokens_to_first(toks))
        return toks

    def drain(self) -> None:
        for w in self.pending:
            w.wait()
        self.pending = []


def run_pipe_cli(args) -> int:
    """``--pipe-head`` / ``--pipe-tail``: two-stage pipeline between two processes that rendezvous
    on ``--pipe-peer`` / ``--pipe-listen`` (HOST:PORT), greedy decode of ``--pipe-max-tokens``."""
    import os
    import sys

    from ..engine.kv_pool import BlockPool, KVCache, KVCacheSpec
    from ..formats.gguf import load_gguf
    from ..formats.tokenizer import load_tokenizer_from_metadata
    from ..models.config import config_from_gguf
    from ..models.transformer import BatchMeta, Transformer
    from ..models.weights import load_weights

    addr = args.pipe_peer if args.pipe_head else args.pipe_listen
    if not addr or ":" not in addr:
        raise SystemExit("error: --pipe-head needs --pipe-peer HOST:PORT, --pipe-tail needs --pipe-listen HOST:PORT")
    host, port = addr.rsplit(":", 1)
    rank = 0 if args.pipe_head else 1
    os.environ.update({"MASTER_ADDR": host if host not in ("0.0.0.0", "") else "127.0.0.1", "MASTER_PORT": port,
                       "RANK": str(rank), "WORLD_SIZE": "2"})
    use_cuda = torch.cuda.is_available() and args.backend in ("auto", "cuda")
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=2)
    dev = torch.device("cuda", 0) if use_cuda else torch.device("cpu")
    g = load_gguf(args.model)
    cfg = config_from_gguf(g)
    ranges = split_layers(cfg.n_layers, 2)
    act = torch.bfloat16 if use_cuda else torch.float32
    w = load_weights(g, cfg, dev, act, layer_range=ranges[rank])
    stage = PipelineStage(Transformer(w), StageIO(rank, 2))
    tok = load_tokenizer_from_metadata(g.metadata)
    prompt = ([int(x) for x in args.tokens.split(",")] if args.tokens else tok.encode_with_special_tokens(args.prompt))
    n_prompt = torch.tensor([len(prompt)], dtype=torch.int64, device=dev)
    dist.broadcast(n_prompt, 0)
    ids = torch.tensor(prompt if rank == 0 else [0] * int(n_prompt), dtype=torch.int64, device=dev)
    dist.broadcast(ids, 0)
    prompt = ids.tolist()
    max_new = args.pipe_max_tokens
    page = 16
    nblk = (len(prompt) + max_new + page) // page + 1
    kv = KVCache(KVCacheSpec(len(w.layers), cfg.n_kv_heads, cfg.head_dim, page, "bf16" if use_cuda else "f32"), nblk, dev)
    blocks = list(range(nblk))
    i32 = dict(dtype=torch.int32, device=dev)

    def meta_for(tokens: Sequence[int], start: int) -> BatchMeta:
        n = len(tokens)
        pos = torch.arange(start, start + n, **i32)
        return BatchMeta(torch.tensor(tokens, **i32), pos, pos.clone(), torch.tensor([0, n], **i32),
                         torch.tensor([start + n], **i32), torch.tensor([blocks], **i32),
                         torch.tensor([n - 1], **i32), n, start + n, 1)

    out_tokens: List[int] = []
    feed, start = prompt, 0
    for _ in range(max_new):
        toks = stage.forward_microbatch(meta_for(feed, start), kv)
        stage.drain()
        if rank == 0:
            nxt = int(stage.io.recv_tokens_from_last(1, dev)[0])
        else:
            nxt = int(toks[0])
        out_tokens.append(nxt)
        start += len(feed)
        feed = [nxt]
        if nxt == tok.special_tokens.eos:
            break
    if rank == 0:
        print(tok.decode_without_special_tokens(out_tokens))
        print(f"pipeline stats: tokens={len(out_tokens)}", file=sys.stderr)
    dist.barrier()
    dist.destroy_process_group()
    return 0
