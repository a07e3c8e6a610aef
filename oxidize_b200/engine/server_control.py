"""Serving control plane for tensor-parallel ranks, and the generation-time token mask.

Under TP every rank runs the same engine in lock step.  Rank 0 owns HTTP and the scheduler's
inputs; before each step it broadcasts the requests admitted and aborted since the previous step
so that the followers apply the same mutations and then call ``step()`` themselves.  Scheduling
is deterministic and sampled tokens are identical on all ranks, so nothing else is exchanged.

The suppressed-token set is the reference server's (``oxidize-server/src/runtime/generate.rs:759-790``):
{unk, bos, pad, sep, cls, mask} plus every non-EOS vocabulary entry whose decoded piece starts
with ``[PAD`` or looks like ``<...>``.  Here it becomes a ``-inf`` bias on the lm_head GEMM, i.e.
it is applied inside the kernel epilogue instead of a host loop over the vocabulary.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


def suppressed_generation_tokens(tokenizer, vocab_size: int) -> List[int]:
    st = tokenizer.special_tokens
    out: List[int] = []
    seen = set()
    for t in (st.unk, st.bos, st.pad, st.sep, st.cls, st.mask):
        if t is not None and t not in seen and 0 <= t < vocab_size:
            seen.add(t)
            out.append(t)
    for t in range(min(vocab_size, tokenizer.vocab_size)):
        if t in seen or t == st.eos:
            continue
        try:
            piece = tokenizer.decode([t])
        except Exception:
            continue
        if piece.startswith("[PAD") or (len(piece) >= 2 and piece.startswith("<") and piece.endswith(">")):
            seen.add(t)
            out.append(t)
    return out


def install_suppressed_tokens(llm, token_ids: Sequence[int] = None) -> int:
    """Mask tokens that must never be generated: adds a {0, -inf} bias to this rank's lm_head."""
    if token_ids is None:
        if llm.tokenizer is None:
            return 0
        token_ids = suppressed_generation_tokens(llm.tokenizer, llm.cfg.vocab_size)
    head = llm.weights.lm_head
    n = head.out_features
    v0 = llm.weights.vocab_start
    bias = torch.zeros(n, dtype=torch.float32, device=llm.device)
    local = [t - v0 for t in token_ids if v0 <= t < v0 + n]
    if local:
        bias[torch.tensor(local, dtype=torch.long, device=llm.device)] = float("-inf")
    head.bias = bias
    llm.suppressed_token_ids = list(token_ids)
    return len(token_ids)


class SpmdControl:
    """Leader/follower step synchronisation over ``torch.distributed`` object broadcast."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = group

    def leader_sync(self, admits: List[Tuple[str, List[int], object]], aborts: List[str], stop: bool = False) -> None:
        box = [{"admits": admits, "aborts": aborts, "stop": stop}]
        self.dist.broadcast_object_list(box, src=0, group=self.group)

    def follower_recv(self):
        box = [None]
        self.dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]


def follower_loop(llm, control: SpmdControl = None) -> None:
    """Body of ranks > 0 while rank 0 serves HTTP."""
    control = control or SpmdControl()
    while True:
        msg = control.follower_recv()
        if msg["stop"]:
            return
        for rid, ids, params in msg["admits"]:
            llm.add_request(ids, params, rid)
        for rid in msg["aborts"]:
            llm.abort(rid)
        if llm.has_unfinished:
            llm.step()
