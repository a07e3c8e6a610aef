"""Grammar-constrained sampling and beam search.

``TokenGrammar`` is a context-free grammar whose terminals are token ids, the shape of the
reference's grammar constraint (``oxidize-core/src/model/sampling.rs`` grammar types ``:147-234``):
during sampling only tokens that keep some parse alive can be drawn.  The parser keeps a set of
stacks of pending symbols (the scheme llama.cpp's GBNF sampler uses): non-terminals on top of a
stack are expanded into all their alternatives, so the allowed tokens are the terminals on top of
the stacks; accepting a token pops it from every stack that expected it.

``beam_search`` is the width-``k`` search of ``sampling.rs:737``: hypotheses are extended by
their ``k`` best next tokens, ranked by length-normalised log-probability, finished ones are set
aside when they emit EOS.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple, Union

import numpy as np

Symbol = Union[int, str]
Stack = Tuple[Symbol, ...]  # pending symbols, next one first


class GrammarError(ValueError):
    pass


class TokenGrammar:
    def __init__(self, rules: Dict[str, Sequence[Sequence[Symbol]]], root: str = "root", eos_token_ids: Iterable[int] = (),
                 max_stacks: int = 4096):
        if root not in rules:
            raise GrammarError(f"grammar has no rule {root!r}")
        for name, alts in rules.items():
            for alt in alts:
                for sym in alt:
                    if isinstance(sym, str) and sym not in rules:
                        raise GrammarError(f"rule {name!r} refers to unknown rule {sym!r}")
        self.rules = {k: [tuple(a) for a in v] for k, v in rules.items()}
        self.root = root
        self.eos = set(int(t) for t in eos_token_ids)
        self.max_stacks = max_stacks

    # ---- stack expansion
    def _expand(self, stacks: Iterable[Stack]) -> Set[Stack]:
        """Replace leading non-terminals by their alternatives until every stack starts with a terminal
        (or is empty = the parse may end here)."""
        out: Set[Stack] = set()
        todo = list(stacks)
        seen: Set[Stack] = set()
        while todo:
            st = todo.pop()
            if st in seen:
                continue
            seen.add(st)
            if not st or isinstance(st[0], int):
                out.add(st)
                continue
            for alt in self.rules[st[0]]:
                todo.append(alt + st[1:])
            if len(seen) > self.max_stacks:
                raise GrammarError("grammar expansion does not terminate (left recursion?)")
        return out

    def _stacks(self, state: dict) -> Set[Stack]:
        st = state.get("grammar_stacks")
        if st is None:
            st = state["grammar_stacks"] = self._expand([(self.root,)])
        return st

    # ---- sampler interface
    def allowed_tokens(self, state: dict) -> Optional[Set[int]]:
        stacks = self._stacks(state)
        allowed = {st[0] for st in stacks if st}
        if any(not st for st in stacks):
            allowed |= self.eos
        return allowed

    def advance(self, state: dict, token: int) -> None:
        stacks = self._stacks(state)
        if token in self.eos and any(not st for st in stacks):
            state["grammar_stacks"] = {()}
            state["grammar_done"] = True
            return
        nxt = [st[1:] for st in stacks if st and st[0] == token]
        if not nxt:
            raise GrammarError(f"token {token} is not allowed by the grammar here")
        state["grammar_stacks"] = self._expand(nxt)

    def is_complete(self, state: dict) -> bool:
        return any(not st for st in self._stacks(state))

    def accepts(self, tokens: Sequence[int]) -> bool:
        state: dict = {}
        try:
            for t in tokens:
                self.advance(state, t)
        except GrammarError:
            return False
        return self.is_complete(state)


def log_softmax(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float64)
    m = x.max(axis=-1, keepdims=True)
    return x - m - np.log(np.exp(x - m).sum(axis=-1, keepdims=True))


def beam_search(next_logits: Callable[[List[List[int]]], np.ndarray], prompt: Sequence[int], beam_width: int = 4,
                max_new_tokens: int = 32, eos_token_id: Optional[int] = None, length_penalty: float = 1.0
                ) -> List[Tuple[List[int], float]]:
    """``next_logits(list of token lists) -> [n, vocab]`` scores every live hypothesis in one batch.
    Returns up to ``beam_width`` (generated tokens, score) pairs, best first; score is the summed
    log-probability divided by ``len ** length_penalty``."""
    if beam_width < 1:
        raise ValueError("beam_width must be >= 1")
    live: List[Tuple[List[int], float]] = [([], 0.0)]
    done: List[Tuple[List[int], float]] = []

    def norm(tokens, lp):
        return lp / (max(len(tokens), 1) ** length_penalty)

    for _ in range(max_new_tokens):
        if not live:
            break
        lps = log_softmax(np.asarray(next_logits([list(prompt) + t for t, _ in live])))
        cand: List[Tuple[List[int], float]] = []
        for (toks, lp), row in zip(live, lps):
            top = np.argsort(-row, kind="stable")[:beam_width]
            for t in top:
                cand.append((toks + [int(t)], lp + float(row[t])))
        cand.sort(key=lambda c: -norm(*c))
        live = []
        for toks, lp in cand:
            if eos_token_id is not None and toks[-1] == eos_token_id:
                done.append((toks, lp))
            else:
                live.append((toks, lp))
            if len(live) >= beam_width:
                break
        if len(done) >= beam_width and (not live or norm(*max(done, key=lambda c: norm(*c))) >= norm(*live[0])):
            break
    allh = done + live
    allh.sort(key=lambda c: -norm(*c))
    return [(t, norm(t, lp)) for t, lp in allh[:beam_width]]
