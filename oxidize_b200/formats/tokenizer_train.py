"""Byte-level BPE tokenizer training (the reference's C port and its training tools carry a BPE trainer:
``oxidize-c/src/format`` tokenizer trainer, ``oxidize-training/tools``).

The corpus is cut by the same pre-tokenizer pattern the byte-level BPE tokenizer applies at encode time, bytes are written
in the GPT-2 byte alphabet, and the most frequent adjacent pair is merged until the vocabulary has the requested size.
The result is the metadata a GGUF file carries for ``tokenizer.ggml.model = gpt2`` (tokens, merges, token types, special
token ids), so a trained tokenizer loads through the ordinary loader.

    python -m oxidize_b200.formats.tokenizer_train corpus.txt --vocab-size 4096 --output tokenizer.json
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import Counter
from typing import Dict, List, Optional, Sequence, Tuple

from .tokenizer import _PRETOK, gpt2_byte_table

TOKEN_NORMAL, TOKEN_CONTROL = 1, 3


def train_bpe(texts: Sequence[str], vocab_size: int, special_tokens: Sequence[str] = ("<|bos|>", "<|eos|>"),
              min_frequency: int = 2) -> Dict[str, object]:
    """Returns GGUF tokenizer metadata: ``tokenizer.ggml.model / tokens / merges / token_type / bos_token_id / eos_token_id``."""
    table = gpt2_byte_table()
    alphabet = [table[b] for b in range(256)]
    if vocab_size < len(alphabet) + len(special_tokens):
        raise ValueError(f"vocab_size must be at least {len(alphabet) + len(special_tokens)} (the byte alphabet and the special tokens)")
    words: Counter = Counter()
    for text in texts:
        for piece in _PRETOK.findall(text):
            words["".join(table[b] for b in piece.encode("utf-8"))] += 1
    # every distinct word as a list of symbols, with its count; pair statistics are kept incrementally
    syms: List[List[str]] = [list(w) for w in words]
    counts: List[int] = list(words.values())
    pairs: Counter = Counter()
    where: Dict[Tuple[str, str], set] = {}
    for i, s in enumerate(syms):
        for a, b in zip(s, s[1:]):
            pairs[(a, b)] += counts[i]
            where.setdefault((a, b), set()).add(i)
    tokens = list(alphabet)
    merges: List[str] = []
    budget = vocab_size - len(tokens) - len(special_tokens)
    while budget > 0 and pairs:
        # most frequent pair; ties broken by the pair itself so that training is deterministic
        (a, b), freq = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        if freq < min_frequency:
            break
        merged = a + b
        tokens.append(merged)
        merges.append(f"{a} {b}")
        budget -= 1
        for i in list(where.get((a, b), ())):
            s, c = syms[i], counts[i]
            j, out = 0, []
            while j < len(s):
                if j + 1 < len(s) and s[j] == a and s[j + 1] == b:
                    out.append(merged)
                    j += 2
                else:
                    out.append(s[j])
                    j += 1
            for p in zip(s, s[1:]):  # take the word's old pairs out, put its new ones in
                pairs[p] -= c
                if pairs[p] <= 0:
                    del pairs[p]
                    where.pop(p, None)
                elif p in where:
                    where[p].discard(i)
            for p in zip(out, out[1:]):
                pairs[p] += c
                where.setdefault(p, set()).add(i)
            syms[i] = out
        pairs.pop((a, b), None)
        where.pop((a, b), None)
    types = [TOKEN_NORMAL] * len(tokens) + [TOKEN_CONTROL] * len(special_tokens)
    tokens += list(special_tokens)
    md: Dict[str, object] = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": merges,
                             "tokenizer.ggml.token_type": types}
    names = {t: len(tokens) - len(special_tokens) + i for i, t in enumerate(special_tokens)}
    for key, cands in (("bos", ("<|bos|>", "<s>", "<|begin_of_text|>")), ("eos", ("<|eos|>", "</s>", "<|end_of_text|>", "<|endoftext|>"))):
        tid = next((names[c] for c in cands if c in names), None)
        if tid is not None:
            md[f"tokenizer.ggml.{key}_token_id"] = tid
    return md


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="oxidize train-tokenizer", description="Train a byte-level BPE tokenizer")
    ap.add_argument("corpus", nargs="+", help="text files")
    ap.add_argument("--vocab-size", type=int, default=4096)
    ap.add_argument("--min-frequency", type=int, default=2)
    ap.add_argument("--special", action="append", default=[], help="special tokens (default <|bos|>, <|eos|>)")
    ap.add_argument("--output", required=True, help="JSON file with the GGUF tokenizer metadata")
    a = ap.parse_args(argv)
    texts = []
    for p in a.corpus:
        with open(p, encoding="utf-8") as f:
            texts.append(f.read())
    try:
        md = train_bpe(texts, a.vocab_size, tuple(a.special) or ("<|bos|>", "<|eos|>"), a.min_frequency)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    with open(a.output, "w", encoding="utf-8") as f:
        json.dump(md, f, ensure_ascii=False)
    print(f"wrote {a.output}: {len(md['tokenizer.ggml.tokens'])} tokens, {len(md['tokenizer.ggml.merges'])} merges")
    return 0


if __name__ == "__main__":
    sys.exit(main())
