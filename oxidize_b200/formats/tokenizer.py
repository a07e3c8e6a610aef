"""Tokenizers built from GGUF metadata: byte-level BPE (gpt2), SentencePiece unigram (llama),
WordPiece (bert) and tiktoken-style rank BPE; streaming detokenizer; token healing; the
non-Jinja chat-template renderer.

Family selection by ``tokenizer.ggml.model`` and the special-token keys are those of the
reference (``oxidize-core/src/format/tokenizer.rs:236-295``); ``add_bos`` defaults follow
``add_bos_default`` (``tokenizer.rs:70-82``: SentencePiece adds BOS, the others do not, unless
``tokenizer.ggml.add_bos_token`` says otherwise).  The chat-template contract (ChatML shortcut,
``{% for message in messages %}`` mini renderer) is ``process_chat_template``
(``tokenizer.rs:315-452``).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from functools import lru_cache
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple


class TokenizerError(ValueError):
    pass


@dataclass
class SpecialTokens:
    bos: Optional[int] = None
    eos: Optional[int] = None
    unk: Optional[int] = None
    pad: Optional[int] = None
    sep: Optional[int] = None
    cls: Optional[int] = None
    mask: Optional[int] = None
    add_bos_token: Optional[bool] = None
    add_eos_token: Optional[bool] = None
    control: frozenset = frozenset()  # ids whose token_type marks them control/user-defined

    def ids(self) -> List[int]:
        return [x for x in (self.bos, self.eos, self.unk, self.pad, self.sep, self.cls, self.mask) if x is not None]

    def is_special(self, tid: int) -> bool:
        return tid in self.ids() or tid in self.control


@lru_cache(maxsize=1)
def gpt2_byte_table() -> Tuple[str, ...]:
    """byte -> printable unicode char of the GPT-2 byte-level alphabet."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    table = [""] * 256
    for b, c in zip(bs, cs):
        table[b] = chr(c)
    return tuple(table)


@lru_cache(maxsize=1)
def _gpt2_char_to_byte() -> Dict[str, int]:
    return {c: b for b, c in enumerate(gpt2_byte_table())}


# GPT-2 pre-tokenizer split, written without \p classes (stdlib ``re``).
_PRETOK = re.compile(
    r"'s|'t|'re|'ve|'m|'ll|'d| ?[^\W\d_]+| ?\d+| ?(?:[^\s\w]|_)+|\s+(?!\S)|\s+", re.UNICODE)


class BaseTokenizer:
    family = "base"

    def __init__(self, tokens: Sequence[str], special: SpecialTokens):
        self.tokens = list(tokens)
        self.special_tokens = special
        self.vocab: Dict[str, int] = {}
        for i, t in enumerate(self.tokens):
            self.vocab.setdefault(t, i)
        sp = [(self.tokens[i], i) for i in sorted(set(special.ids()) | set(special.control)) if 0 <= i < len(self.tokens)]
        sp = [(t, i) for t, i in sp if t]
        sp.sort(key=lambda x: -len(x[0]))
        self._special_lookup = sp
        self._special_re = re.compile("|".join(re.escape(t) for t, _ in sp)) if sp else None

    # ---- public API
    @property
    def vocab_size(self) -> int:
        return len(self.tokens)

    def add_bos_default(self) -> bool:
        if self.special_tokens.add_bos_token is not None:
            return bool(self.special_tokens.add_bos_token)
        return self.family == "spm"

    def encode(self, text: str) -> List[int]:
        raise NotImplementedError

    def token_bytes(self, tid: int) -> bytes:
        raise NotImplementedError

    def decode(self, ids: Iterable[int]) -> str:
        return b"".join(self.token_bytes(i) for i in ids).decode("utf-8", errors="replace")

    def encode_with_special_tokens(self, text: str, add_bos: Optional[bool] = None, add_eos: bool = False,
                                   parse_special: bool = True) -> List[int]:
        out: List[int] = []
        if parse_special and self._special_re is not None:
            pos = 0
            for m in self._special_re.finditer(text):
                if m.start() > pos:
                    out.extend(self.encode(text[pos : m.start()]))
                out.append(self.vocab[m.group(0)])
                pos = m.end()
            if pos < len(text):
                out.extend(self.encode(text[pos:]))
        else:
            out = self.encode(text)
        if add_bos is None:
            add_bos = self.add_bos_default()
        st = self.special_tokens
        if add_bos and st.bos is not None and (not out or out[0] != st.bos):
            out.insert(0, st.bos)
        if add_eos and st.eos is not None:
            out.append(st.eos)
        return out

    def decode_without_special_tokens(self, ids: Iterable[int]) -> str:
        return self.decode([i for i in ids if not self.special_tokens.is_special(i)])

    def heal_tokens(self, ids: Sequence[int]) -> List[int]:
        """Re-tokenise every run of ordinary tokens so that a prompt cut mid-word maps to
        the canonical segmentation (``heal_tokens`` tokenizer.rs:96-128)."""
        if len(ids) < 2:
            return list(ids)
        out: List[int] = []
        span: List[int] = []
        for t in ids:
            if self.special_tokens.is_special(t):
                if span:
                    out.extend(self.encode(self.decode(span)))
                    span = []
                out.append(t)
            else:
                span.append(t)
        if span:
            out.extend(self.encode(self.decode(span)))
        return out

    def streaming_detokenizer(self) -> "StreamingDetokenizer":
        return StreamingDetokenizer(self)


class BpeTokenizer(BaseTokenizer):
    """Byte-level BPE with a merge table (``tokenizer.ggml.model = gpt2``)."""

    family = "bpe"

    def __init__(self, tokens, merges: Sequence[str], special: SpecialTokens):
        super().__init__(tokens, special)
        self.ranks: Dict[Tuple[str, str], int] = {}
        for i, m in enumerate(merges):
            a, _, b = m.partition(" ")
            if b:
                self.ranks.setdefault((a, b), i)
        self._cache: Dict[str, List[int]] = {}

    def _bpe(self, word: str) -> List[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = list(word)
        while len(parts) > 1:
            best, best_i = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                break
            parts[best_i : best_i + 2] = [parts[best_i] + parts[best_i + 1]]
        ids: List[int] = []
        for p in parts:
            tid = self.vocab.get(p)
            if tid is not None:
                ids.append(tid)
                continue
            for ch in p:  # unknown merge result: fall back to single byte-chars
                t = self.vocab.get(ch)
                if t is not None:
                    ids.append(t)
                elif self.special_tokens.unk is not None:
                    ids.append(self.special_tokens.unk)
        if len(self._cache) < 65536:
            self._cache[word] = ids
        return ids

    def encode(self, text: str) -> List[int]:
        table = gpt2_byte_table()
        out: List[int] = []
        for piece in _PRETOK.findall(text):
            out.extend(self._bpe("".join(table[b] for b in piece.encode("utf-8"))))
        return out

    def token_bytes(self, tid: int) -> bytes:
        if not 0 <= tid < len(self.tokens):
            raise TokenizerError(f"token id {tid} out of range")
        c2b = _gpt2_char_to_byte()
        tok = self.tokens[tid]
        out = bytearray()
        for ch in tok:
            b = c2b.get(ch)
            if b is None:
                out.extend(ch.encode("utf-8"))
            else:
                out.append(b)
        return bytes(out)


class SentencePieceTokenizer(BaseTokenizer):
    """Unigram SentencePiece (``llama`` / ``gemma``): Viterbi over piece scores, ``▁`` for
    spaces, ``<0xNN>`` byte fallback."""

    family = "spm"
    _BYTE_RE = re.compile(r"^<0x([0-9A-Fa-f]{2})>$")

    def __init__(self, tokens, scores: Sequence[float], special: SpecialTokens, token_types: Sequence[int] = ()):
        super().__init__(tokens, special)
        self.scores = list(scores) if scores else [0.0] * len(self.tokens)
        self.byte_ids: Dict[int, int] = {}
        for i, t in enumerate(self.tokens):
            m = self._BYTE_RE.match(t)
            if m:
                self.byte_ids[int(m.group(1), 16)] = i
        self.max_len = max((len(t) for t in self.tokens), default=1)
        self.add_dummy_prefix = True

    def encode(self, text: str) -> List[int]:
        if not text:
            return []
        s = text.replace(" ", "▁")
        if self.add_dummy_prefix and not s.startswith("▁"):
            s = "▁" + s
        n = len(s)
        NEG = -1e30
        best = [NEG] * (n + 1)
        back: List[Tuple[int, Optional[int]]] = [(0, None)] * (n + 1)
        best[0] = 0.0
        unk_pen = min(self.scores, default=0.0) - 10.0
        for i in range(n):
            if best[i] <= NEG:
                continue
            for L in range(1, min(self.max_len, n - i) + 1):
                tid = self.vocab.get(s[i : i + L])
                if tid is None or tid in self.byte_ids.values() or self.special_tokens.is_special(tid):
                    continue
                sc = best[i] + self.scores[tid]
                if sc > best[i + L]:
                    best[i + L] = sc
                    back[i + L] = (i, tid)
            sc = best[i] + unk_pen
            if sc > best[i + 1]:
                best[i + 1] = sc
                back[i + 1] = (i, None)
        out: List[int] = []
        j = n
        while j > 0:
            i, tid = back[j]
            if tid is None:
                raw = s[i:j].encode("utf-8")
                ids = [self.byte_ids[b] for b in raw if b in self.byte_ids]
                if len(ids) != len(raw):
                    ids = [self.special_tokens.unk] if self.special_tokens.unk is not None else []
                out.extend(reversed(ids))
            else:
                out.append(tid)
            j = i
        out.reverse()
        return out

    def token_bytes(self, tid: int) -> bytes:
        if not 0 <= tid < len(self.tokens):
            raise TokenizerError(f"token id {tid} out of range")
        for b, i in self.byte_ids.items():
            if i == tid:
                return bytes([b])
        return self.tokens[tid].replace("▁", " ").encode("utf-8")

    def decode(self, ids: Iterable[int]) -> str:
        ids = list(ids)
        txt = b"".join(self.token_bytes(i) for i in ids).decode("utf-8", errors="replace")
        if self.add_dummy_prefix and txt.startswith(" "):
            first = next((i for i in ids if not self.special_tokens.is_special(i)), None)
            if first is not None and self.tokens[first].startswith("▁"):
                txt = txt[1:]
        return txt


class WordPieceTokenizer(BaseTokenizer):
    """BERT WordPiece: whitespace/punctuation split, greedy longest match, ``##`` continuations."""

    family = "wordpiece"
    _SPLIT = re.compile(r"\w+|[^\w\s]", re.UNICODE)

    def __init__(self, tokens, special: SpecialTokens, lowercase: bool = True):
        super().__init__(tokens, special)
        self.lowercase = lowercase

    def encode(self, text: str) -> List[int]:
        if self.lowercase:
            text = text.lower()
        out: List[int] = []
        unk = self.special_tokens.unk
        for word in self._SPLIT.findall(text):
            i, pieces, bad = 0, [], False
            while i < len(word):
                j = len(word)
                cur = None
                while j > i:
                    sub = word[i:j] if i == 0 else "##" + word[i:j]
                    if sub in self.vocab:
                        cur = self.vocab[sub]
                        break
                    j -= 1
                if cur is None:
                    bad = True
                    break
                pieces.append(cur)
                i = j
            if bad:
                if unk is not None:
                    out.append(unk)
            else:
                out.extend(pieces)
        return out

    def token_bytes(self, tid: int) -> bytes:
        if not 0 <= tid < len(self.tokens):
            raise TokenizerError(f"token id {tid} out of range")
        return self.tokens[tid].encode("utf-8")

    def decode(self, ids: Iterable[int]) -> str:
        words: List[str] = []
        for i in ids:
            t = self.tokens[i]
            if t.startswith("##") and words:
                words[-1] += t[2:]
            else:
                words.append(t)
        return " ".join(words)


class TiktokenTokenizer(BaseTokenizer):
    """Rank-based byte BPE: the vocabulary index of a byte string is its merge priority."""

    family = "tiktoken"

    def __init__(self, tokens, special: SpecialTokens):
        super().__init__(tokens, special)
        c2b = _gpt2_char_to_byte()
        self.byte_vocab: Dict[bytes, int] = {}
        for i, t in enumerate(self.tokens):
            try:
                raw = bytes(c2b[ch] for ch in t)
            except KeyError:
                raw = t.encode("utf-8")
            self.byte_vocab.setdefault(raw, i)
        self._bytes = [None] * len(self.tokens)
        for raw, i in self.byte_vocab.items():
            self._bytes[i] = raw

    def _bpe(self, raw: bytes) -> List[int]:
        parts = [bytes([b]) for b in raw]
        while len(parts) > 1:
            best, best_i = None, -1
            for i in range(len(parts) - 1):
                r = self.byte_vocab.get(parts[i] + parts[i + 1])
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                break
            parts[best_i : best_i + 2] = [parts[best_i] + parts[best_i + 1]]
        unk = self.special_tokens.unk
        return [self.byte_vocab.get(p, unk if unk is not None else 0) for p in parts]

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        for piece in _PRETOK.findall(text):
            out.extend(self._bpe(piece.encode("utf-8")))
        return out

    def token_bytes(self, tid: int) -> bytes:
        if not 0 <= tid < len(self.tokens):
            raise TokenizerError(f"token id {tid} out of range")
        raw = self._bytes[tid]
        return raw if raw is not None else self.tokens[tid].encode("utf-8")


class StreamingDetokenizer:
    """Emits text token by token, holding back bytes of an incomplete UTF-8 sequence."""

    def __init__(self, tok: BaseTokenizer):
        self.tok = tok
        self.pending = b""
        self._first = True

    def push(self, tid: int) -> str:
        raw = self.tok.token_bytes(tid)
        if self._first and self.tok.family == "spm" and raw.startswith(b" "):
            raw = raw[1:]
        self._first = False
        data = self.pending + raw
        # find the longest prefix that is valid UTF-8
        cut = len(data)
        for back in range(1, min(4, len(data)) + 1):
            b = data[-back]
            if b & 0xC0 == 0x80:
                continue
            need = 1 if b < 0x80 else 2 if b >> 5 == 0b110 else 3 if b >> 4 == 0b1110 else 4 if b >> 3 == 0b11110 else 1
            if need > back:
                cut = len(data) - back
            break
        out, self.pending = data[:cut], data[cut:]
        return out.decode("utf-8", errors="replace")

    def finish(self) -> str:
        out, self.pending = self.pending, b""
        return out.decode("utf-8", errors="replace")


# --------------------------------------------------------------------------- loading


def _special_from_metadata(md: Mapping) -> SpecialTokens:
    def g(*keys):
        for k in keys:
            v = md.get(f"tokenizer.ggml.{k}")
            if v is not None:
                return int(v)
        return None

    types = md.get("tokenizer.ggml.token_type") or []
    control = frozenset(i for i, t in enumerate(types) if t in (3, 4))
    ab = md.get("tokenizer.ggml.add_bos_token")
    ae = md.get("tokenizer.ggml.add_eos_token")
    return SpecialTokens(bos=g("bos_token_id"), eos=g("eos_token_id"), unk=g("unknown_token_id"),
                         pad=g("padding_token_id", "pad_token_id"), sep=g("separator_token_id", "sep_token_id"),
                         cls=g("cls_token_id"), mask=g("mask_token_id"),
                         add_bos_token=None if ab is None else bool(ab), add_eos_token=None if ae is None else bool(ae),
                         control=control)


def load_tokenizer_from_metadata(md: Mapping) -> BaseTokenizer:
    model = md.get("tokenizer.ggml.model")
    if model is None:
        raise TokenizerError("GGUF has no tokenizer.ggml.model")
    tokens = md.get("tokenizer.ggml.tokens")
    if not tokens:
        raise TokenizerError("GGUF has no tokenizer.ggml.tokens")
    sp = _special_from_metadata(md)
    if model in ("llama", "gemma", "gemma4"):
        return SentencePieceTokenizer(tokens, md.get("tokenizer.ggml.scores") or [], sp)
    if model == "bert":
        return WordPieceTokenizer(tokens, sp)
    if model in ("gpt2", "lfm2", "lfm2moe"):
        return BpeTokenizer(tokens, md.get("tokenizer.ggml.merges") or [], sp)
    if model == "tiktoken":
        return TiktokenTokenizer(tokens, sp)
    raise TokenizerError(f"unsupported tokenizer model {model!r}")


def load_tokenizer_from_gguf(path_or_file) -> BaseTokenizer:
    from .gguf import GGUFFile, load_gguf

    g = path_or_file if isinstance(path_or_file, GGUFFile) else load_gguf(path_or_file)
    return load_tokenizer_from_metadata(g.metadata)


# --------------------------------------------------------------------------- chat template

CHATML_SENTINEL = "<|im_start|>"
_FOR_RE = re.compile(r"\{%-?\s*for\s+message\s+in\s+messages\s*-?%\}(.*?)\{%-?\s*endfor\s*-?%\}", re.S)
_GEN_RE = re.compile(r"\{%-?\s*if\s+add_generation_prompt\s*-?%\}(.*?)\{%-?\s*endif\s*-?%\}", re.S)
_VAR_RE = re.compile(r"\{\{-?\s*(.*?)\s*-?\}\}")


def chat_template_from_metadata(md: Mapping, arch: Optional[str] = None) -> Optional[str]:
    t = md.get("tokenizer.chat_template") or md.get("tokenizer.ggml.chat_template")
    if t:
        return str(t)
    arch = arch or md.get("general.architecture")
    if arch in ("qwen", "qwen2", "qwen2moe", "qwen35", "qwen3", "qwen3moe", "qwen3_5_moe"):
        return CHATML_SENTINEL
    return None


def _expand_vars(body: str, msg: Mapping[str, str], extra: Mapping[str, str]) -> str:
    def sub(m):
        expr = m.group(1)
        parts = [p.strip() for p in expr.split("+")]
        out = []
        for p in parts:
            if p in ("message['role']", 'message["role"]', "message.role"):
                out.append(msg.get("role", ""))
            elif p in ("message['content']", 'message["content"]', "message.content",
                       "message['content'] | trim", "message.content | trim"):
                c = msg.get("content", "")
                out.append(c.strip() if "trim" in p else c)
            elif len(p) >= 2 and p[0] == p[-1] and p[0] in "'\"":
                out.append(p[1:-1].encode().decode("unicode_escape"))
            elif p in extra:
                out.append(extra[p])
            else:
                out.append("")
        return "".join(out)

    return _VAR_RE.sub(sub, body)


def _render_jinja(template: str, messages, add_generation_prompt: bool, bos_token: str, eos_token: str) -> Optional[str]:
    """The template through a sandboxed Jinja environment set up the way checkpoints expect (``trim_blocks``,
    ``lstrip_blocks``, a ``raise_exception`` helper); None when Jinja is missing or the template does not render."""
    try:
        import jinja2
        from jinja2.sandbox import ImmutableSandboxedEnvironment
    except ImportError:
        return None

    def raise_exception(message):
        raise jinja2.TemplateError(message)

    try:
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = raise_exception
        return env.from_string(template).render(messages=[dict(m) for m in messages], add_generation_prompt=add_generation_prompt,
                                                bos_token=bos_token, eos_token=eos_token)
    except Exception:  # noqa: BLE001 - syntax the sandbox refuses, a role order the template rejects ...
        return None


def render_chat_template(template: Optional[str], messages: Sequence[Mapping[str, str]],
                         add_generation_prompt: bool = True, bos_token: str = "", eos_token: str = "",
                         jinja: bool = True) -> str:
    """Render ``messages``.  Any template mentioning ``<|im_start|>`` produces canonical ChatML (the reference's first
    rule).  Other templates are rendered by Jinja when it is available (real checkpoints' templates use variables, nested
    conditions and filters); where that fails, or with ``jinja=False``, the reference's second rule applies: the body of the
    message loop is expanded once per message by plain string substitution (``format/tokenizer.rs:315-452``)."""
    if template is None:
        template = CHATML_SENTINEL
    if CHATML_SENTINEL in template:
        out = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
        if add_generation_prompt:
            out += "<|im_start|>assistant\n"
        return out
    if jinja and ("{%" in template or "{{" in template):
        rendered = _render_jinja(template, messages, add_generation_prompt, bos_token, eos_token)
        if rendered is not None:
            return rendered
    extra = {"bos_token": bos_token, "eos_token": eos_token}
    m = _FOR_RE.search(template)
    if not m:
        return "".join(f"{x['role']}: {x['content']}\n" for x in messages) + ("assistant: " if add_generation_prompt else "")
    head, body, tail = template[: m.start()], m.group(1), template[m.end():]
    out = _expand_vars(_strip_tags(head), {}, extra)
    for msg in messages:
        out += _expand_vars(_strip_tags(body), msg, extra)
    g = _GEN_RE.search(tail)
    if g:
        pre, gen, post = tail[: g.start()], g.group(1), tail[g.end():]
        out += _expand_vars(_strip_tags(pre), {}, extra)
        if add_generation_prompt:
            out += _expand_vars(_strip_tags(gen), {}, extra)
        out += _expand_vars(_strip_tags(post), {}, extra)
    else:
        out += _expand_vars(_strip_tags(tail), {}, extra)
    return out


_TAG_RE = re.compile(r"\{%.*?%\}", re.S)


def _strip_tags(s: str) -> str:
    return _TAG_RE.sub("", s)
