"""``Llama``: the small llama-cpp-python-style class the reference ships as its Python binding
(``oxidize-py/oxidize.pyi:42-60``, ``oxidize-py/src/lib.rs``): ``generate``, ``generate_async``,
``create_completion`` / ``__call__``, ``create_chat_completion(_async)``, ``tokenize`` / ``detokenize``,
``generate_from_tokens`` and ``embed`` / ``embed_tensor``, here on top of :class:`oxidize_b200.engine.llm.LLM`.

Differences from the binding, all in the direction of doing the real thing: the model's own hyper-parameters are read
from the checkpoint (``vocab_size`` / ``context_size`` / ``layer_count`` arguments are accepted and ignored except that
``context_size`` caps the serving context), sampling parameters may be passed, ``finish_reason`` reports ``stop`` when
the model ended the text, and ``embed`` returns pooled hidden states of the model instead of byte buckets.
"""
from __future__ import annotations

import asyncio
import uuid
from typing import Any, Dict, List, Optional, Sequence, Union

from .engine.llm import LLM, EngineConfig
from .engine.sampler import SamplingParams
from .formats.tokenizer import render_chat_template


def _as_list(tokens) -> List[int]:
    if hasattr(tokens, "tolist"):
        tokens = tokens.tolist()
    return [int(t) for t in tokens]


def _convert(values, kind: Optional[str], dtype: str):
    if kind in (None, "list"):
        return list(values)
    if kind == "numpy":
        import numpy as np

        return np.asarray(values, dtype=np.int64 if dtype == "int" else np.float32)
    if kind == "torch":
        import torch

        return torch.tensor(values, dtype=torch.int64 if dtype == "int" else torch.float32)
    raise ValueError("output_tensor must be 'list', 'numpy' or 'torch'")


class Llama:
    def __init__(self, model_path: str, vocab_size: int = 0, context_size: int = 4096, layer_count: int = 0,
                 device: Optional[str] = None, temperature: float = 0.0, engine_config: Optional[EngineConfig] = None,
                 **engine_kwargs: Any) -> None:
        if not model_path:
            raise ValueError("model_path cannot be empty")
        import torch

        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        cfg = engine_config or EngineConfig(max_model_len=context_size, **engine_kwargs)
        self.llm = LLM.from_gguf(model_path, cfg, device=device)
        self.model_path = model_path
        self.temperature = temperature
        self._chat_template = getattr(self.llm, "chat_template", None)

    # ------------------------------------------------------------------ helpers
    def _params(self, max_tokens: int, **kw: Any) -> SamplingParams:
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        kw.setdefault("temperature", self.temperature)
        return SamplingParams(max_tokens=max_tokens, **kw)

    def _run(self, prompt: Union[str, Sequence[int]], max_tokens: int, **kw: Any):
        if isinstance(prompt, str) and not prompt:
            raise ValueError("prompt cannot be empty")
        return self.llm.generate([prompt], self._params(max_tokens, **kw))[0]

    @staticmethod
    def _reason(out) -> str:
        return "length" if out.finish_reason in (None, "length") else "stop"

    # ------------------------------------------------------------------ text in, text out
    def generate(self, prompt: str, max_tokens: int = 16, **sampling: Any) -> str:
        return self._run(prompt, max_tokens, **sampling).text

    async def generate_async(self, prompt: str, max_tokens: int = 16, **sampling: Any) -> str:
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.generate(prompt, max_tokens, **sampling))

    def create_completion(self, prompt: str, max_tokens: int = 16, **sampling: Any) -> Dict[str, Any]:
        out = self._run(prompt, max_tokens, **sampling)
        return {"id": f"cmpl-{uuid.uuid4().hex[:24]}", "object": "text_completion",
                "choices": [{"index": 0, "text": out.text, "finish_reason": self._reason(out)}],
                "usage": {"prompt_tokens": len(out.prompt_token_ids), "completion_tokens": len(out.token_ids),
                          "total_tokens": len(out.prompt_token_ids) + len(out.token_ids)}}

    __call__ = create_completion

    def create_chat_completion(self, messages: Union[Sequence[str], Sequence[Dict[str, str]]], max_tokens: int = 16,
                               **sampling: Any) -> Dict[str, Any]:
        if not messages:
            raise ValueError("messages cannot be empty")
        # bare strings are user turns, as in the binding
        msgs = [m if isinstance(m, dict) else {"role": "user", "content": str(m)} for m in messages]
        out = self._run(render_chat_template(self._chat_template, msgs, True), max_tokens, **sampling)
        return {"id": f"chatcmpl-{uuid.uuid4().hex[:24]}", "object": "chat.completion",
                "choices": [{"index": 0, "message": {"role": "assistant", "content": out.text},
                             "finish_reason": self._reason(out)}],
                "usage": {"prompt_tokens": len(out.prompt_token_ids), "completion_tokens": len(out.token_ids),
                          "total_tokens": len(out.prompt_token_ids) + len(out.token_ids)}}

    async def create_chat_completion_async(self, messages, max_tokens: int = 16, **sampling: Any) -> Dict[str, Any]:
        return await asyncio.get_running_loop().run_in_executor(
            None, lambda: self.create_chat_completion(messages, max_tokens, **sampling))

    # ------------------------------------------------------------------ tokens
    def tokenize(self, text: str, add_bos: bool = True) -> List[int]:
        tok = self.llm.tokenizer
        ids = list(tok.encode(text))
        bos = tok.special_tokens.bos
        if bos is not None and bos >= 0:
            if add_bos and (not ids or ids[0] != bos):
                ids = [bos] + ids
            elif not add_bos and ids and ids[0] == bos:
                ids = ids[1:]
        return ids

    def detokenize(self, tokens) -> bytes:
        return self.llm.tokenizer.decode_without_special_tokens(_as_list(tokens)).encode("utf-8")

    def generate_from_tokens(self, prompt_tokens, max_tokens: int = 16, output_tensor: Optional[str] = None, **sampling: Any):
        ids = _as_list(prompt_tokens)
        if not ids:
            raise ValueError("prompt_tokens cannot be empty")
        return _convert(self._run(ids, max_tokens, **sampling).token_ids, output_tensor, "int")

    # ------------------------------------------------------------------ embeddings
    def embed(self, text: str) -> List[float]:
        if not text:
            raise ValueError("text cannot be empty")
        return [float(x) for x in self.llm.embed([text])[0]]

    def embed_tensor(self, text: str, output_tensor: Optional[str] = None):
        return _convert(self.embed(text), output_tensor, "float")
