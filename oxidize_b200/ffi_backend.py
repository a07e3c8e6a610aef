"""Python half of the C ABI (``csrc/ffi.cpp`` → ``liboxidize_ffi.so``): the functions the C entry points call.

A model handle is an :class:`oxidize_b200.engine.llm.LLM`; a session is a position counter plus a cache of its own that
is created on the first forward (the reference's ``Session``: one sequence, its KV state, ``oxidize-ffi/src/lib.rs``).
``model_forward`` feeds the given tokens at the session's position and writes the logits that follow the last of them
into the caller's float buffer.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import numpy as np
import torch


class Session:
    def __init__(self) -> None:
        self.pos = 0
        self.kv = None
        self.owner = None  # the model whose cache this is

    def reset(self) -> None:
        if self.owner is not None and self.kv is not None:
            self.owner.model.release_state(self.kv)
        self.pos, self.kv, self.owner = 0, None, None


def model_load(path: str, device: Optional[str] = None):
    from .engine.llm import LLM, EngineConfig

    import os

    device = device or os.environ.get("OXIDIZE_FFI_DEVICE") or ("cuda" if torch.cuda.is_available() else "cpu")
    return LLM.from_gguf(path, EngineConfig(max_num_seqs=1, num_kv_blocks=8, cuda_graphs=False), device=device)


def model_vocab_size(llm) -> int:
    return int(llm.cfg.vocab_size)


def session_new() -> Session:
    return Session()


def model_forward(llm, session: Session, tokens: List[int], logits_ptr: int, vocab_size: int) -> int:
    """0 on success; negative codes: -2 bad argument, -3 context exhausted."""
    from .models.transformer import BatchMeta

    n = len(tokens)
    if n == 0 or vocab_size < llm.cfg.vocab_size or any(not 0 <= t < llm.cfg.vocab_size for t in tokens):
        return -2
    m, dev = llm.model, llm.device
    page = llm.config.kv_page_size
    cap = llm.config.max_model_len
    if session.owner is not llm:
        session.reset()
        session.owner = llm
        session.kv = m.new_cache((cap + page - 1) // page, page, llm.kv.spec.dtype_name)
    if session.pos + n > cap:
        return -3
    i32 = dict(dtype=torch.int32, device=dev)
    lo, hi = session.pos, session.pos + n
    pos = torch.arange(lo, hi, **i32)
    nblk = (cap + page - 1) // page
    meta = BatchMeta(torch.tensor(tokens, **i32), pos, pos.clone(), torch.tensor([0, n], **i32), torch.tensor([hi], **i32),
                     torch.arange(nblk, **i32)[None, :], torch.tensor([n - 1], **i32), n, hi, 1)
    logits = m.forward(meta, session.kv).float().reshape(-1).cpu().contiguous()
    session.pos = hi
    ctypes.memmove(logits_ptr, logits.data_ptr(), llm.cfg.vocab_size * 4)
    return 0


def sample_argmax(logits_ptr: int, vocab_size: int) -> int:
    a = np.ctypeslib.as_array(ctypes.cast(logits_ptr, ctypes.POINTER(ctypes.c_float)), shape=(vocab_size,))
    best = float(a.max())
    return int(np.flatnonzero(a == best)[-1])  # the last maximal element, as the reference's max_by does


# quantization type ids of the C ABI (GGML type ids)
def gemv_quantized(qtype: int, q_ptr: int, q_len: int, rows: int, cols: int, vec_ptr: int, out_ptr: int) -> int:
    """out[rows] = W[rows, cols] (packed, GGML type ``qtype``) x vector[cols]; 0 on success."""
    from .formats.gguf import GGML_TYPE_BY_ID
    from .quant import ref as qref

    t = GGML_TYPE_BY_ID.get(int(qtype))
    if t is None or rows <= 0 or cols <= 0 or cols % t.block_size:
        return -2
    need = rows * cols // t.block_size * t.type_size
    if q_len < need:
        return -2
    raw = np.ctypeslib.as_array(ctypes.cast(q_ptr, ctypes.POINTER(ctypes.c_uint8)), shape=(need,))
    w = np.asarray(qref.dequantize(t.name, raw, rows * cols), dtype=np.float32).reshape(rows, cols)
    v = np.ctypeslib.as_array(ctypes.cast(vec_ptr, ctypes.POINTER(ctypes.c_float)), shape=(cols,))
    out = np.ctypeslib.as_array(ctypes.cast(out_ptr, ctypes.POINTER(ctypes.c_float)), shape=(rows,))
    out[:] = w @ v
    return 0
