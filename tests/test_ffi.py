"""The C ABI (`liboxidize_ffi.so`): called in-process through ctypes, and from a stand-alone C program that embeds the
interpreter."""
import ctypes
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest
import torch

from oxidize_b200.build import CSRC, build_ffi
from oxidize_b200.engine.llm import LLM, EngineConfig
from oxidize_b200.models.config import preset
from oxidize_b200.quant import ref as qref
from oxidize_b200.utils.synth import synth_gguf

LIB = build_ffi()
pytestmark = pytest.mark.skipif(not LIB, reason="no interpreter headers to build the shim with")


@pytest.fixture(scope="module")
def model_path(tmp_path_factory):
    p = str(tmp_path_factory.mktemp("ffi") / "tiny.gguf")
    synth_gguf(p, preset("tiny-llama", n_layers=2, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96),
               "F32", seed=4, norm_jitter=0.1)
    return p


def _lib():
    L = ctypes.CDLL(LIB)
    vp, u32, sz = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_size_t
    L.oxidize_ffi_version.restype = ctypes.c_char_p
    L.oxidize_model_load.restype = vp
    L.oxidize_model_load.argtypes = [ctypes.c_char_p]
    L.oxidize_model_free.argtypes = [vp]
    L.oxidize_model_vocab_size.restype = u32
    L.oxidize_model_vocab_size.argtypes = [vp]
    L.oxidize_session_new.restype = vp
    L.oxidize_session_reset.argtypes = [vp]
    L.oxidize_session_free.argtypes = [vp]
    L.oxidize_model_forward.restype = ctypes.c_int32
    L.oxidize_model_forward.argtypes = [vp, vp, ctypes.POINTER(u32), sz, ctypes.POINTER(ctypes.c_float), sz]
    L.oxidize_sample_argmax.restype = u32
    L.oxidize_sample_argmax.argtypes = [ctypes.POINTER(ctypes.c_float), sz]
    L.oxidize_gemv_quantized.restype = ctypes.c_int32
    L.oxidize_gemv_quantized.argtypes = [u32, ctypes.c_char_p, sz, sz, sz, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float)]
    return L


def test_c_abi_in_process(model_path, monkeypatch):
    monkeypatch.setenv("OXIDIZE_FFI_DEVICE", "cpu")
    L = _lib()
    assert b"oxidize" in L.oxidize_ffi_version()
    m = L.oxidize_model_load(model_path.encode())
    assert m and L.oxidize_model_vocab_size(m) == 300
    s = L.oxidize_session_new()
    prompt = [5, 9, 200, 31, 7]
    logits = (ctypes.c_float * 300)()
    toks = (ctypes.c_uint32 * len(prompt))(*prompt)
    assert L.oxidize_model_forward(m, s, toks, len(prompt), logits, 300) == 0
    llm = LLM.from_gguf(model_path, EngineConfig(max_model_len=64, max_num_seqs=1, num_kv_blocks=8), device="cpu")
    want = llm.next_token_logits([prompt])[0]
    assert np.allclose(np.frombuffer(logits, dtype=np.float32), want, atol=1e-4)
    # decode two more tokens through the session, one at a time
    seq = list(prompt)
    for _ in range(2):
        nxt = L.oxidize_sample_argmax(logits, 300)
        seq.append(nxt)
        one = (ctypes.c_uint32 * 1)(nxt)
        assert L.oxidize_model_forward(m, s, one, 1, logits, 300) == 0
        assert np.allclose(np.frombuffer(logits, dtype=np.float32), llm.next_token_logits([seq])[0], atol=1e-4)
    # reset: the same prompt gives the first logits again; bad arguments are refused
    L.oxidize_session_reset(s)
    assert L.oxidize_model_forward(m, s, toks, len(prompt), logits, 300) == 0
    assert np.allclose(np.frombuffer(logits, dtype=np.float32), want, atol=1e-4)
    assert L.oxidize_model_forward(m, s, toks, len(prompt), logits, 10) == -2
    bad = (ctypes.c_uint32 * 1)(4000)
    assert L.oxidize_model_forward(m, s, bad, 1, logits, 300) == -2
    assert L.oxidize_model_load(b"/nonexistent.gguf") is None
    L.oxidize_session_free(s)
    L.oxidize_model_free(m)
    # argmax: the last of equal maxima
    v = (ctypes.c_float * 5)(1.0, 7.0, 3.0, 7.0, 2.0)
    assert L.oxidize_sample_argmax(v, 5) == 3
    # packed-weight GEMV against the decoded matrix
    rng = np.random.default_rng(0)
    w = rng.standard_normal((8, 256)).astype(np.float32)
    x = rng.standard_normal(256).astype(np.float32)
    for name, tid in (("Q8_0", 8), ("Q4_K", 12), ("F32", 0)):
        raw = np.ascontiguousarray(qref.quantize(name, w.reshape(-1))).view(np.uint8).tobytes()
        out = (ctypes.c_float * 8)()
        assert L.oxidize_gemv_quantized(tid, raw, len(raw), 8, 256, x.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), out) == 0
        deq = np.asarray(qref.dequantize(name, np.frombuffer(raw, dtype=np.uint8), 8 * 256)).reshape(8, 256)
        assert np.allclose(np.frombuffer(out, dtype=np.float32), deq @ x, atol=1e-4)
    assert L.oxidize_gemv_quantized(12, raw, 10, 8, 256, x.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), out) == -2


C_PROGRAM = r"""
#include <stdio.h>
#include <stdlib.h>
#include "oxidize_ffi.h"
int main(int argc, char** argv) {
  void* m = oxidize_model_load(argv[1]);
  if (!m) return 2;
  uint32_t V = oxidize_model_vocab_size(m);
  void* s = oxidize_session_new();
  uint32_t prompt[5] = {5, 9, 200, 31, 7};
  float* logits = (float*)malloc(sizeof(float) * V);
  if (oxidize_model_forward(m, s, prompt, 5, logits, V) != 0) return 3;
  printf("%u", V);
  for (int i = 0; i < 6; ++i) {
    uint32_t t = oxidize_sample_argmax(logits, V);
    printf(" %u", t);
    if (oxidize_model_forward(m, s, &t, 1, logits, V) != 0) return 4;
  }
  printf("\n");
  oxidize_session_free(s);
  oxidize_model_free(m);
  return 0;
}
"""


def test_c_program_embeds_the_interpreter(model_path, tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "main.c"
    src.write_text(C_PROGRAM)
    exe = str(tmp_path / "main")
    subprocess.run([cc, "-O1", "-o", exe, str(src), f"-I{CSRC}", f"-L{CSRC}", "-loxidize_ffi", f"-Wl,-rpath,{CSRC}"], check=True)
    env = dict(os.environ, OXIDIZE_FFI_DEVICE="cpu", OXIDIZE_PYTHON=sys.executable)
    r = subprocess.run([exe, model_path], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(x) for x in r.stdout.split()]
    llm = LLM.from_gguf(model_path, EngineConfig(max_model_len=64, max_num_seqs=1, num_kv_blocks=8), device="cpu")
    from oxidize_b200.engine.sampler import SamplingParams

    want = llm.generate([[5, 9, 200, 31, 7]], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, tie="highest"))[0].token_ids
    assert got[0] == 300 and got[1:] == want
