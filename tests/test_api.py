"""The llama-cpp-python-style ``Llama`` class (the reference's Python binding surface) on a tiny synthetic model."""
import asyncio

import numpy as np
import pytest
import torch

import oxidize_b200
from oxidize_b200.models.config import preset
from oxidize_b200.utils.synth import synth_gguf


@pytest.fixture(scope="module")
def llama(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("api") / "tiny.gguf")
    synth_gguf(path, preset("tiny-llama", arch="qwen2", n_layers=2, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2,
                            head_dim=16, ffn_size=96), "F32", seed=1)
    return oxidize_b200.Llama(path, context_size=256, device="cpu", max_num_seqs=2, num_kv_blocks=64)


def test_text_generation_surfaces_agree(llama):
    text = llama.generate("hello there", max_tokens=5)
    comp = llama("hello there", max_tokens=5)
    assert comp["object"] == "text_completion" and comp["choices"][0]["text"] == text
    assert comp["choices"][0]["finish_reason"] in ("length", "stop") and comp["usage"]["completion_tokens"] <= 5
    assert asyncio.run(llama.generate_async("hello there", max_tokens=5)) == text
    with pytest.raises(ValueError):
        llama.generate("", max_tokens=3)
    with pytest.raises(ValueError):
        llama.generate("x", max_tokens=0)


def test_chat_completion_renders_the_template(llama):
    r = llama.create_chat_completion([{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}], max_tokens=4)
    assert r["object"] == "chat.completion" and r["choices"][0]["message"]["role"] == "assistant"
    # a Qwen file without a stored template gets ChatML; bare strings are user turns
    r2 = llama.create_chat_completion(["hi"], max_tokens=4)
    r3 = asyncio.run(llama.create_chat_completion_async([{"role": "user", "content": "hi"}], max_tokens=4))
    assert r2["choices"][0]["message"]["content"] == r3["choices"][0]["message"]["content"]
    assert r2["usage"]["prompt_tokens"] > len(llama.tokenize("hi", add_bos=False))
    with pytest.raises(ValueError):
        llama.create_chat_completion([], max_tokens=4)


def test_token_level_calls(llama):
    ids = llama.tokenize("hello there", add_bos=False)
    assert ids and llama.detokenize(ids).decode() == "hello there"
    out = llama.generate_from_tokens(ids, max_tokens=4)
    assert isinstance(out, list) and len(out) == 4
    assert llama.generate_from_tokens(np.asarray(ids), max_tokens=4, output_tensor="numpy").tolist() == out
    t = llama.generate_from_tokens(torch.tensor(ids), max_tokens=4, output_tensor="torch")
    assert isinstance(t, torch.Tensor) and t.tolist() == out
    with pytest.raises(ValueError):
        llama.generate_from_tokens([], max_tokens=2)
    with pytest.raises(ValueError):
        llama.generate_from_tokens(ids, max_tokens=2, output_tensor="jax")


def test_embeddings_are_pooled_hidden_states(llama):
    a, b = llama.embed("hello there"), llama.embed("completely different words")
    assert len(a) == 64 and abs(np.linalg.norm(a) - 1.0) < 1e-5
    assert not np.allclose(a, b, atol=1e-3) and np.allclose(a, llama.embed("hello there"))
    assert llama.embed_tensor("hello there", "numpy").dtype == np.float32
    # last-token pooling of a causal model depends only on the prefix up to that token
    last = llama.llm.embed([[5, 6, 7, 8]], pooling="last")[0]
    mean = llama.llm.embed([[5, 6, 7, 8]], pooling="mean")[0]
    assert not np.allclose(last, mean, atol=1e-3)
    with pytest.raises(ValueError):
        llama.embed("")
