"""GGUF reader/writer, quant oracle, tokenizer and chat-template tests (CPU only)."""
import os
import struct

import numpy as np
import pytest

from oxidize_b200.formats import gguf as G
from oxidize_b200.formats import tokenizer as T
from oxidize_b200.quant import ref as Q

# the reference checkout, when one sits beside this repository (or where OXIDIZE_REFERENCE_DIR points)
_REF = os.environ.get("OXIDIZE_REFERENCE_DIR",
                      os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
FIXTURES = os.path.join(_REF, "oxidize-core", "tests", "fixtures")


def _write_small(path, alignment=32):
    w = G.GGUFWriter(path, arch="llama", alignment=alignment)
    w.add("llama.block_count", 2, G.GGUFValueType.UINT32)
    w.add("general.name", "unit")
    w.add("some.float", 1.5)
    w.add("some.bool", True)
    w.add("some.i64", -5, G.GGUFValueType.INT64)
    w.add("some.arr", [1, 2, 3])
    w.add("some.strs", ["a", "bc"], G.GGUFValueType.ARRAY, G.GGUFValueType.STRING)
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    w.add_tensor("a.weight", x)
    q = Q.quantize("Q4_K", np.random.default_rng(0).standard_normal(2 * 256).astype(np.float32))
    w.add_tensor("b.weight", q, (2, 256), "Q4_K")
    w.write()
    return x, q


def test_roundtrip(tmp_path):
    p = str(tmp_path / "m.gguf")
    x, q = _write_small(p)
    g = G.load_gguf(p)
    assert g.version == 3 and g.architecture == "llama" and g.alignment == 32
    assert g.get("llama.block_count") == 2 and g.get("some.float") == 1.5 and g.get("some.bool") is True
    assert g.get("some.i64") == -5 and g.get("some.arr") == [1, 2, 3] and g.get("some.strs") == ["a", "bc"]
    assert g.tensors["a.weight"].shape == (3, 4) and g.tensors["a.weight"].dims == (4, 3)
    np.testing.assert_array_equal(g.tensor("a.weight"), x)
    assert g.tensors["b.weight"].type.name == "Q4_K" and g.tensor("b.weight").shape == (2, 144)
    np.testing.assert_array_equal(g.tensor_bytes("b.weight"), q)
    for info in g.tensors.values():
        assert (g.data_offset + info.offset) % 32 == 0


def test_custom_alignment(tmp_path):
    p = str(tmp_path / "m64.gguf")
    _write_small(p, alignment=64)
    g = G.load_gguf(p)
    assert g.alignment == 64 and g.data_offset % 64 == 0


def test_pypi_reader_parses_our_file(tmp_path):
    gguf = pytest.importorskip("gguf")
    p = str(tmp_path / "m.gguf")
    x, _ = _write_small(p)
    r = gguf.GGUFReader(p)
    names = [t.name for t in r.tensors]
    assert names == ["a.weight", "b.weight"]
    np.testing.assert_array_equal(np.asarray(r.tensors[0].data).reshape(3, 4), x)


@pytest.mark.skipif(not os.path.isdir(FIXTURES), reason="reference fixtures not mounted")
def test_reference_fixtures():
    g = G.load_gguf(os.path.join(FIXTURES, "valid-v3.gguf"))
    assert g.version == 3
    for bad in ("invalid-magic.gguf", "invalid-alignment.gguf", "unsupported-version.gguf"):
        with pytest.raises(G.GGUFError):
            G.load_gguf(os.path.join(FIXTURES, bad))


def test_rejects_malformed():
    with pytest.raises(G.GGUFError):
        G.parse_gguf(b"GGML" + b"\0" * 40)
    with pytest.raises(G.GGUFError):
        G.parse_gguf(b"GGUF" + struct.pack("<I", 9) + b"\0" * 16)
    with pytest.raises(G.GGUFError):  # truncated metadata
        G.parse_gguf(b"GGUF" + struct.pack("<IQQ", 3, 0, 5))
    # tensor extent beyond the file
    head = b"GGUF" + struct.pack("<IQQ", 3, 1, 0)
    name = b"t"
    head += struct.pack("<Q", 1) + name + struct.pack("<I", 1) + struct.pack("<Q", 1024) + struct.pack("<IQ", 0, 0)
    with pytest.raises(G.GGUFError):
        G.parse_gguf(head + b"\0" * 64)


def test_fuzz_parser_never_crashes():
    rng = np.random.default_rng(0)
    base = bytearray(b"GGUF" + struct.pack("<IQQ", 3, 2, 3) + bytes(rng.integers(0, 256, 200, dtype=np.uint8)))
    for _ in range(300):
        b = bytearray(base)
        for _ in range(4):
            b[rng.integers(4, len(b))] = rng.integers(0, 256)
        try:
            G.parse_gguf(bytes(b))
        except G.GGUFError:
            pass


def test_split_shards(tmp_path):
    for i, name in enumerate(["x.weight", "y.weight"], 1):
        w = G.GGUFWriter(str(tmp_path / f"m-{i:05d}-of-00002.gguf"))
        w.add_tensor(name, np.full((2, 2), i, dtype=np.float32))
        w.write()
    g = G.load_gguf(str(tmp_path / "m-00002-of-00002.gguf"))
    assert sorted(g.tensors) == ["x.weight", "y.weight"]
    assert float(g.tensor("y.weight")[0, 0]) == 2.0 and float(g.tensor("x.weight")[0, 0]) == 1.0


def test_hf_name_map():
    assert G.map_hf_tensor_name("model.layers.3.self_attn.q_proj.weight") == ("blk.3.attn_q.weight", None)
    assert G.map_hf_tensor_name("model.layers.0.mlp.experts.5.down_proj.weight") == ("blk.0.ffn_down_exps.weight", 5)
    assert G.map_hf_tensor_name("lm_head.weight") == ("output.weight", None)
    assert G.map_hf_tensor_name("nonsense") is None


# --------------------------------------------------------------------------- quant
@pytest.mark.parametrize("name", ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K",
                                  "IQ4_NL", "IQ4_XS"])
def test_decoders_match_pypi(name):
    gguf = pytest.importorskip("gguf")
    t = G.ggml_type(name)
    rng = np.random.default_rng(1)
    raw = rng.integers(0, 256, size=t.type_size * 16, dtype=np.uint8)
    ours = Q.dequantize(name, raw)
    theirs = gguf.quants.dequantize(raw, getattr(gguf.GGMLQuantizationType, name)).reshape(-1)
    ok = np.isfinite(theirs)
    np.testing.assert_allclose(ours[ok], theirs[ok], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name,tol", [("Q4_0", 0.12), ("Q5_0", 0.06), ("Q8_0", 0.01), ("Q4_K", 0.1), ("Q6_K", 0.03),
                                      ("Q8_K", 0.01), ("NVFP4", 0.16), ("BF16", 0.005), ("F16", 0.001)])
def test_quantize_roundtrip_error(name, tol):
    x = (np.random.default_rng(2).standard_normal(8192) * 0.02).astype(np.float32)
    y = Q.dequantize(name, Q.quantize(name, x), x.size)
    assert np.sqrt(((x - y) ** 2).mean()) / x.std() < tol


def test_size_validation():
    with pytest.raises(G.GGUFError):
        G.quantized_nbytes(G.ggml_type("Q4_K"), 1408)
    assert G.quantized_nbytes(G.ggml_type("Q4_K"), 512) == 288
    assert G.quantized_nbytes(G.ggml_type("NVFP4"), 128) == 72
    assert G.ggml_type(40).name == "NVFP4" and G.ggml_type(12).name == "Q4_K" and G.ggml_type(14).name == "Q6_K"


def test_nvfp4_scale_semantics():
    assert Q.ue4m3_to_f32(np.array([0x00, 0x7F, 0x38], dtype=np.uint8)).tolist() == [0.0, 0.0, 0.5]
    # bit 7 ignored by default (Rust decoder), honoured on request (CUDA decoder)
    assert Q.ue4m3_to_f32(np.array([0xB8], dtype=np.uint8))[0] == 0.5
    assert Q.ue4m3_to_f32(np.array([0xB8], dtype=np.uint8), honour_sign=True)[0] == -0.5


def test_torch_quantizers_decode_with_numpy_oracle():
    import torch

    from oxidize_b200.quant import torch_quant as TQ

    w = torch.randn(8, 512) * 0.02
    for name, tol in (("Q8_0", 0.01), ("Q4_K", 0.12), ("Q6_K", 0.03), ("NVFP4", 0.16)):
        raw = TQ.quantize(name, w).numpy()
        y = Q.dequantize(name, raw, w.numel()).reshape(8, 512)
        assert np.sqrt(((w.numpy() - y) ** 2).mean()) / w.numpy().std() < tol, name


# --------------------------------------------------------------------------- tokenizer
def _bpe():
    b2u = T.gpt2_byte_table()
    toks = ["<unk>", "<s>", "</s>"] + [b2u[b] for b in range(256)]
    merges = []
    for a, b in [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), ("Ġ", "w")]:
        toks.append(a + b)
        merges.append(f"{a} {b}")
    md = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": toks, "tokenizer.ggml.merges": merges,
          "tokenizer.ggml.token_type": [3, 3, 3] + [1] * (len(toks) - 3), "tokenizer.ggml.bos_token_id": 1,
          "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.unknown_token_id": 0}
    return T.load_tokenizer_from_metadata(md)


def test_bpe_roundtrip_and_merges():
    tk = _bpe()
    ids = tk.encode("hello world")
    assert tk.tokens[ids[0]] == "hello"
    assert tk.decode(ids) == "hello world"
    assert tk.decode(tk.encode("héllo ✓ 日本")) == "héllo ✓ 日本"
    assert not tk.add_bos_default()
    assert tk.encode_with_special_tokens("a</s>b")[1] == 2
    assert tk.encode_with_special_tokens("hi", add_bos=True)[0] == 1


def test_streaming_detokenizer_holds_partial_utf8():
    tk = _bpe()
    ids = tk.encode("✓!")
    sd = tk.streaming_detokenizer()
    pieces = [sd.push(i) for i in ids]
    assert "".join(pieces) + sd.finish() == "✓!"
    assert pieces[0] == "" and "�" not in "".join(pieces)


def test_heal_tokens():
    tk = _bpe()
    b2u = T.gpt2_byte_table()
    split = [tk.vocab[b2u[ord(c)]] for c in "hello"]
    assert tk.heal_tokens(split) == tk.encode("hello")


def test_sentencepiece_and_wordpiece():
    toks = ["<unk>", "<s>", "</s>", "▁hello", "▁world", "▁", "h", "e", "l", "o"] + [f"<0x{b:02X}>" for b in range(256)]
    scores = [0, 0, 0, -1.0, -1.0, -5.0, -6, -6, -6, -6] + [-20.0] * 256
    md = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": toks, "tokenizer.ggml.scores": scores,
          "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.unknown_token_id": 0}
    sp = T.load_tokenizer_from_metadata(md)
    assert sp.encode("hello world") == [3, 4]
    assert sp.decode([3, 4]) == "hello world"
    assert sp.add_bos_default()
    assert sp.decode(sp.encode("hé")) == "hé"  # byte fallback
    wp = T.load_tokenizer_from_metadata({"tokenizer.ggml.model": "bert", "tokenizer.ggml.tokens":
                                         ["[UNK]", "un", "##aff", "##able", "hello"], "tokenizer.ggml.unknown_token_id": 0})
    assert wp.encode("unaffable hello zzz") == [1, 2, 3, 4, 0]
    assert wp.decode([1, 2, 3, 4]) == "unaffable hello"
    with pytest.raises(T.TokenizerError):
        T.load_tokenizer_from_metadata({"tokenizer.ggml.model": "mystery", "tokenizer.ggml.tokens": ["a"]})


def test_chat_templates():
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    out = T.render_chat_template("{% for m in x %}<|im_start|>...", msgs, True)
    assert out == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    llama3 = ("{% for message in messages %}{{ '<|start_header_id|>' + message['role'] + '<|end_header_id|>\\n\\n' + "
              "message['content'] + '<|eot_id|>' }}{% endfor %}{% if add_generation_prompt %}"
              "{{ '<|start_header_id|>assistant<|end_header_id|>\\n\\n' }}{% endif %}")
    out = T.render_chat_template(llama3, msgs[1:], True)
    assert out == "<|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n"
    assert T.render_chat_template(llama3, msgs[1:], False).endswith("<|eot_id|>")
    assert T.chat_template_from_metadata({}, "qwen3") == T.CHATML_SENTINEL
    assert T.chat_template_from_metadata({}, "llama") is None
    # both renderers agree on that template; the plain-substitution one is the fallback
    assert T.render_chat_template(llama3, msgs, True, jinja=False) == T.render_chat_template(llama3, msgs, True)
    # the template Llama-3 checkpoints actually ship: a variable, a loop index, a filter, set statements
    real = ("{% set loop_messages = messages %}{% for message in loop_messages %}{% set content = '<|start_header_id|>' + "
            "message['role'] + '<|end_header_id|>\n\n'+ message['content'] | trim + '<|eot_id|>' %}{% if loop.index0 == 0 %}"
            "{% set content = bos_token + content %}{% endif %}{{ content }}{% endfor %}{% if add_generation_prompt %}"
            "{{ '<|start_header_id|>assistant<|end_header_id|>\n\n' }}{% endif %}")
    out = T.render_chat_template(real, [{"role": "system", "content": " be brief "}, {"role": "user", "content": "hi"}], True,
                                 bos_token="<|begin_of_text|>")
    assert out == ("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nbe brief<|eot_id|><|start_header_id|>user"
                   "<|end_header_id|>\n\nhi<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n")
    # Mistral-style: roles must alternate (the template raises otherwise -> falls back), [INST] wrapping
    mistral = ("{{ bos_token }}{% for message in messages %}{% if (message['role'] == 'user') != (loop.index0 % 2 == 0) %}"
               "{{ raise_exception('Conversation roles must alternate user/assistant/user/assistant/...') }}{% endif %}"
               "{% if message['role'] == 'user' %}{{ '[INST] ' + message['content'] + ' [/INST]' }}{% elif message['role'] == "
               "'assistant' %}{{ message['content'] + eos_token}}{% endif %}{% endfor %}")
    conv = [{"role": "user", "content": "a"}, {"role": "assistant", "content": "b"}, {"role": "user", "content": "c"}]
    assert T.render_chat_template(mistral, conv, True, "<s>", "</s>") == "<s>[INST] a [/INST]b</s>[INST] c [/INST]"
    assert "a" in T.render_chat_template(mistral, [{"role": "assistant", "content": "a"}], True)  # rejected by the template: fallback
    # a template cannot reach outside the sandbox
    assert "__class__" not in T.render_chat_template("{{ ''.__class__.__mro__ }}x{% for message in messages %}{{ message.content }}{% endfor %}",
                                                     [{"role": "user", "content": "q"}], False)


def test_codebook_iquants_decode_through_gguf_package():
    """IQ1/IQ2/IQ3 decode needs ggml's codebook grids; they come from the `gguf` package.  Round trip:
    quantize with the package, decode with ours, compare with the package's own decode."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants as gq

    from oxidize_b200.quant import ref as qref

    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (4, 512)).astype(np.float32)
    done = 0
    for name in ("IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"):
        qt = getattr(gguf.GGMLQuantizationType, name)
        try:
            raw = gq.quantize(x, qt)
        except Exception:
            continue  # the package decodes these types but cannot always encode them
        want = gq.dequantize(raw, qt).reshape(-1)
        got = qref.dequantize(name, raw.reshape(-1), x.size)
        np.testing.assert_array_equal(got, want.astype(np.float32))
        done += 1
    # decode-only check on random block bytes for every codebook type (structure, size, finiteness of scales aside)
    for name in qref._CODEBOOK_TYPES:
        t = qref.ggml_type(name)
        raw = rng.integers(0, 255, size=t.type_size * 3, dtype=np.uint8)
        raw[:2] = np.array([0.01], dtype=np.float16).view(np.uint8)  # a sane first scale
        out = qref.dequantize(name, raw)
        assert out.shape == (3 * t.block_size,)
    with pytest.raises(Exception):
        qref.dequantize("IQ2_XS", np.zeros(10, dtype=np.uint8))


def test_turboquant_weight_codec():
    from oxidize_b200.quant import turbo

    rng = np.random.default_rng(0)
    w = rng.standard_normal((7, 100)).astype(np.float32)  # a ragged last block
    x = rng.standard_normal(100).astype(np.float32)
    for bits, tol in ((8, 0.02), (4, 0.3)):
        d = turbo.quantize(w, bits)
        back = turbo.dequantize(d)
        assert back.shape == w.shape
        # error bounded by half a step of each block's scale
        step = np.repeat(d.scales, turbo.BLOCK, axis=1)[:, :100]
        assert (np.abs(back - w) <= 0.5 * step + 1e-6).all()
        assert np.allclose(turbo.gemv(d, x), back @ x, atol=1e-4)
        assert np.abs(turbo.gemv(d, x) - w @ x).max() < tol * np.abs(w @ x).max() + tol
    assert turbo.quantize(w, 4).nbytes <= 0.2 * w.nbytes  # 20 bytes per 32 values (padding of the ragged block included)
    z = turbo.quantize(np.zeros((2, 32), dtype=np.float32), 4)
    assert (turbo.dequantize(z) == 0).all()
    with pytest.raises(ValueError):
        turbo.quantize(w, 3)
    with pytest.raises(ValueError):
        turbo.gemv(turbo.quantize(w, 8), x[:50])


def test_bpe_tokenizer_training_round_trips_and_compresses(tmp_path):
    from oxidize_b200.formats import tokenizer_train as TT

    corpus = ("the quick brown fox jumps over the lazy dog. " * 40 + "pack my box with five dozen liquor jugs! " * 30
              + "naïve café — déjà vu, 東京 is far. " * 10)
    md = TT.train_bpe([corpus], 400)
    toks, merges = md["tokenizer.ggml.tokens"], md["tokenizer.ggml.merges"]
    assert len(toks) <= 400 and len(set(toks)) == len(toks) and len(merges) == len(toks) - 256 - 2
    assert md["tokenizer.ggml.bos_token_id"] == len(toks) - 2 and md["tokenizer.ggml.eos_token_id"] == len(toks) - 1
    assert md == TT.train_bpe([corpus], 400)  # deterministic
    tok = T.load_tokenizer_from_metadata(md)
    for text in ("the quick brown fox", "liquor jugs! déjà vu 東京", "unseen wörds & bytes \x00\x7f"):
        ids = tok.encode(text)
        assert tok.decode(ids) == text
    # frequent words became single tokens; the trained vocabulary beats bytes by a wide margin on its own corpus
    assert len(tok.encode(" quick")) == 1 and len(tok.encode(" the")) == 1
    assert len(tok.encode(corpus)) < 0.3 * len(corpus.encode("utf-8"))
    # every merge's parts were known when it was made
    known = set(toks[:256])
    for m in merges:
        a, b = m.split(" ")
        assert a in known and b in known
        known.add(a + b)
    with pytest.raises(ValueError):
        TT.train_bpe([corpus], 100)
    f = tmp_path / "c.txt"
    f.write_text(corpus)
    out = tmp_path / "tok.json"
    assert TT.main([str(f), "--vocab-size", "300", "--output", str(out)]) == 0
    import json as _json

    assert len(_json.loads(out.read_text())["tokenizer.ggml.tokens"]) <= 300
