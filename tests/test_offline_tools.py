"""Offline checkpoint tools: requantize, prune (name filter, magnitude, Wanda, n:m patterns), merge (linear, SLERP,
sharded output), LoRA merge."""
import json
import os

import numpy as np
import pytest
import torch

from oxidize_b200.cli.main import main as cli_main
from oxidize_b200.engine.llm import LLM, EngineConfig
from oxidize_b200.engine.sampler import SamplingParams
from oxidize_b200.formats.gguf import load_gguf
from oxidize_b200.formats.safetensors_io import SafeTensorsFile, save_file
from oxidize_b200.models.config import preset
from oxidize_b200.offline import lora, merge, prune, requantize
from oxidize_b200.offline.gguf_edit import decode_f32
from oxidize_b200.utils.synth import synth_gguf

EC = dict(max_model_len=128, max_num_seqs=2, num_kv_blocks=32, prefill_chunk_size=32, max_num_batched_tokens=32)


@pytest.fixture(scope="module")
def base(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("tools") / "base.gguf")
    cfg = preset("tiny-llama", n_layers=2, vocab_size=300, hidden_size=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_size=512)
    synth_gguf(path, cfg, "F32", seed=0, norm_jitter=0.1)
    return path


def _logits(path):
    llm = LLM.from_gguf(path, EngineConfig(**EC), device="cpu")
    return torch.from_numpy(llm.next_token_logits([[5, 9, 200, 31, 7, 11, 80]]))[0]


def test_requantize_keeps_metadata_and_the_function(base, tmp_path):
    out = str(tmp_path / "q.gguf")
    counts = requantize.requantize_gguf(base, out, "Q4_K_M", context_length=8192)
    g0, g = load_gguf(base), load_gguf(out)
    assert counts["Q4_K"] > 0 and counts["Q6_K"] > 0 and counts["F32"] == 5  # norms stay f32
    assert g.tensors["blk.0.attn_q.weight"].type.name == "Q4_K" and g.tensors["blk.0.attn_norm.weight"].type.name == "F32"
    assert g.tensors["output.weight"].type.name == "Q6_K"
    assert g.get("tokenizer.ggml.tokens") == g0.get("tokenizer.ggml.tokens")
    assert g.get("llama.context_length") == 8192 and g.get("llama.rope.scaling.type") == "yarn"
    assert abs(g.get("llama.rope.scaling.factor") - 4.0) < 1e-6 and g.get("llama.rope.scaling.original_context_length") == 2048
    # 4-bit weights: close to, not equal to, the f32 model
    out8 = str(tmp_path / "q8.gguf")
    assert cli_main(["quantize", "--input", base, "--output", out8, "--target", "Q8_0"]) == 0
    a, b = _logits(base), _logits(out8)
    assert 0 < (a - b).abs().max() / a.abs().max() < 0.05
    assert os.path.getsize(out8) < 0.4 * os.path.getsize(base)
    with pytest.raises(ValueError):
        requantize.requantize_gguf(base, out, "Q9_Z")


def test_requantize_appends_an_encoded_tensor(base, tmp_path):
    raw = tmp_path / "extra.bin"
    np.arange(2 * 32, dtype=np.float32).tofile(raw)
    out = str(tmp_path / "a.gguf")
    requantize.requantize_gguf(base, out, "F32", append_tensors=[f"extra.weight:{raw}:2,32:F32"])
    g = load_gguf(out)
    assert np.array_equal(g.tensor("extra.weight"), np.arange(64, dtype=np.float32).reshape(2, 32))
    with pytest.raises(ValueError):
        requantize.parse_append("broken")


def test_prune_masks():
    rng = np.random.default_rng(0)
    s = rng.random((6, 64)).astype(np.float32)
    m = prune.prune_mask(s, 0.5)
    assert m.sum(axis=1).tolist() == [32] * 6
    assert all(s[r][m[r]].min() >= s[r][~m[r]].max() for r in range(6))
    m24 = prune.prune_mask(s, 0.5, "n2of4").reshape(6, 16, 4)
    assert (m24.sum(axis=2) == 2).all()
    m48 = prune.prune_mask(s, 0.5, "n4of8").reshape(6, 8, 8)
    assert (m48.sum(axis=2) == 4).all()
    with pytest.raises(ValueError):
        prune.prune_mask(s[:, :30], 0.5, "n2of4")


def test_prune_methods(base, tmp_path):
    out = str(tmp_path / "p.gguf")
    rep = prune.prune_gguf(base, out, "magnitude", sparsity=0.5)
    g = load_gguf(out)
    w = decode_f32(g, "blk.0.ffn_down.weight")
    assert abs((w == 0).mean() - 0.5) < 0.01 and abs(rep["pruned"]["blk.0.ffn_down.weight"] - 0.5) < 0.01
    assert not (decode_f32(g, "token_embd.weight") == 0).any()  # protected by default
    a, b = _logits(base), _logits(out)
    assert torch.isfinite(b).all() and 0 < (a - b).abs().max()
    # Wanda: calibration norms change which weights survive
    llm = LLM.from_gguf(base, EngineConfig(**EC), device="cpu")
    norms = prune.collect_activation_norms(llm, [list(range(3, 60)), [7, 8, 9, 10, 11]])
    assert norms["blk.0.attn_q.weight"].shape == (256,) and norms["blk.1.ffn_down.weight"].shape == (512,)
    assert np.array_equal(norms["blk.0.attn_q.weight"], norms["blk.0.attn_v.weight"])
    outw = str(tmp_path / "w.gguf")
    prune.prune_gguf(base, outw, "wanda", sparsity=0.5, pattern="n2of4", calibration=norms)
    ww = decode_f32(load_gguf(outw), "blk.0.ffn_down.weight")
    assert ((ww.reshape(-1, 4) != 0).sum(axis=1) <= 2).all()
    assert ((ww == 0) != (w == 0)).any()
    with pytest.raises(ValueError):
        prune.prune_gguf(base, outw, "wanda", sparsity=0.5)
    # name filter: drop one layer's FFN, dry run writes nothing
    rep = prune.prune_gguf(base, None, "name-filter", drop=["blk.1.ffn"], dry_run=True)
    assert len(rep["removed"]) == 4 and all("blk.1.ffn" in n for n in rep["removed"])
    outn = str(tmp_path / "n.gguf")
    assert cli_main(["prune", "--input", base, "--output", outn, "--keep", "blk.0", "--keep", "token_embd"]) == 0
    assert all(n.startswith("blk.0") or n.startswith("token_embd") for n in load_gguf(outn).tensors)


def _fake_hf(path, seed, bf16=False):
    rng = np.random.default_rng(seed)
    os.makedirs(path, exist_ok=True)
    t = {"model.embed_tokens.weight": rng.standard_normal((50, 16)).astype(np.float32),
         "model.layers.0.self_attn.q_proj.weight": rng.standard_normal((16, 16)).astype(np.float32),
         "model.layers.0.mlp.up_proj.weight": rng.standard_normal((32, 16)).astype(np.float32),
         "model.layers.0.input_layernorm.weight": np.ones(16, dtype=np.float32),
         "model.position_ids": np.arange(8, dtype=np.int64)}
    dtypes = {}
    if bf16:
        k = "model.layers.0.mlp.up_proj.weight"
        t[k] = merge.f32_to_bf16_bits(t[k])
        dtypes[k] = "BF16"
    save_file(t, os.path.join(path, "model.safetensors"), {"format": "pt"}, dtypes)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump({"model_type": "llama"}, f)
    return t


def test_merge_linear_slerp_and_shards(tmp_path):
    a_dir, b_dir = str(tmp_path / "a"), str(tmp_path / "b")
    ta, tb = _fake_hf(a_dir, 1, bf16=True), _fake_hf(b_dir, 2, bf16=True)
    out = str(tmp_path / "lin.safetensors")
    rep = merge.merge_checkpoints(a_dir, b_dir, out, "linear", t=0.25)
    assert rep["blended"] == 4 and rep["tensors"] == 5
    f = SafeTensorsFile(out)
    q = "model.layers.0.self_attn.q_proj.weight"
    assert np.allclose(f.tensor_f32(q), 0.75 * ta[q] + 0.25 * tb[q], atol=1e-6)
    assert f.dtype("model.layers.0.mlp.up_proj.weight") == "BF16" and np.array_equal(f.tensor("model.position_ids"), np.arange(8))
    # per-category weights: attention 0.3, mlp 0.5, other 0.4
    merge.merge_checkpoints(a_dir, b_dir, out, "linear")
    f = SafeTensorsFile(out)
    assert np.allclose(f.tensor_f32(q), 0.7 * ta[q] + 0.3 * tb[q], atol=1e-6)
    e = "model.embed_tokens.weight"
    assert np.allclose(f.tensor_f32(e), 0.6 * ta[e] + 0.4 * tb[e], atol=1e-6)
    # SLERP: end points, norm between the inputs' norms, and not the chord
    x, y = ta[q], tb[q]
    assert np.allclose(merge.slerp(x, y, 0.0), x, atol=1e-5) and np.allclose(merge.slerp(x, y, 1.0), y, atol=1e-5)
    mid = merge.slerp(x, y, 0.5)
    assert abs(np.linalg.norm(mid) - 0.5 * (np.linalg.norm(x) + np.linalg.norm(y))) < 1e-3
    assert np.linalg.norm(mid) > np.linalg.norm(0.5 * (x + y))
    assert np.allclose(merge.slerp(x, 2 * x, 0.5), 1.5 * x, atol=1e-5)  # parallel: linear
    # sharded directory output with an index and the side files of A
    out_dir = str(tmp_path / "merged")
    rep = merge.merge_checkpoints(a_dir, b_dir, out_dir, "slerp", max_shard_gib=3e-6)
    assert len(rep["files"]) > 1 and os.path.exists(os.path.join(out_dir, "config.json"))
    idx = json.load(open(os.path.join(out_dir, "model.safetensors.index.json")))
    assert set(idx["weight_map"]) == set(ta)
    back = merge.open_checkpoint(out_dir)
    assert np.allclose(back[q][0].tensor_f32(q), merge.slerp(x, y, 0.3), atol=1e-6)
    # one-sided tensors and shape mismatches
    tb2 = dict(tb)
    tb2["extra.weight"] = np.ones((2, 2), dtype=np.float32)
    tb2.pop("model.layers.0.mlp.up_proj.weight")
    tb2["model.layers.0.mlp.up_proj.weight"] = merge.f32_to_bf16_bits(np.ones((32, 16), dtype=np.float32))
    save_file(tb2, os.path.join(b_dir, "model.safetensors"), None, {"model.layers.0.mlp.up_proj.weight": "BF16"})
    with pytest.raises(ValueError):
        merge.merge_checkpoints(a_dir, b_dir, out, "linear")
    assert merge.merge_checkpoints(a_dir, b_dir, None, "linear", missing="keep-b", dry_run=True)["tensors"] == 6
    assert merge.merge_checkpoints(a_dir, b_dir, None, "linear", missing="skip", dry_run=True)["tensors"] == 5
    assert cli_main(["merge", "--a", a_dir, "--b", b_dir, "--dry-run"]) == 2  # missing tensor, policy error


def test_lora_merge_from_a_peft_directory(base, tmp_path):
    rng = np.random.default_rng(3)
    r = 4
    A = rng.standard_normal((r, 256)).astype(np.float32) * 0.05
    B = rng.standard_normal((256, r)).astype(np.float32) * 0.05
    ad = tmp_path / "adapter"
    ad.mkdir()
    save_file({"base_model.model.model.layers.1.self_attn.q_proj.lora_A.weight": A,
               "base_model.model.model.layers.1.self_attn.q_proj.lora_B.weight": B}, str(ad / "adapter_model.safetensors"))
    (ad / "adapter_config.json").write_text(json.dumps({"r": r, "lora_alpha": 8, "target_modules": ["q_proj"]}))
    out = str(tmp_path / "merged.gguf")
    changed = lora.merge_lora_gguf(base, str(ad), out)
    assert changed == ["blk.1.attn_q.weight"]
    w0, w1 = decode_f32(load_gguf(base), "blk.1.attn_q.weight"), decode_f32(load_gguf(out), "blk.1.attn_q.weight")
    assert np.allclose(w1, w0 + 2.0 * (B @ A), atol=1e-5)
    assert np.array_equal(decode_f32(load_gguf(base), "blk.0.attn_q.weight"), decode_f32(load_gguf(out), "blk.0.attn_q.weight"))
    assert not torch.allclose(_logits(base), _logits(out))
    # an adapter for a tensor the checkpoint lacks is refused
    save_file({"base_model.model.model.layers.9.self_attn.q_proj.lora_A.weight": A,
               "base_model.model.model.layers.9.self_attn.q_proj.lora_B.weight": B}, str(ad / "adapter_model.safetensors"))
    assert cli_main(["lora-merge", "--base", base, "--adapter", str(ad), "--output", out]) == 2


def test_perplexity_orders_checkpoints_by_damage(base, tmp_path, capsys):
    """token_logprobs agrees with next_token_logits, and perplexity of a text the model itself wrote rises as the
    checkpoint is pruned harder."""
    llm = LLM.from_gguf(base, EngineConfig(**EC), device="cpu")
    text = llm.generate([[5, 9, 20, 31, 7]], SamplingParams(temperature=0.0, max_tokens=60, ignore_eos=True))[0]
    ids = text.prompt_token_ids + text.token_ids
    lp = llm.token_logprobs(ids, chunk=16)  # several chunks
    assert lp.shape == (len(ids) - 1,)
    row = torch.log_softmax(torch.from_numpy(llm.next_token_logits([ids[:10]]))[0].double(), -1)
    assert abs(float(row[ids[10]]) - lp[9]) < 1e-4
    assert np.allclose(lp, llm.token_logprobs(ids, chunk=256), atol=1e-5)
    ppl = {0.0: llm.perplexity(ids)}
    for sp_ in (0.5, 0.9):
        out = str(tmp_path / f"p{sp_}.gguf")
        prune.prune_gguf(base, out, "magnitude", sparsity=sp_)
        ppl[sp_] = LLM.from_gguf(out, EngineConfig(**EC), device="cpu").perplexity(ids)
    assert ppl[0.0] < ppl[0.5] < ppl[0.9]
    f = tmp_path / "t.txt"
    f.write_text(llm.tokenizer.decode_without_special_tokens(ids))
    assert cli_main(["perplexity", base, "--file", str(f), "--ctx", "32", "--backend", "cpu", "--json"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["windows"] >= 2 and rep["perplexity"] > 1.0
    with pytest.raises(ValueError):
        llm.token_logprobs([1])


def test_csv_classifier(tmp_path, capsys):
    from oxidize_b200.offline import classifier as CL

    rng = np.random.default_rng(0)
    centers = {"red": (2.0, 0.0, 50.0), "green": (-2.0, 1.0, 10.0), "blue": (0.0, -3.0, 90.0)}
    lines = ["x,y,z,colour"]
    for name, c in centers.items():
        for _ in range(60):
            p = rng.normal(c, (0.5, 0.5, 5.0))
            lines.append(f"{p[0]:.4f},{p[1]:.4f},{p[2]:.4f},{name}")
    rng.shuffle(lines[1:])
    f = tmp_path / "d.csv"
    f.write_text("\n".join(lines) + "\n")
    data = CL.load_csv_dataset(str(f))
    assert data.inputs.shape == (180, 3) and sorted(data.classes) == ["blue", "green", "red"]
    model, hist = CL.train_classifier(data, epochs=30, hidden_size=32, learning_rate=1e-2)
    acc, loss = CL.evaluate_classifier(model, data)
    assert hist[-1] < 0.3 * hist[0] and acc > 0.97
    assert data.classes[int(model.predict(np.array([[2.0, 0.0, 50.0]]))[0])] == "red"
    assert cli_main(["train-classifier", "--train-csv", str(f), "--epochs", "5", "--eval-csv", str(f), "--save", str(tmp_path / "m.pt")]) == 0
    assert "accuracy" in capsys.readouterr().out and (tmp_path / "m.pt").exists()
    # label in the first column, integer labels, no header
    g = tmp_path / "n.csv"
    g.write_text("\n".join(f"{i % 2},{(i % 2) * 2 - 1 + rng.normal(0, 0.1):.3f}" for i in range(40)) + "\n")
    d2 = CL.load_csv_dataset(str(g), label_column=0)
    assert d2.inputs.shape == (40, 1) and len(d2.classes) == 2
    bad = tmp_path / "bad.csv"
    bad.write_text("1,2,a\n3,x,a\n")
    assert cli_main(["train-classifier", "--train-csv", str(bad)]) == 2
