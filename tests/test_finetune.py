"""LoRA / QLoRA trainer: its dense differentiable forward against the engine, learning, export + merge, exact resume,
self-training round."""
import json
import os

import numpy as np
import pytest
import torch

from oxidize_b200.cli.main import main as cli_main
from oxidize_b200.engine.llm import LLM, EngineConfig
from oxidize_b200.engine.sampler import SamplingParams
from oxidize_b200.formats.gguf import load_gguf
from oxidize_b200.formats.tokenizer import load_tokenizer_from_metadata
from oxidize_b200.models.config import config_from_gguf, preset
from oxidize_b200.models.weights import load_weights
from oxidize_b200.offline import finetune as ft
from oxidize_b200.offline.lora import merge_lora_gguf
from oxidize_b200.utils.synth import synth_gguf

EC = dict(max_model_len=128, max_num_seqs=2, num_kv_blocks=32, prefill_chunk_size=32, max_num_batched_tokens=32)
SMALL = dict(n_layers=2, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96)


def _model(path, lora=None, qlora=False):
    g = load_gguf(path)
    cfg = config_from_gguf(g)
    return ft.LoraModel(load_weights(g, cfg, "cpu", torch.float32), lora or ft.LoraConfig(), qlora), g


@pytest.mark.parametrize("family", ["llama", "qwen3-bias", "gemma3"])
def test_training_forward_matches_the_engine(family, tmp_path):
    if family == "llama":
        cfg = preset("tiny-llama", **SMALL)
    elif family == "qwen3-bias":
        cfg = preset("tiny-llama", arch="qwen3", qk_norm=True, attn_bias=True, rope_dim=8, **SMALL)
    else:
        cfg = preset("gemma3-27b", **{**SMALL, "n_layers": 3}, sliding_window=8, sliding_window_pattern=2, embedding_scale=8.0,
                     attn_scale=0.2, context_length=4096)
    path = str(tmp_path / "m.gguf")
    synth_gguf(path, cfg, "F32", seed=2, norm_jitter=0.2)
    model, _ = _model(path)
    ids = list(range(5, 45))
    with torch.no_grad():
        mine = model(torch.tensor([ids]))[0, -1]
    llm = LLM.from_gguf(path, EngineConfig(**EC), device="cpu")
    want = torch.from_numpy(llm.next_token_logits([ids]))[0]
    assert (mine - want).abs().max() / want.abs().max() < 1e-4


def _overfit_setup(tmp_path, quant="F32"):
    path = str(tmp_path / "base.gguf")
    synth_gguf(path, preset("tiny-llama", **SMALL), quant, seed=1, norm_jitter=0.1)
    tok = load_tokenizer_from_metadata(load_gguf(path).metadata)
    data = tmp_path / "sft.jsonl"
    data.write_text(json.dumps({"prompt": "hello there ", "completion": "general kenobi"}) + "\n"
                    + json.dumps({"text": "a b c d e f"}) + "\n")
    return path, tok, str(data)


def test_lora_learns_exports_and_merges(tmp_path):
    path, tok, data = _overfit_setup(tmp_path)
    # (the head is a target too: with N(0, 0.02) weights behind a final norm the base head cannot produce a confident logit)
    lora = ft.LoraConfig(r=8, alpha=16, targets=("q_proj", "v_proj", "down_proj", "lm_head"))
    model, g = _model(path, lora)
    ex = ft.load_examples(data, tok, None, 64)
    assert len(ex) == 2 and ex[0].loss_from == len(tok.encode("hello there ")) and ex[1].loss_from == 1
    before = float(ft.batch_loss(model, ex[:1]))
    tr = ft.Trainer(model, ft.TrainConfig(steps=60, batch_size=1, lr=2e-2, seed=0))
    losses = tr.train(ex[:1])
    assert losses[-1] < 0.05 * before
    # B starts at zero: before training the adapter is the identity
    fresh, _ = _model(path, lora)
    assert abs(float(ft.batch_loss(fresh, ex[:1])) - before) < 1e-6
    # export in the PEFT layout, fold into the GGUF, and the serving engine now writes the learned completion
    adapter = model.save_adapter(str(tmp_path / "adapter"))
    cfgj = json.load(open(os.path.join(adapter, "adapter_config.json")))
    assert cfgj["r"] == 8 and cfgj["target_modules"] == ["q_proj", "v_proj", "down_proj", "lm_head"]
    merged = str(tmp_path / "merged.gguf")
    assert len(merge_lora_gguf(path, adapter, merged)) == 7
    want = tok.encode("general kenobi")
    llm = LLM.from_gguf(merged, EngineConfig(**EC), device="cpu")
    got = llm.generate([tok.encode("hello there ")], SamplingParams(temperature=0.0, max_tokens=len(want), ignore_eos=True))[0].token_ids
    assert got == want
    assert ft.generate_with_adapter(model, tok.encode("hello there "), len(want)) == want


def test_resume_continues_the_exact_run(tmp_path):
    path, tok, data = _overfit_setup(tmp_path)
    ex = ft.load_examples(data, tok, None, 64)
    cfg = ft.TrainConfig(batch_size=1, lr=1e-3, seed=5)
    straight = ft.Trainer(_model(path)[0], cfg)
    straight.train(ex, 6)
    first = ft.Trainer(_model(path)[0], cfg)
    first.train(ex, 3)
    ck = first.save_checkpoint(str(tmp_path / "ck"))
    second = ft.Trainer(_model(path)[0], cfg)
    second.load_checkpoint(ck)
    assert second.state.step == 3
    second.train(ex, 3)
    for k in straight.model.A:
        assert torch.equal(straight.model.A[k], second.model.A[k]) and torch.equal(straight.model.B[k], second.model.B[k])
    assert straight.state.losses == second.state.losses
    other = ft.Trainer(_model(path, ft.LoraConfig(r=4))[0], cfg)
    with pytest.raises(Exception):
        other.load_checkpoint(ck)


def test_qlora_keeps_the_base_encoded(tmp_path):
    path, tok, data = _overfit_setup(tmp_path, "Q8_0")
    model, _ = _model(path, qlora=True)
    ex = ft.load_examples(data, tok, None, 64)
    tr = ft.Trainer(model, ft.TrainConfig(batch_size=2, lr=5e-3))
    losses = tr.train(ex, 12)
    assert losses[-1] < losses[0]
    lw = model.w.layers[0]
    assert lw.wqkv.parts[0].qtype == "Q8_0" and lw.wqkv.parts[0]._dense is None and model.w.embed._dense is None
    assert all(p.grad is None or torch.isfinite(p.grad).all() for p in model.parameters())


def test_self_training_round_and_cli(tmp_path):
    path, tok, data = _overfit_setup(tmp_path)
    model, _ = _model(path)
    tr = ft.Trainer(model, ft.TrainConfig(batch_size=2, lr=1e-3))
    log = str(tmp_path / "self.jsonl")
    rep = ft.self_train_round(tr, tok, ["hello there", "a b c"], max_new=6, steps=2, min_tokens=2, log_path=log)
    assert rep["round"] == 1 and rep["generated"] == 2 and rep["accepted"] >= 1 and rep["loss_last"] is not None
    assert all("prompt" in json.loads(l) for l in open(log))
    none = ft.self_train_round(tr, tok, ["hello there"], max_new=6, steps=2, must_match="this never appears")
    assert none["accepted"] == 0 and none["round"] == 2
    out = str(tmp_path / "run")
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("hello there\n")
    rc = cli_main(["finetune", "--model", path, "--data", data, "--output", out, "--steps", "3", "--batch-size", "2",
                   "--self-train-rounds", "1", "--prompts", str(prompts), "--self-train-max-new", "4",
                   "--merge-output", str(tmp_path / "m.gguf")])
    assert rc == 0 and os.path.exists(os.path.join(out, "adapter", "adapter_model.safetensors"))
    assert os.path.exists(os.path.join(out, "round-0000", "trainer_state.pt")) and os.path.exists(tmp_path / "m.gguf")
    rc = cli_main(["finetune", "--model", path, "--data", data, "--output", out, "--steps", "1",
                   "--resume-from", os.path.join(out, "round-0001")])
    assert rc == 0
    # a mixture-of-experts checkpoint is refused with a message, not a traceback
    moe = str(tmp_path / "moe.gguf")
    synth_gguf(moe, preset("mixtral-8x7b", **SMALL, n_experts=4, n_experts_used=2, expert_ffn_size=32), "F32", seed=0)
    assert cli_main(["finetune", "--model", moe, "--data", data, "--output", out]) == 2


def test_preference_training_moves_the_policy_toward_the_chosen_answers(tmp_path):
    path, tok, _ = _overfit_setup(tmp_path)
    prefs = tmp_path / "prefs.jsonl"
    prefs.write_text("\n".join(json.dumps(r) for r in [
        {"prompt": "hello there ", "chosen": "general kenobi", "rejected": "go away"},
        {"prompt": "a b c ", "chosen": "d e f", "rejected": "x y z"}]) + "\n")
    pairs = ft.load_preference_pairs(str(prefs), tok, 64)
    assert len(pairs) == 2 and pairs[0].chosen.loss_from == pairs[0].rejected.loss_from
    model, _ = _model(path, ft.LoraConfig(r=8, alpha=16, targets=("q_proj", "v_proj", "down_proj", "lm_head")))
    loss0, acc0 = ft.dpo_loss(model, pairs, beta=0.5)
    # before training the policy IS the reference: zero margin, loss log 2
    assert abs(float(loss0) - np.log(2)) < 1e-5 and acc0 == 0.0
    tr = ft.Trainer(model, ft.TrainConfig(batch_size=2, lr=5e-3, seed=0))
    losses = tr.train(pairs, 40, dpo_beta=0.5)
    loss1, acc1 = ft.dpo_loss(model, pairs, beta=0.5)
    assert losses[-1] < 0.5 * losses[0] and acc1 == 1.0 and float(loss1) < 0.35
    # the reference policy did not move: with the adapters off the model is still the base
    model.adapters_on = False
    with torch.no_grad():
        base_lp = ft.sequence_logprobs(model, [pairs[0].chosen])
    model.adapters_on = True
    fresh, _ = _model(path, ft.LoraConfig(r=8, alpha=16, targets=("q_proj",)))
    with torch.no_grad():
        assert torch.allclose(base_lp, ft.sequence_logprobs(fresh, [pairs[0].chosen]), atol=1e-5)
    out = str(tmp_path / "run")
    assert cli_main(["finetune", "--model", path, "--dpo-data", str(prefs), "--output", out, "--steps", "2", "--batch-size", "2"]) == 0
    bad = tmp_path / "bad.jsonl"
    bad.write_text(json.dumps({"prompt": "x", "chosen": "y"}) + "\n")
    assert cli_main(["finetune", "--model", path, "--dpo-data", str(bad), "--output", out]) == 2


def test_training_from_scratch_writes_a_checkpoint_the_engine_serves(tmp_path):
    """train-tokenizer -> pretrain -> GGUF -> engine: the loss falls, the exported file computes what the trainer's forward
    computes, and the served model continues a memorised phrase."""
    from oxidize_b200.formats import tokenizer_train as TT
    from oxidize_b200.offline import pretrain as PT

    corpus = tmp_path / "corpus.txt"
    corpus.write_text("the cat sat on the mat. the dog sat on the log. " * 60)
    tokj = tmp_path / "tok.json"
    assert TT.main([str(corpus), "--vocab-size", "300", "--output", str(tokj)]) == 0
    out = str(tmp_path / "tiny.gguf")
    rc = cli_main(["pretrain", "--corpus", str(corpus), "--tokenizer", str(tokj), "--output", out, "--hidden", "64", "--layers", "2",
                   "--heads", "4", "--kv-heads", "2", "--ffn", "128", "--seq-len", "32", "--steps", "120", "--batch-size", "8",
                   "--lr", "1e-2", "--warmup-steps", "5"])
    assert rc == 0
    llm = LLM.from_gguf(out, EngineConfig(**EC), device="cpu")
    assert llm.cfg.tie_embeddings and llm.tokenizer is not None
    text = llm.generate(["the cat sat on"], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))[0].text
    assert "the mat" in text
    assert llm.perplexity("the cat sat on the mat. the dog sat on the log. " * 3) < 3.0
    # the exported file is the trained function: the trainer's forward on the loaded weights gives the engine's logits
    model, _ = _model(out)
    ids = llm.tokenizer.encode("the dog sat on the")
    with torch.no_grad():
        mine = model(torch.tensor([ids]))[0, -1]
    want = torch.from_numpy(llm.next_token_logits([ids]))[0]
    assert (mine - want).abs().max() / want.abs().max() < 1e-4
    # continue from the file, exporting 8-bit matrices
    out2 = str(tmp_path / "more.gguf")
    rc = cli_main(["pretrain", "--corpus", str(corpus), "--tokenizer", str(tokj), "--output", out2, "--init", out, "--seq-len", "32",
                   "--steps", "3", "--quant", "Q8_0"])
    assert rc == 0 and load_gguf(out2).tensors["blk.0.attn_q.weight"].type.name == "Q8_0"
