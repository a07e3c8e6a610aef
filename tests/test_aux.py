"""CLI surface, converter, SafeTensors IO, auto-tuner, GPU-cluster manifests, pipeline split (all CPU).

Mirrors the reference's unit tests for the same pieces: CLI rewriting (`oxidize/src/cli.rs`),
auto-tuner tiers with synthetic inventories (`oxidize-core/src/autotune.rs`), GPU classification
(`oxidize/src/gpu_cluster.rs`), pipeline layer split (`oxidize-core/src/pipeline.rs`).
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# --------------------------------------------------------------------------- CLI
def test_cli_rewrites_verbs():
    from oxidize_b200.cli.main import rewrite_args

    assert rewrite_args(["run", "m.gguf", "hello", "world", "--max-tokens", "7"]) == [
        "--verb", "run", "--model", "m.gguf", "--prompt", "hello world", "--max-tokens", "7"]
    assert rewrite_args(["serve", "m.gguf", "--port=9"]) == ["--verb", "serve", "--model", "m.gguf", "--api-only", "--port=9"]
    assert rewrite_args(["chat", "m.gguf"])[-1] == "--chat"
    # a boolean flag must not swallow the positional that follows it
    assert rewrite_args(["run", "--json", "m.gguf", "hi"]) == ["--verb", "run", "--model", "m.gguf", "--prompt", "hi", "--json"]
    assert rewrite_args(["--model", "x"]) == ["--model", "x"]


def test_cli_parser_keeps_reference_flag_names():
    from oxidize_b200.cli.main import build_parser, user_passed

    p = build_parser()
    a = p.parse_args(["--model", "m", "--ctx-size", "2048", "--temperature", "0.5", "--top-k", "10", "--kv-cache-dtype", "q8",
                      "--port", "8081", "--draft-model", "d.gguf", "--draft-tokens", "3", "--tp", "2"])
    assert a.ctx_size == 2048 and a.temperature == 0.5 and a.top_k == 10 and a.kv_cache_dtype == "q8" and a.port == 8081
    assert a.draft_model == "d.gguf" and a.draft_tokens == 3 and a.tp == 2
    passed = user_passed(["--ctx-size", "2048", "--top-k=10"])
    assert "ctx_size" in passed and "top_k" in passed and "temperature" not in passed


def test_cli_run_and_show_end_to_end(tmp_path):
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    cfg = preset("tiny-llama", n_layers=1, vocab_size=300, n_heads=4, n_kv_heads=2)
    path = str(tmp_path / "tiny.gguf")
    synth_gguf(path, cfg, "F32", seed=3, tokenizer=True)
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "oxidize_b200.cli.main", "run", path, "hello", "--max-tokens", "4", "--backend",
                        "cpu", "--temperature", "0", "--no-auto"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    r2 = subprocess.run([sys.executable, "-m", "oxidize_b200.cli.main", "show", path], capture_output=True, text=True, env=env,
                        timeout=300)
    assert r2.returncode == 0, r2.stderr[-2000:]
    assert "llama" in r2.stdout.lower()


# --------------------------------------------------------------------------- SafeTensors + converter
def test_safetensors_roundtrip_and_errors(tmp_path):
    from oxidize_b200.formats.safetensors_io import SafeTensorsError, SafeTensorsFile, save_file

    t = {"a": np.arange(12, dtype=np.float32).reshape(3, 4), "b": np.arange(6, dtype=np.float16),
         "c": (np.arange(8, dtype=np.float32) * 0.5).astype(np.float32)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, metadata={"format": "pt"})
    f = SafeTensorsFile(p)
    assert sorted(f.keys()) == ["a", "b", "c"]
    assert f.shape("a") == (3, 4) and f.dtype("b") == "F16"
    np.testing.assert_array_equal(f.tensor("a"), t["a"])
    np.testing.assert_array_equal(f.tensor_f32("b"), t["b"].astype(np.float32))
    bad = str(tmp_path / "bad.safetensors")
    with open(bad, "wb") as fh:
        fh.write((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafeTensorsError):
        SafeTensorsFile(bad)


def test_convert_hf_directory_to_gguf_and_run(tmp_path):
    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.engine.sampler import SamplingParams
    from oxidize_b200.formats.convert import convert_safetensors_to_gguf
    from oxidize_b200.formats.gguf import load_gguf
    from oxidize_b200.formats.safetensors_io import save_file

    rng = np.random.default_rng(0)
    H, F, L, V, nh, nkv = 64, 128, 2, 96, 4, 2
    hd = H // nh
    t = {"model.embed_tokens.weight": rng.normal(0, 0.05, (V, H)).astype(np.float32),
         "model.norm.weight": np.ones(H, dtype=np.float32),
         "lm_head.weight": rng.normal(0, 0.05, (V, H)).astype(np.float32)}
    for i in range(L):
        pre = f"model.layers.{i}."
        t[pre + "input_layernorm.weight"] = np.ones(H, dtype=np.float32)
        t[pre + "post_attention_layernorm.weight"] = np.ones(H, dtype=np.float32)
        t[pre + "self_attn.q_proj.weight"] = rng.normal(0, 0.05, (nh * hd, H)).astype(np.float32)
        t[pre + "self_attn.k_proj.weight"] = rng.normal(0, 0.05, (nkv * hd, H)).astype(np.float32)
        t[pre + "self_attn.v_proj.weight"] = rng.normal(0, 0.05, (nkv * hd, H)).astype(np.float32)
        t[pre + "self_attn.o_proj.weight"] = rng.normal(0, 0.05, (H, nh * hd)).astype(np.float32)
        t[pre + "mlp.gate_proj.weight"] = rng.normal(0, 0.05, (F, H)).astype(np.float32)
        t[pre + "mlp.up_proj.weight"] = rng.normal(0, 0.05, (F, H)).astype(np.float32)
        t[pre + "mlp.down_proj.weight"] = rng.normal(0, 0.05, (H, F)).astype(np.float32)
    src = tmp_path / "hf"
    src.mkdir()
    save_file(t, str(src / "model.safetensors"))
    json.dump({"architectures": ["LlamaForCausalLM"], "hidden_size": H, "intermediate_size": F, "num_hidden_layers": L,
               "num_attention_heads": nh, "num_key_value_heads": nkv, "vocab_size": V, "rms_norm_eps": 1e-5,
               "rope_theta": 10000.0, "max_position_embeddings": 256}, open(src / "config.json", "w"))
    out = str(tmp_path / "m.gguf")
    convert_safetensors_to_gguf(str(src), out, quant="F16")
    g = load_gguf(out)
    assert g.metadata["general.architecture"] == "llama"
    assert g.metadata["llama.block_count"] == L and g.metadata["llama.attention.head_count_kv"] == nkv
    assert "blk.1.ffn_down.weight" in g.tensors and "token_embd.weight" in g.tensors
    llm = LLM.from_gguf(out, EngineConfig(max_model_len=64, max_num_seqs=2, num_kv_blocks=16), device="cpu")
    o = llm.generate([[1, 2, 3, 4]], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    assert len(o[0].token_ids) == 3


# --------------------------------------------------------------------------- auto-tuner
def _fp(weight_gb, **kw):
    from oxidize_b200.utils.autotune import ModelFingerprint

    base = dict(arch="llama", n_layers=80, hidden_size=8192, n_heads=64, n_kv_heads=8, head_dim=128, is_moe=False,
                n_experts=0, weight_bytes=int(weight_gb * 1e9), context_length=8192, has_mtp=False, dominant_quant="BF16")
    base.update(kw)
    fields = ModelFingerprint.__dataclass_fields__.keys()
    return ModelFingerprint(**{k: v for k, v in base.items() if k in fields})


def test_autotune_tiers_with_synthetic_inventories():
    from oxidize_b200.utils.autotune import GpuInfo, HardwareInventory, apply_plan, parse_nvidia_smi_csv, plan

    gpus = parse_nvidia_smi_csv("0, NVIDIA B200, 183359\n1, NVIDIA B200, 183359\nbogus line\n")
    assert [g.index for g in gpus] == [0, 1] and gpus[0].memory_bytes == 183359 << 20
    eight = HardwareInventory(64, 2 << 40, [GpuInfo(i, "NVIDIA B200", 183359 << 20) for i in range(8)])
    p70 = plan(eight, _fp(141))
    assert p70.backend == "cuda" and p70.tp_size == 1 or p70.tp_size in (2, 4, 8)
    assert p70.kv_cache_dtype in ("bf16", "q8", "q4") and p70.num_kv_blocks > 0
    big = plan(eight, _fp(800))
    assert big.tp_size == 8
    cpu = plan(HardwareInventory(16, 64 << 30, []), _fp(4))
    assert cpu.backend == "cpu" and not cpu.cuda_graphs and cpu.threads == 16
    mtp = plan(eight, _fp(30, has_mtp=True))
    assert mtp.speculative == "mtp"
    # explicit beats implicit
    merged = apply_plan({"tp": 2, "kv_cache_dtype": "bf16", "ctx_size": 0}, {"tp"}, big)
    assert merged["tp"] == 2 and merged["kv_cache_dtype"] == big.kv_cache_dtype and merged["ctx_size"] == big.ctx_size
    assert "Rationale" in big.render() and json.loads(big.to_json())["tp_size"] == 8


# --------------------------------------------------------------------------- GPU cluster helper
def test_gpu_cluster_classification_and_manifests():
    from oxidize_b200.utils.gpu_cluster import classify_gpu, classify_inventory, render_cluster_manifests

    assert classify_gpu("NVIDIA B200") == "b200"
    assert classify_gpu("NVIDIA A100-SXM4-80GB") == "a100"
    assert classify_gpu("NVIDIA RTX PRO 6000 Blackwell Workstation Edition") == "rtx-pro-6000"
    assert classify_gpu("Some Unknown Accelerator") is None
    inv = classify_inventory(["NVIDIA B200"] * 8 + ["Quadro K620"])
    assert inv.get("b200") == 8
    files = render_cluster_manifests("prod", "b200", 2)
    text = "\n".join(files.values()) if isinstance(files, dict) else str(files)
    assert "nvidia.com/gpu" in text and "prod" in text


# --------------------------------------------------------------------------- pipeline split / launcher
def test_pipeline_layer_split_covers_all_layers():
    from oxidize_b200.parallel.pp import split_layers

    for n_layers, n_stages in [(80, 2), (80, 3), (32, 4), (5, 5), (7, 2)]:
        parts = split_layers(n_layers, n_stages)
        assert len(parts) == n_stages and parts[0][0] == 0 and parts[-1][1] == n_layers
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        sizes = [hi - lo for lo, hi in parts]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        split_layers(2, 3)


def test_torchrun_command_uses_loopback():
    from oxidize_b200.parallel.launcher import free_port, torchrun_command

    cmd = torchrun_command(4, ["serve", "m.gguf", "--tp", "4"], port=29999)
    s = " ".join(cmd)
    assert "--nproc-per-node" in s and "4" in cmd and "127.0.0.1" in s and "29999" in s and "serve" in cmd
    assert 1024 < free_port() < 65536


# --------------------------------------------------------------------------- decode profiler / tracing
def test_decode_profiler_and_value_trace(tmp_path):
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    cfg = preset("tiny-llama", n_layers=2, vocab_size=300, n_heads=4, n_kv_heads=2)
    path = str(tmp_path / "tiny.gguf")
    synth_gguf(path, cfg, "F32", seed=3)
    env = dict(os.environ, PYTHONPATH=ROOT, OXIDIZE_DECODE_PROFILE="1", OXIDIZE_TRACE_FWD="1")
    r = subprocess.run([sys.executable, "-m", "oxidize_b200.cli.main", "run", path, "hello", "--max-tokens", "3", "--backend",
                        "cpu", "--temperature", "0", "--no-auto"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "[trace] layer   1" in r.stderr
    assert "operator" in r.stderr and "linear" in r.stderr and "paged_attention" in r.stderr


def test_prefill_token_budget_follows_tile_waves():
    """The step's token budget is picked so that the projections' tile grids fill whole waves of SMs."""
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.autotune import prefill_token_budget

    big = preset("llama3-70b")
    # per-rank shapes change with the tensor-parallel degree, and so does the best budget
    got = {tp: prefill_token_budget(big, tp) for tp in (1, 2, 4, 8)}
    assert all(2048 <= v <= 3072 and v % 256 == 0 for v in got.values())
    assert got[1] == 2304  # nine token tiles fill the last wave of every projection better than eight
    # a toy model whose grids never fill one wave: the wave is paid anyway, so the largest budget is the most efficient
    tiny = preset("tiny-llama")
    assert prefill_token_budget(tiny, 1) == 3072
    assert prefill_token_budget(big, 8, lo=1024, hi=1024) == 1024


def test_guard_bands_catch_writes_outside_a_buffer():
    """The canary allocator names the buffer that was written before its start or past its end."""
    import torch

    from oxidize_b200.utils.guards import GUARD_BYTES, GuardedAllocator, MemoryGuardError

    g = GuardedAllocator()
    a = g.empty(100, torch.float32, "cpu", "partials")
    b = g.empty(7, torch.int32, "cpu", "tickets", zero=True)
    assert a.numel() == 100 and b.numel() == 7 and int(b.sum()) == 0 and len(g) == 2
    a.fill_(1.0)
    b.fill_(3)
    g.verify()  # writes inside the payload leave the bands alone
    # an overrun of three floats past the end of `a` (the storage behind the view is the guarded allocation)
    raw = torch.tensor([], dtype=torch.uint8).set_(a.untyped_storage())
    raw[GUARD_BYTES + 400 + 5] = 0
    with pytest.raises(MemoryGuardError, match="partials: written 5 bytes past its end"):
        g.verify()
    raw[GUARD_BYTES + 400 + 5] = 0xA5
    g.verify()
    rawb = torch.tensor([], dtype=torch.uint8).set_(b.untyped_storage())
    rawb[GUARD_BYTES - 1] = 1
    with pytest.raises(MemoryGuardError, match="tickets: written before its start"):
        g.verify()
    g.forget(b)
    g.verify()
    assert len(g) == 1


def test_config_file_and_environment_layers(tmp_path, monkeypatch):
    """defaults < plan < YAML < OXIDIZE_CFG_* < explicit flags; the file's engine: section reaches EngineConfig."""
    from oxidize_b200.cli import main as M

    cfgf = tmp_path / "serve.yaml"
    cfgf.write_text("ctx-size: 96\nmax_running: 3\ntemperature: 0.25\nkv-cache-dtype: q8\nengine:\n  async_decode: false\n  resident_layers: 1\n")
    parser = M.build_parser()
    argv = M.rewrite_args(["run", "m.gguf", "hi", "--config", str(cfgf), "--temperature", "0.9"])
    passed = M.user_passed(argv)
    args = parser.parse_args(argv)
    monkeypatch.setenv("OXIDIZE_CFG_MAX_RUNNING", "5")
    extra = M.apply_config_file(args, passed, parser)
    assert args.ctx_size == 96 and args.kv_cache_dtype == "q8"
    assert args.max_running == 5  # the environment beats the file
    assert args.temperature == 0.9  # the command line beats both
    assert {"ctx_size", "max_running", "kv_cache_dtype"} <= passed and extra == {"async_decode": False, "resident_layers": 1}
    bad = tmp_path / "bad.yaml"
    bad.write_text("no-such-flag: 1\n")
    args2 = parser.parse_args(M.rewrite_args(["run", "m.gguf", "hi", "--config", str(bad)]))
    with pytest.raises(SystemExit):
        M.apply_config_file(args2, set(), parser)
    # end to end: the engine section lands in the engine's configuration
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    monkeypatch.delenv("OXIDIZE_CFG_MAX_RUNNING")
    model = str(tmp_path / "m.gguf")
    synth_gguf(model, preset("tiny-llama", n_layers=2, vocab_size=300, hidden_size=64, n_heads=2, n_kv_heads=2, head_dim=32, ffn_size=96),
               "F32", seed=0)
    argv = M.rewrite_args(["run", model, "hi", "--config", str(cfgf), "--backend", "cpu"])
    passed = M.user_passed(argv)
    args = parser.parse_args(argv)
    args.engine_extra = M.apply_config_file(args, passed, parser)
    llm, _ = M.make_engine(args, passed)
    assert llm.config.max_model_len == 96 and llm.config.max_num_seqs == 3 and llm.config.async_decode is False
    assert llm.config.resident_layers == 1 and llm.kv.spec.dtype_name == "q8"


def test_hf_directory_is_converted_on_the_fly_with_its_tokenizer(tmp_path, monkeypatch):
    """`oxidize run HF_DIR "..."`: SafeTensors + config.json + tokenizer.json become a GGUF in the model directory once;
    the converted tokenizer encodes like the `tokenizers` library does on the same file."""
    T = pytest.importorskip("transformers")
    import json

    from oxidize_b200.cli import main as M
    from oxidize_b200.formats import tokenizer_train as TT
    from oxidize_b200.formats.convert import tokenizer_metadata_from_hf
    from oxidize_b200.formats.tokenizer import load_tokenizer_from_metadata

    corpus = "the quick brown fox jumps over the lazy dog. " * 30 + "déjà vu café. " * 10
    md = TT.train_bpe([corpus], 320)
    toks, merges = md["tokenizer.ggml.tokens"], md["tokenizer.ggml.merges"]
    src = tmp_path / "hf"
    torch_seed = 0
    import torch

    torch.manual_seed(torch_seed)
    T.LlamaForCausalLM(T.LlamaConfig(vocab_size=len(toks), hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                     num_attention_heads=4, num_key_value_heads=2)).save_pretrained(str(src), safe_serialization=True)
    n_special = 2
    (src / "tokenizer.json").write_text(json.dumps({
        "version": "1.0", "truncation": None, "padding": None,
        "added_tokens": [{"id": len(toks) - n_special + i, "content": toks[len(toks) - n_special + i], "single_word": False,
                          "lstrip": False, "rstrip": False, "normalized": False, "special": True} for i in range(n_special)],
        "normalizer": None, "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": True},
        "post_processor": None, "decoder": {"type": "ByteLevel", "add_prefix_space": True, "trim_offsets": True, "use_regex": True},
        "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": None, "end_of_word_suffix": None,
                  "fuse_unk": False, "byte_fallback": False, "vocab": {t: i for i, t in enumerate(toks[: len(toks) - n_special])},
                  "merges": merges}}))
    (src / "tokenizer_config.json").write_text(json.dumps({"bos_token": "<|bos|>", "eos_token": {"content": "<|eos|>"},
                                                           "chat_template": "{% for message in messages %}{{ message.content }}{% endfor %}"}))
    got = tokenizer_metadata_from_hf(str(src))
    assert got["tokenizer.ggml.tokens"] == toks and got["tokenizer.ggml.merges"] == merges
    assert got["tokenizer.ggml.eos_token_id"] == len(toks) - 1 and got["tokenizer.ggml.bos_token_id"] == len(toks) - 2
    assert "chat_template" in "".join(got)
    mine = load_tokenizer_from_metadata(got)
    try:
        from tokenizers import Tokenizer

        theirs = Tokenizer.from_file(str(src / "tokenizer.json"))
        for text in ("the quick brown fox", "a lazy café, déjà vu!"):
            assert mine.encode(text) == theirs.encode(text, add_special_tokens=False).ids
    except ImportError:
        pass
    monkeypatch.setattr(M, "MODEL_DIR", str(tmp_path / "models"))
    path = M.resolve_model(str(src))
    assert path.endswith(".gguf") and os.path.dirname(path) == str(tmp_path / "models")
    assert M.resolve_model(str(src)) == path and len(os.listdir(tmp_path / "models")) == 1  # reused, not converted again
    from oxidize_b200.engine.llm import LLM, EngineConfig
    from oxidize_b200.engine.sampler import SamplingParams

    llm = LLM.from_gguf(path, EngineConfig(max_model_len=64, max_num_seqs=1, num_kv_blocks=8), device="cpu")
    assert llm.tokenizer is not None and llm.eos_token_id == len(toks) - 1 and llm.chat_template
    out = llm.generate(["the quick brown"], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))[0]
    assert len(out.token_ids) == 3
    empty = tmp_path / "empty"
    empty.mkdir()
    (empty / "config.json").write_text("{}")
    with pytest.raises(SystemExit):
        M.resolve_model(str(empty))


def test_offload_planner_and_mapping_hints(tmp_path):
    from oxidize_b200.formats.gguf import load_gguf
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils import autotune
    from oxidize_b200.utils.synth import synth_gguf

    GB = 1 << 30
    assert autotune.plan_resident_layers(80, 2 * GB, 4 * GB, 20 * GB, 200 * GB) == 0  # fits
    assert autotune.plan_resident_layers(80, 2 * GB, 4 * GB, 20 * GB, 100 * GB) == 37  # (100 - 4 - 20 - 2) / 2
    assert autotune.plan_resident_layers(80, 2 * GB, 4 * GB, 20 * GB, 10 * GB) == 1  # never less than one
    assert autotune.plan_resident_layers(4, 2 * GB, 1 * GB, 1 * GB, 9 * GB) == 2
    p = str(tmp_path / "m.gguf")
    synth_gguf(p, preset("tiny-llama", n_layers=1, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96),
               "F32", seed=0)
    g = load_gguf(p)
    assert "willneed" in g.advise(willneed=True, hugepages=True)  # huge pages may be refused for a file mapping: not an error
    assert g.advise() == []
