"""Vision tower + projector against the `transformers` CLIP / LLaVA implementations, image preprocessing, the multimodal
prompt builder, and image tokens through the serving engine (logits against LLaVA end to end)."""
import os

import numpy as np
import pytest
import torch

T = pytest.importorskip("transformers")

from oxidize_b200.engine.llm import LLM, EngineConfig  # noqa: E402
from oxidize_b200.engine.sampler import SamplingParams  # noqa: E402
from oxidize_b200.formats.convert import convert_safetensors_to_gguf  # noqa: E402
from oxidize_b200.vision import ImagePreprocessor, MultimodalPrompt, VisionConfig, convert_vision_tower, load_vision_encoder  # noqa: E402

IMAGE_TOKEN = 190


@pytest.fixture(scope="module")
def llava(tmp_path_factory):
    d = tmp_path_factory.mktemp("llava")
    torch.manual_seed(0)
    vc = T.CLIPVisionConfig(image_size=28, patch_size=7, hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                            num_attention_heads=4, projection_dim=16)
    tc = T.LlamaConfig(vocab_size=199, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, max_position_embeddings=256)
    cfg = T.LlavaConfig(vision_config=vc, text_config=tc, image_token_index=IMAGE_TOKEN, vision_feature_layer=-2,
                        vision_feature_select_strategy="default", image_seq_length=16)
    model = T.LlavaForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.ndim >= 2:
                p.mul_(3.0)
            elif "norm" in n and "weight" in n:
                p.add_(torch.randn_like(p) * 0.2)
            else:
                p.add_(torch.randn_like(p) * 0.05)  # biases away from zero
    src = str(d / "hf")
    model.save_pretrained(src, safe_serialization=True)
    mmproj = convert_vision_tower(src, str(d / "mmproj.gguf"))
    return model, src, mmproj, d


def test_vision_tower_and_projector_match_transformers(llava):
    model, src, mmproj, _ = llava
    enc = load_vision_encoder(mmproj)
    c = enc.config
    assert (c.image_size, c.patch_size, c.hidden_size, c.num_hidden_layers, c.projection_dim, c.feature_layer) == (28, 7, 32, 3, 64, -2)
    assert c.num_image_tokens == 16 and not c.use_gelu
    pixels = torch.randn(3, 28, 28)
    with torch.no_grad():
        out = model.model.vision_tower(pixels[None], output_hidden_states=True)
        want_h = [h[0] for h in out.hidden_states]
        feats = model.model.get_image_features(pixel_values=pixels[None])
        want = (feats.pooler_output if hasattr(feats, "pooler_output") else feats)
        want = want[0] if isinstance(want, (list, tuple)) else want
        want = want.reshape(-1, 64)
    got_h = enc.hidden_states(pixels)
    assert len(got_h) == len(want_h) == 4
    for a, b in zip(got_h, want_h):
        assert torch.allclose(a, b, atol=2e-5)
    assert torch.allclose(enc.encode(pixels), want, atol=2e-5)


def test_preprocessing():
    cfg = VisionConfig(image_size=28, patch_size=7, hidden_size=32, num_attention_heads=4, num_hidden_layers=1, intermediate_size=64,
                       projection_dim=16)
    pre = ImagePreprocessor(cfg)
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, (28, 28, 3), dtype=np.uint8)
    x = pre(img)
    mean, std = torch.tensor(cfg.image_mean)[:, None, None], torch.tensor(cfg.image_std)[:, None, None]
    want = (torch.from_numpy(img).permute(2, 0, 1).float() / 255 - mean) / std
    assert torch.allclose(x, want, atol=1e-6)
    # RGBA and greyscale inputs, resize + centre crop of a non-square image
    assert torch.allclose(pre(np.concatenate([img, img[:, :, :1]], axis=2)), want)
    assert pre(img[:, :, 0]).shape == (3, 28, 28)
    assert pre(rng.integers(0, 256, (60, 90, 3), dtype=np.uint8)).shape == (3, 28, 28)
    # patch rows are the convolution's receptive fields in raster order
    p = pre.patches(x)
    assert p.shape == (16, 147) and torch.equal(p[5].reshape(3, 7, 7), x[:, 7:14, 7:14])
    with pytest.raises(ValueError):
        pre(np.zeros((4, 4, 2)))
    with pytest.raises(ValueError):
        VisionConfig(image_size=30, patch_size=7).validate()


def test_image_tokens_through_the_engine_match_llava(llava, tmp_path):
    model, src, mmproj, d = llava
    # the language model: the checkpoint's text part, converted like any other
    path = convert_safetensors_to_gguf(src, str(tmp_path / "lm.gguf"), "F32")
    llm = LLM.from_gguf(path, EngineConfig(kv_cache_dtype="f32", max_model_len=128, max_num_seqs=2, num_kv_blocks=32,
                                           prefill_chunk_size=8, max_num_batched_tokens=8), device="cpu")
    enc = load_vision_encoder(mmproj)
    pixels = torch.randn(3, 28, 28, generator=torch.Generator().manual_seed(3))
    before, after = [5, 9, 20, 31], [7, 11, 80]
    ids = before + [IMAGE_TOKEN] * 16 + after
    with torch.no_grad():
        want = model(input_ids=torch.tensor([ids]), pixel_values=pixels[None]).logits[0, -1]
    emb = enc.encode(pixels)
    llm.runner.keep_logits = True
    llm.add_request(ids, SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True), input_embeds=emb,
                    embed_positions=list(range(4, 20)))
    got = None
    while llm.has_unfinished:  # three prefill chunks of 8 rows: the image tokens straddle chunk boundaries
        llm.step()
        lg = llm.last_step[1].logits
        if lg is not None and lg.shape[0] == 1:
            got = lg.float()[0]
    assert (got - want).abs().max() / want.abs().max() < 2e-5
    # without the image rows the same ids give different logits; the placeholder ids do not enter the prefix cache
    plain = torch.from_numpy(llm.next_token_logits([ids]))[0]
    assert (plain - want).abs().max() / want.abs().max() > 1e-3
    assert llm.scheduler.finished[-1].num_cached_tokens == 0
    with pytest.raises(ValueError):
        llm.add_request(ids, None, input_embeds=emb, embed_positions=list(range(4, 19)))
    with pytest.raises(ValueError):
        llm.add_request(ids, None, input_embeds=emb[:, :32], embed_positions=list(range(4, 20)))


def test_multimodal_prompt_builder(llava, tmp_path):
    from oxidize_b200.formats.gguf import load_gguf
    from oxidize_b200.formats.tokenizer import load_tokenizer_from_metadata
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    p = str(tmp_path / "t.gguf")
    synth_gguf(p, preset("tiny-llama", n_layers=1, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96),
               "F32", seed=0)
    tok = load_tokenizer_from_metadata(load_gguf(p).metadata)
    img = torch.randn(16, 64)
    ids, pos, rows = MultimodalPrompt().add_text("hello ").add_image(img).add_text("there").add_image(img[:3]).build(tok, 299, add_bos=False)
    n0 = len(tok.encode("hello "))
    assert pos == list(range(n0, n0 + 16)) + list(range(len(ids) - 3, len(ids))) and rows.shape == (19, 64)
    assert all(ids[i] == 299 for i in pos) and 299 not in [t for i, t in enumerate(ids) if i not in pos]
    with pytest.raises(ValueError):
        MultimodalPrompt().build(tok, 299)
    with pytest.raises(ValueError):
        MultimodalPrompt().add_image(torch.zeros(0, 64))


def test_cli_image_prompt(llava, tmp_path):
    """`oxidize run MODEL "describe <image> please" --image F --mmproj P` builds the spliced prompt and generates."""
    from PIL import Image

    from oxidize_b200.cli.main import image_prompt
    from oxidize_b200.models.config import preset
    from oxidize_b200.utils.synth import synth_gguf

    _, _, mmproj, _ = llava
    p = str(tmp_path / "lm.gguf")
    synth_gguf(p, preset("tiny-llama", n_layers=1, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_size=96),
               "F32", seed=0)
    img = str(tmp_path / "x.png")
    Image.fromarray(np.random.default_rng(0).integers(0, 256, (40, 50, 3), dtype=np.uint8)).save(img)
    llm = LLM.from_gguf(p, EngineConfig(max_model_len=128, max_num_seqs=2, num_kv_blocks=32), device="cpu")
    ids, pos, rows = image_prompt(llm, mmproj, img, "describe <image> please")
    assert rows.shape == (16, 64) and len(pos) == 16 and pos[0] > 0 and pos[-1] < len(ids) - 1
    out = llm.generate([(ids, pos, rows)], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))[0]
    assert len(out.token_ids) == 4
    other = llm.generate([(ids, pos, rows * 0)], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))[0]
    assert other.prompt_token_ids == ids
    with pytest.raises(SystemExit):
        image_prompt(llm, None, img, "x")


def test_chat_completions_with_image_parts(llava, tmp_path):
    """OpenAI-style image parts (base64 data URLs) and the `images` field reach the model as image tokens."""
    import base64
    import io

    from fastapi.testclient import TestClient
    from PIL import Image

    from oxidize_b200.engine.async_engine import AsyncEngine
    from oxidize_b200.models.config import preset
    from oxidize_b200.serving.app import GenerationDefaults, ServerState, create_app
    from oxidize_b200.utils.synth import synth_gguf

    _, _, mmproj, _ = llava
    p = str(tmp_path / "lm.gguf")
    synth_gguf(p, preset("tiny-llama", arch="qwen2", n_layers=1, vocab_size=300, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16,
                         ffn_size=96), "F32", seed=0)
    llm = LLM.from_gguf(p, EngineConfig(max_model_len=256, max_num_seqs=2, num_kv_blocks=64), device="cpu")
    eng = AsyncEngine(llm)
    try:
        def b64(seed):
            buf = io.BytesIO()
            Image.fromarray(np.random.default_rng(seed).integers(0, 256, (30, 30, 3), dtype=np.uint8)).save(buf, format="PNG")
            return base64.b64encode(buf.getvalue()).decode()

        def ask(client, content, **extra):
            return client.post("/v1/chat/completions", json={"model": "m", "max_tokens": 4, "temperature": 0,
                                                             "messages": [{"role": "user", "content": content, **extra}]})

        with_vision = TestClient(create_app(ServerState(eng, "m", GenerationDefaults(), api_keys=[], vision=load_vision_encoder(mmproj))))
        parts = [{"type": "text", "text": "what is "}, {"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64(1)}},
                 {"type": "text", "text": " ?"}]
        r = with_vision.post("/v1/chat/completions", json={"model": "m", "max_tokens": 4, "temperature": 0,
                                                          "messages": [{"role": "user", "content": parts}]})
        assert r.status_code == 200
        text_only = ask(with_vision, "what is  ?").json()
        # 16 image tokens entered the prompt (the text around them is tokenized in two pieces, which may cost a token)
        assert abs(r.json()["usage"]["prompt_tokens"] - text_only["usage"]["prompt_tokens"] - 16) <= 2
        r2 = ask(with_vision, "describe", images=[b64(2)])
        assert r2.status_code == 200 and r2.json()["usage"]["prompt_tokens"] > 16
        assert ask(with_vision, [{"type": "image_url", "image_url": {"url": "https://example.com/x.png"}}]).status_code == 400
        assert ask(with_vision, [{"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}]).status_code == 400
        assert ask(with_vision, [{"type": "audio", "audio": "x"}]).status_code == 400
        no_vision = TestClient(create_app(ServerState(eng, "m", GenerationDefaults(), api_keys=[])))
        assert ask(no_vision, parts).status_code == 400 and ask(no_vision, "plain text").status_code == 200
    finally:
        eng.shutdown()
