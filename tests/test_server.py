"""HTTP API: routes, SSE framing, auth, limits, metrics, realtime WS — with and without a model
(the no-model placeholder behaviour mirrors the reference's route tests, oxidize-server/src/app.rs:146-430)."""
import io
import json

import numpy as np
import pytest
from starlette.testclient import TestClient

from oxidize_b200.engine.async_engine import AsyncEngine
from oxidize_b200.engine.llm import LLM, EngineConfig
from oxidize_b200.engine.server_control import install_suppressed_tokens, suppressed_generation_tokens
from oxidize_b200.models.config import preset
from oxidize_b200.serving.app import GenerationDefaults, ServerState, create_app, trim_stop_text
from oxidize_b200.serving.middleware import (AuditLogger, LimitConfig, RequestLimiter, key_is_valid, load_api_keys)
from oxidize_b200.utils.synth import synth_gguf


@pytest.fixture(scope="module")
def engine(tmp_path_factory):
    cfg = preset("tiny-llama", n_layers=2, vocab_size=300)
    p = str(tmp_path_factory.mktemp("srv") / "tiny.gguf")
    synth_gguf(p, cfg, "F16", seed=0)
    llm = LLM.from_gguf(p, EngineConfig(max_model_len=256, max_num_seqs=4, num_kv_blocks=96, prefill_chunk_size=32,
                                        max_num_batched_tokens=64), device="cpu")
    install_suppressed_tokens(llm)
    eng = AsyncEngine(llm)
    yield eng
    eng.shutdown()


def test_probes_and_placeholder_without_model():
    c = TestClient(create_app(ServerState(api_keys=[])))
    assert c.get("/healthz").status_code == 200 and c.get("/livez").status_code == 200
    assert c.get("/readyz").status_code == 503
    r = c.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": "hi"}]})
    assert r.status_code == 200 and r.json()["object"] == "chat.completion"
    assert "placeholder" in r.json()["choices"][0]["message"]["content"]
    r = c.post("/v1/completions", json={"model": "m", "prompt": "x", "guided_choice": ["yes", "no"]})
    assert r.json()["choices"][0]["text"] == "yes"
    r = c.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": "hi"}], "n": 2})
    assert r.status_code == 400
    assert c.get("/v1/models").json()["data"][0]["id"] == "oxidize-default"
    assert c.post("/v1/embeddings", json={"input": "a"}).json()["data"][0]["embedding"] == []
    assert "paths" in c.get("/openapi.json").json()
    body = c.get("/metrics").text
    assert "oxidize_requests_total" in body and "oxidize_request_duration_seconds" in body


def test_placeholder_stream_framing():
    c = TestClient(create_app(ServerState(api_keys=[])))
    with c.stream("POST", "/v1/chat/completions",
                  json={"model": "m", "stream": True, "messages": [{"role": "user", "content": "hi"}]}) as r:
        lines = [l for l in r.iter_lines() if l]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert all(ch["object"] == "chat.completion.chunk" for ch in chunks)
    assert chunks[-1]["choices"][0]["finish_reason"] == "stop"


def test_auth_and_limits():
    st = ServerState(api_keys=["secret"], limits=LimitConfig(max_requests_per_second=1000, max_in_flight=1, max_queued=0))
    c = TestClient(create_app(st))
    assert c.get("/healthz").status_code == 200  # probes stay open
    assert c.get("/v1/models").status_code == 401
    assert c.get("/v1/models", headers={"x-api-key": "secret"}).status_code == 200
    assert c.get("/v1/models", headers={"authorization": "Bearer secret"}).status_code == 200
    assert c.get("/v1/models", headers={"authorization": "Bearer nope"}).status_code == 401
    assert key_is_valid("a", ["b", "a"]) and not key_is_valid(None, ["a"])
    assert load_api_keys({"OXIDIZE_API_KEY": "k1", "OXIDIZE_API_KEYS": "k2, k3"}) == ["k1", "k2", "k3"]
    now = [0.0]
    lim = RequestLimiter(LimitConfig(max_requests_per_second=2, max_in_flight=8, max_queued=8), clock=lambda: now[0])
    assert lim.try_acquire() is None and lim.try_acquire() is None and lim.try_acquire() == "rate_limited"
    now[0] += 1.0
    assert lim.try_acquire() is None
    lim2 = RequestLimiter(LimitConfig(max_requests_per_second=100, max_in_flight=1, max_queued=1))
    assert lim2.try_acquire() is None and lim2.try_acquire() is None and lim2.try_acquire() == "queue_full"
    lim2.release()
    assert lim2.try_acquire() is None


def test_completion_with_model(engine):
    buf = io.StringIO()
    st = ServerState(engine, "tiny", GenerationDefaults(max_tokens=8, temperature=0.0), api_keys=[],
                     audit=AuditLogger(stream=buf))
    c = TestClient(create_app(st))
    assert c.get("/readyz").status_code == 200
    r = c.post("/v1/completions", json={"model": "tiny", "prompt": "hello", "max_tokens": 6})
    assert r.status_code == 200
    body = r.json()
    assert body["object"] == "text_completion" and body["usage"]["completion_tokens"] >= 1
    assert body["usage"]["total_tokens"] == body["usage"]["prompt_tokens"] + body["usage"]["completion_tokens"]
    r2 = c.post("/v1/completions", json={"model": "tiny", "prompt": "hello", "max_tokens": 6})
    assert r2.json()["choices"][0]["text"] == body["choices"][0]["text"]  # greedy is reproducible
    rec = [json.loads(l) for l in buf.getvalue().splitlines()]
    assert rec and rec[0]["event"] == "request" and rec[0]["model"] == "tiny" and "duration_ms" in rec[0]
    assert "oxidize_tokens_generated_total" in c.get("/metrics").text
    r = c.post("/v1/completions", json={"model": "tiny", "prompt": "x", "top_p": 2.0})
    assert r.status_code == 400


def test_embeddings_with_model(engine):
    """/v1/embeddings returns pooled, L2-normalised hidden states of the loaded model, computed on the engine thread."""
    c = TestClient(create_app(ServerState(engine, "tiny", GenerationDefaults(), api_keys=[])))
    r = c.post("/v1/embeddings", json={"model": "tiny", "input": ["hello world", "something else entirely", "hello world"]})
    assert r.status_code == 200
    body = r.json()
    vecs = [np.asarray(d["embedding"], dtype=np.float64) for d in body["data"]]
    assert [d["index"] for d in body["data"]] == [0, 1, 2] and body["usage"]["prompt_tokens"] > 0
    assert all(v.shape == (512,) and abs(np.linalg.norm(v) - 1.0) < 1e-4 for v in vecs)
    assert np.allclose(vecs[0], vecs[2]) and not np.allclose(vecs[0], vecs[1], atol=1e-3)
    assert c.post("/v1/embeddings", json={"model": "tiny", "input": ""}).status_code == 400
    # a generation request still works afterwards (the call ran between engine steps, on a cache of its own)
    assert c.post("/v1/completions", json={"model": "tiny", "prompt": "hello", "max_tokens": 3}).status_code == 200


def test_chat_stream_with_model(engine):
    st = ServerState(engine, "tiny", GenerationDefaults(max_tokens=8, temperature=0.0), api_keys=[])
    c = TestClient(create_app(st))
    with c.stream("POST", "/v1/chat/completions", json={"model": "tiny", "stream": True, "max_tokens": 5,
                                                        "messages": [{"role": "user", "content": "hi"}]}) as r:
        lines = [l for l in r.iter_lines() if l]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"].get("role") == "assistant"
    assert chunks[-1]["choices"][0]["finish_reason"] in ("stop", "length")


def test_realtime_websocket(engine):
    st = ServerState(engine, "tiny", GenerationDefaults(max_tokens=4, temperature=0.0), api_keys=[])
    c = TestClient(create_app(st))
    with c.websocket_connect("/v1/realtime") as ws:
        assert ws.receive_json()["type"] == "session.created"
        ws.send_json({"type": "session.update", "session": {"instructions": "be brief", "max_response_output_tokens": 4}})
        assert ws.receive_json()["type"] == "session.updated"
        ws.send_json({"type": "conversation.item.create", "item": {"role": "user", "content": "hello"}})
        assert ws.receive_json()["type"] == "conversation.item.created"
        ws.send_json({"type": "response.create"})
        kinds = []
        while True:
            ev = ws.receive_json()
            kinds.append(ev["type"])
            if ev["type"] == "response.done":
                break
        assert kinds[0] == "response.created" and "response.text.done" in kinds
        ws.send_json({"type": "bogus"})
        assert ws.receive_json()["type"] == "error"


def test_suppressed_tokens_and_stop_trim(engine):
    llm = engine.llm
    ids = suppressed_generation_tokens(llm.tokenizer, llm.cfg.vocab_size)
    st = llm.tokenizer.special_tokens
    assert st.unk in ids and st.bos in ids and st.eos not in ids
    assert len(ids) > 10  # "<123>" style pieces of the synthetic vocabulary
    assert llm.weights.lm_head.bias is not None and float(llm.weights.lm_head.bias[ids[0]]) == float("-inf")
    assert trim_stop_text("hello END world", ["END", "zzz"]) == "hello "
    assert trim_stop_text("abc", []) == "abc"


def test_guided_choice_and_penalty_fields_with_model(engine):
    st = ServerState(engine, "tiny", GenerationDefaults(max_tokens=12, temperature=0.8), api_keys=[])
    c = TestClient(create_app(st))
    tok = st.tokenizer
    if tok is None or engine.llm.eos_token_id is None:
        pytest.skip("synthetic model has no tokenizer / EOS")
    choices = ["yes", "no", "maybe"]
    for seed in range(3):
        r = c.post("/v1/completions", json={"model": "tiny", "prompt": "answer:", "guided_choice": choices, "seed": seed,
                                            "max_tokens": 12})
        assert r.status_code == 200, r.text
        ids = tok.encode_with_special_tokens(r.json()["choices"][0]["text"], add_bos=False)
        assert any(ids == tok.encode_with_special_tokens(ch, add_bos=False) for ch in choices), r.json()
    r = c.post("/v1/completions", json={"model": "tiny", "prompt": "hello", "max_tokens": 6, "temperature": 0.5, "seed": 1,
                                        "frequency_penalty": 0.5, "presence_penalty": 0.5})
    assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] >= 1


def test_data_parallel_replicas_behind_one_front(tmp_path):
    """Two engine replicas behind the router: requests spread over both, results equal a single engine's (greedy),
    an unhealthy replica is avoided, and the HTTP layer serves through the router unchanged."""
    import threading

    from oxidize_b200.engine.async_engine import ReplicaRouter
    from oxidize_b200.engine.sampler import SamplingParams

    cfg = preset("tiny-llama", n_layers=2, vocab_size=300)
    p = str(tmp_path / "tiny_dp.gguf")
    synth_gguf(p, cfg, "F16", seed=0)
    ec = EngineConfig(max_model_len=256, max_num_seqs=4, num_kv_blocks=96, prefill_chunk_size=32, max_num_batched_tokens=64)
    engines = [AsyncEngine(LLM.from_gguf(p, ec, device="cpu"), name=f"rep{i}") for i in range(2)]
    router = ReplicaRouter(engines)
    try:
        sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
        prompts = [[5, 9, 200, 31, 7], list(range(3, 40)), [100, 101], [7, 7, 7, 7], [250, 3, 9]]
        served = []
        lock = threading.Lock()
        results = {}

        def run(i):
            evs = router.generate_blocking(prompts[i], sp, timeout=60)
            with lock:
                results[i] = [t for ev in evs for t in ev.new_token_ids]

        orig = [e.submit for e in engines]
        for k, e in enumerate(engines):
            e.submit = (lambda k, f: (lambda *a, **kw: (served.append(k), f(*a, **kw))[1]))(k, orig[k])
        ts = [threading.Thread(target=run, args=(i,)) for i in range(len(prompts))]
        for t in ts:
            t.start()
        for t in ts:
            t.join(90)
        assert sorted(results) == list(range(len(prompts)))
        assert set(served) == {0, 1}, "both replicas must take requests"
        single = LLM.from_gguf(p, ec, device="cpu").generate(prompts, sp)
        assert [results[i] for i in range(len(prompts))] == [o.token_ids for o in single]
        assert router.load() == [0, 0] and router.healthy
        # a replica whose watchdog tripped gets no new requests
        class _Down:
            healthy = False

            def close(self):
                pass

        real, engines[0].watchdog = engines[0].watchdog, _Down()
        served.clear()
        router.generate_blocking(prompts[0], sp, timeout=60)
        assert served == [1]
        engines[0].watchdog = real
        c = TestClient(create_app(ServerState(router, "tiny", GenerationDefaults(max_tokens=6, temperature=0.0), api_keys=[])))
        r = c.post("/v1/completions", json={"model": "tiny", "prompt": "hello", "max_tokens": 5})
        assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] >= 1
        assert c.get("/readyz").status_code == 200
    finally:
        router.shutdown()


def test_cors_origin():
    c = TestClient(create_app(ServerState(api_keys=[], cors_origin="https://app.example")))
    r = c.options("/v1/chat/completions", headers={"origin": "https://app.example", "access-control-request-method": "POST",
                                                    "access-control-request-headers": "content-type"})
    assert r.status_code == 200 and r.headers["access-control-allow-origin"] == "https://app.example"
    r = c.get("/healthz", headers={"origin": "https://app.example"})
    assert r.headers.get("access-control-allow-origin") == "https://app.example"
    assert "access-control-allow-origin" not in c.get("/healthz", headers={"origin": "https://other.example"}).headers
    plain = TestClient(create_app(ServerState(api_keys=[])))
    assert "access-control-allow-origin" not in plain.get("/healthz", headers={"origin": "https://app.example"}).headers
