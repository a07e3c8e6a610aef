"""OpenAI-compatible HTTP API (FastAPI): chat / text completions with SSE streaming, models,
embeddings stub, health probes, Prometheus metrics, OpenAPI document and the realtime
WebSocket.

Route set, request fields and response shapes follow the reference server
(``oxidize-server/src/app.rs:47-63``, ``schema.rs:7-131``, ``routes/responses.rs:19-59,134-198``):
``n`` / ``best_of`` > 1 are rejected, ``stop`` may be a string or a list, the final SSE chunk
carries ``finish_reason`` and is followed by ``data: [DONE]``, ``/readyz`` answers 503 until a
model is loaded, ``/v1/embeddings`` returns an empty vector without a model (pooled hidden states with one), and without a model the completion
routes answer with placeholder text (``AGENTS.md:220``).  Middleware order is limits → API key →
metrics → logging, as at ``app.rs:64-76``.
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, Dict, List, Optional, Union

from fastapi import FastAPI, Request, WebSocket, WebSocketDisconnect
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse
from pydantic import BaseModel, Field

from ..engine.async_engine import AsyncEngine, StreamEvent
from ..engine.sampler import SamplingError, SamplingParams
from ..formats.tokenizer import chat_template_from_metadata, render_chat_template
from .middleware import (OPEN_PATHS, AuditLogger, LimitConfig, Metrics, RequestLimiter, extract_key, key_is_valid,
                         load_api_keys)

PLACEHOLDER_TEXT = "This is a placeholder response: no model is loaded."


class ChatMessage(BaseModel):
    role: str
    # a string, or OpenAI-style parts: {"type": "text", "text": ...} / {"type": "image_url", "image_url": {"url": "data:..."}}
    content: Union[str, List[Dict[str, Any]]] = ""
    images: Optional[List[str]] = None  # base64 images shown in front of the message's text


class _Common(BaseModel):
    model: str = "oxidize-default"
    response_format: Optional[Dict[str, Any]] = None
    guided_json: Optional[Any] = None
    json_schema: Optional[Any] = None
    guided_regex: Optional[str] = None
    guided_choice: Optional[List[str]] = None
    stream: bool = False
    max_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    min_p: Optional[float] = None
    typical_p: Optional[float] = None
    tail_free_z: Optional[float] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    mirostat_tau: Optional[float] = None
    mirostat_eta: Optional[float] = None
    stop: Optional[Union[str, List[str]]] = None
    seed: Optional[int] = None
    n: Optional[int] = None
    best_of: Optional[int] = None


class ChatCompletionRequest(_Common):
    messages: List[ChatMessage]
    max_completion_tokens: Optional[int] = None


class CompletionRequest(_Common):
    prompt: str
    echo: bool = False


class EmbeddingsRequest(BaseModel):
    model: str = "oxidize-default"
    input: Union[str, List[str]] = ""


class GenerationDefaults(BaseModel):
    max_tokens: int = 512
    temperature: float = 0.8
    top_p: Optional[float] = None
    top_k: Optional[int] = None


class ServerState:
    def __init__(self, engine: Optional[AsyncEngine] = None, model_id: str = "oxidize-default",
                 defaults: Optional[GenerationDefaults] = None, api_keys: Optional[List[str]] = None,
                 limits: Optional[LimitConfig] = None, audit: Optional[AuditLogger] = None,
                 chat_template: Optional[str] = None, vision=None, cors_origin: Optional[str] = None):
        self.engine = engine
        self.vision = vision  # vision.VisionEncoder: image parts of chat messages become image tokens
        self.cors_origin = cors_origin  # origin allowed to call the API from a browser ("*": any); None: no CORS headers
        self.model_id = model_id
        self.defaults = defaults or GenerationDefaults()
        self.api_keys = load_api_keys() if api_keys is None else api_keys
        self.limiter = RequestLimiter(limits)
        self.metrics = Metrics()
        self.audit = audit or AuditLogger(enabled=False)
        self.chat_template = chat_template
        self.created = int(time.time())

    @property
    def tokenizer(self):
        return None if self.engine is None else self.engine.llm.tokenizer


def _error(status: int, message: str, kind: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"error": {"message": message, "type": kind, "code": status}}, status_code=status)


def _stops(stop) -> List[str]:
    if stop is None:
        return []
    return [stop] if isinstance(stop, str) else [s for s in stop if s]


def trim_stop_text(text: str, stops: List[str]) -> str:
    idx = [text.find(s) for s in stops if s and s in text]
    return text[: min(idx)] if idx else text


def build_sampling(req: _Common, state: ServerState, max_tokens: Optional[int]) -> SamplingParams:
    d = state.defaults
    tok = state.tokenizer
    stop_seqs = []
    if tok is not None:
        for s in _stops(req.stop):
            ids = tok.encode_with_special_tokens(s, add_bos=False)
            if ids:
                stop_seqs.append(tuple(ids))
    p = SamplingParams(temperature=d.temperature if req.temperature is None else req.temperature,
                       top_p=d.top_p if req.top_p is None else req.top_p,
                       top_k=d.top_k if req.top_k is None else req.top_k, min_p=req.min_p, typical_p=req.typical_p,
                       tail_free_z=req.tail_free_z, seed=req.seed, max_tokens=max_tokens or d.max_tokens,
                       frequency_penalty=max(0.0, req.frequency_penalty or 0.0),
                       presence_penalty=max(0.0, req.presence_penalty or 0.0), mirostat_tau=req.mirostat_tau,
                       mirostat_eta=req.mirostat_eta or 0.1,
                       stop_sequences=tuple(stop_seqs))
    if req.guided_choice and tok is not None:
        # the answer must be exactly one of the choices: a grammar whose alternatives are their token ids
        from ..engine.constrained import TokenGrammar

        alts = [tok.encode_with_special_tokens(c, add_bos=False) for c in req.guided_choice if c]
        eos = getattr(getattr(state.engine, "llm", None), "eos_token_id", None)
        if alts and eos is not None:
            p.grammar = TokenGrammar({"root": [list(a) for a in alts if a]}, eos_token_ids=[eos])
            p.stop_token_ids = tuple(set(p.stop_token_ids) | {eos})
    p.validate()
    return p


def create_app(state: Optional[ServerState] = None) -> FastAPI:
    state = state or ServerState()
    app = FastAPI(title="oxidize-b200", version="0.1.0", openapi_url="/openapi.json", docs_url=None, redoc_url=None)
    app.state.server = state
    if state.cors_origin:
        from fastapi.middleware.cors import CORSMiddleware

        app.add_middleware(CORSMiddleware, allow_origins=[state.cors_origin], allow_methods=["GET", "POST", "OPTIONS"],
                           allow_headers=["authorization", "content-type", "x-api-key"])

    # ------------------------------------------------------------------ middleware (outermost last)
    @app.middleware("http")
    async def limits_and_auth(request: Request, call_next):
        path = request.url.path
        t0 = time.perf_counter()
        m = state.metrics
        status = 500
        m.in_flight.inc()
        acquired = False
        try:
            if path not in OPEN_PATHS:
                cl = request.headers.get("content-length")
                if cl is not None and cl.isdigit() and int(cl) > state.limiter.cfg.max_body_bytes:
                    status = 413
                    return _error(413, "request body too large")
                why = state.limiter.try_acquire()
                if why is not None:
                    m.rate_limited.labels(why).inc()
                    status = 429
                    return _error(429, "too many requests" if why == "rate_limited" else "server queue is full",
                                  "rate_limit_error")
                acquired = True
                if state.api_keys and not key_is_valid(extract_key(request.headers), state.api_keys):
                    state.audit.security("auth_failed", path, request.client.host if request.client else None)
                    status = 401
                    return _error(401, "invalid or missing API key", "authentication_error")
            resp = await call_next(request)
            status = resp.status_code
            return resp
        finally:
            if acquired:
                state.limiter.release()
            m.in_flight.dec()
            m.requests_total.labels(request.method, path, str(status)).inc()
            m.request_duration.labels(request.method, path).observe(time.perf_counter() - t0)
            if state.engine is not None:
                m.queue_depth.set(state.engine.queue_depth)

    # ------------------------------------------------------------------ probes
    @app.get("/healthz")
    async def healthz():
        return {"status": "ok"}

    @app.get("/livez")
    async def livez():
        return {"status": "ok"}

    @app.get("/readyz")
    async def readyz():
        if state.engine is None:
            return JSONResponse({"status": "no model loaded"}, status_code=503)
        if not state.engine.healthy:
            return JSONResponse({"status": "engine unhealthy"}, status_code=503)
        return {"status": "ready"}

    @app.get("/metrics")
    async def metrics():
        if state.engine is not None:
            pool = state.engine.llm.pool
            state.metrics.queue_depth.set(state.engine.queue_depth)
        return PlainTextResponse(state.metrics.render(), media_type="text/plain; version=0.0.4")

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": state.model_id, "object": "model", "created": state.created,
                                            "owned_by": "oxidize"}]}

    @app.post("/v1/embeddings")
    async def embeddings(req: EmbeddingsRequest):
        inputs = [req.input] if isinstance(req.input, str) else list(req.input)
        if state.engine is None:
            vecs, n_tok = [[] for _ in inputs], 0
        else:
            if not inputs or any(not isinstance(t, str) or not t for t in inputs):
                return _error(400, "input must be a non-empty string or a list of non-empty strings")
            tok = state.engine.llm.tokenizer
            n_tok = sum(len(tok.encode(t)) for t in inputs) if tok is not None else 0
            try:
                # mean-pooled, L2-normalised final hidden states, computed on the engine thread between two steps
                arr = await asyncio.get_running_loop().run_in_executor(None, state.engine.embed, inputs)
            except NotImplementedError as e:
                return _error(501, str(e))
            vecs = [v.tolist() for v in arr]
        return {"object": "list", "model": req.model,
                "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)],
                "usage": {"prompt_tokens": n_tok, "total_tokens": n_tok}}

    # ------------------------------------------------------------------ completions
    def _validate(req: _Common) -> Optional[JSONResponse]:
        if (req.n or 1) > 1 or (req.best_of or 1) > 1:
            return _error(400, "n > 1 and best_of > 1 are not supported")
        return None

    def _placeholder(req: _Common) -> str:
        if req.guided_choice:
            return req.guided_choice[0]
        rf = (req.response_format or {}).get("type") if req.response_format else None
        if req.guided_json is not None or req.json_schema is not None or rf in ("json_object", "json_schema"):
            return "{}"
        return PLACEHOLDER_TEXT

    IMAGE_MARK = "<image>"

    def _decode_image(src: str):
        """A data URL or bare base64 → RGB array.  Remote URLs are not fetched."""
        import base64
        import io

        from PIL import Image

        if src.startswith("data:"):
            src = src.split(",", 1)[1] if "," in src else ""
        elif src.startswith(("http://", "https://", "file:")):
            raise ValueError("image URLs are not fetched: send the image as a base64 data URL")
        try:
            return Image.open(io.BytesIO(base64.b64decode(src, validate=False))).convert("RGB")
        except Exception as e:  # noqa: BLE001 - any decoder error is the client's
            raise ValueError(f"cannot decode image: {e}") from None

    def _chat_prompt(messages: List[ChatMessage]):
        """The rendered prompt: a string, or with images (token ids, embedding positions, embedding rows)."""
        tpl = state.chat_template
        if tpl is None and state.engine is not None:
            tpl = getattr(state.engine.llm, "chat_template", None)
        flat, images = [], []
        for m in messages:
            text = ""
            for im in m.images or []:
                images.append(im)
                text += IMAGE_MARK
            if isinstance(m.content, str):
                text += m.content
            else:
                for part in m.content:
                    kind = part.get("type")
                    if kind == "text":
                        text += str(part.get("text", ""))
                    elif kind == "image_url":
                        url = part.get("image_url")
                        images.append(url.get("url", "") if isinstance(url, dict) else str(url or ""))
                        text += IMAGE_MARK
                    else:
                        raise ValueError(f"unsupported content part type {kind!r}")
            flat.append({"role": m.role, "content": text})
        prompt = render_chat_template(tpl, flat, True)
        if not images or state.engine is None:
            return prompt
        if state.vision is None:
            raise ValueError("this server was started without a vision tower (--mmproj): image parts cannot be read")
        from ..vision import ImagePreprocessor, MultimodalPrompt

        enc, llm = state.vision, state.engine.llm
        pre = ImagePreprocessor(enc.config)
        pieces = prompt.split(IMAGE_MARK)
        if len(pieces) != len(images) + 1:
            raise ValueError("the text contains the image marker itself")
        mp = MultimodalPrompt().add_text(pieces[0])
        for src, after in zip(images, pieces[1:]):
            mp.add_image(enc.encode(pre(_decode_image(src))))
            mp.add_text(after)
        st = llm.tokenizer.special_tokens
        return mp.build(llm.tokenizer, st.unk if st.unk is not None and st.unk >= 0 else 0)

    async def _run(req: _Common, prompt: str, chat: bool, request: Request, max_tokens: Optional[int], echo: str = ""):
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
        created = int(time.time())
        obj = "chat.completion" if chat else "text_completion"
        key = extract_key(request.headers)
        t0 = time.perf_counter()
        stops = _stops(req.stop)

        def final_body(text: str, reason: str, pt: int, ct: int):
            choice = ({"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": reason} if chat
                      else {"index": 0, "text": echo + text, "finish_reason": reason})
            return {"id": rid, "object": obj, "created": created, "model": req.model, "choices": [choice],
                    "usage": {"prompt_tokens": pt, "completion_tokens": ct, "total_tokens": pt + ct}}

        def chunk(delta: Optional[str], reason: Optional[str], first: bool = False):
            if chat:
                d: Dict[str, Any] = {}
                if first:
                    d["role"] = "assistant"
                if delta:
                    d["content"] = delta
                ch = {"index": 0, "delta": d, "finish_reason": reason}
                o = "chat.completion.chunk"
            else:
                ch = {"index": 0, "text": delta or "", "finish_reason": reason}
                o = "text_completion"
            return "data: " + json.dumps({"id": rid, "object": o, "created": created, "model": req.model,
                                          "choices": [ch]}) + "\n\n"

        if state.engine is None:
            text = _placeholder(req)
            if req.stream:
                async def gen0():
                    yield chunk(text, None, True)
                    yield chunk(None, "stop")
                    yield "data: [DONE]\n\n"
                return StreamingResponse(gen0(), media_type="text/event-stream")
            return JSONResponse(final_body(text, "stop", 0, 0))
        try:
            params = build_sampling(req, state, max_tokens)
        except SamplingError as e:
            return _error(400, str(e))

        def account(ev: StreamEvent, text: str):
            dt = time.perf_counter() - t0
            m = state.metrics
            m.tokens_generated.inc(ev.completion_tokens)
            m.tokens_prompt.inc(ev.prompt_tokens)
            if dt > 0 and ev.completion_tokens:
                m.tokens_per_second.set(ev.completion_tokens / dt)
            m.queue_wait.observe(ev.queue_wait_s)
            if ev.error:
                m.errors.labels("engine").inc()
            state.audit.request(rid, key, req.model, ev.prompt_tokens, ev.completion_tokens, dt, ev.finish_reason,
                                request.url.path, 500 if ev.error else 200)

        if req.stream:
            async def gen():
                acc = ""
                sent = 0
                first = True
                async for ev in state.engine.stream(prompt, params):
                    if ev.error:
                        yield "data: " + json.dumps({"error": {"message": ev.error, "type": "server_error"}}) + "\n\n"
                        account(ev, acc)
                        break
                    acc += ev.text_delta
                    visible = trim_stop_text(acc, stops)
                    stopped = len(visible) < len(acc)
                    if len(visible) > sent or first:
                        yield chunk(visible[sent:], None, first)
                        first = False
                        sent = len(visible)
                    if ev.finished or stopped:
                        reason = "stop" if stopped or ev.finish_reason in ("stop", None) else ev.finish_reason
                        yield chunk(None, reason)
                        account(ev, visible)
                        break
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")

        acc = ""
        last: Optional[StreamEvent] = None
        async for ev in state.engine.stream(prompt, params):
            last = ev
            if ev.error:
                account(ev, acc)
                return _error(500, ev.error, "server_error")
            acc += ev.text_delta
            if len(trim_stop_text(acc, stops)) < len(acc):
                break
        text = trim_stop_text(acc, stops)
        reason = "stop" if (last is None or len(text) < len(acc) or last.finish_reason in ("stop", None)) else last.finish_reason
        if last is not None:
            account(last, text)
        return JSONResponse(final_body(text, reason, last.prompt_tokens if last else 0, last.completion_tokens if last else 0))

    @app.post("/v1/chat/completions")
    async def chat_completions(req: ChatCompletionRequest, request: Request):
        bad = _validate(req)
        if bad is not None:
            return bad
        if not req.messages:
            return _error(400, "messages must not be empty")
        try:
            # (image decoding and the vision tower run off the event loop)
            prompt = await asyncio.get_running_loop().run_in_executor(None, _chat_prompt, req.messages)
        except ValueError as e:
            return _error(400, str(e))
        return await _run(req, prompt, True, request, req.max_completion_tokens or req.max_tokens)

    @app.post("/v1/completions")
    async def completions(req: CompletionRequest, request: Request):
        bad = _validate(req)
        if bad is not None:
            return bad
        return await _run(req, req.prompt, False, request, req.max_tokens, req.prompt if req.echo else "")

    @app.post("/v1/mesh/chat/completions")
    async def mesh_chat(req: ChatCompletionRequest, request: Request):
        # tensor-parallel ranks already stand behind the ordinary route on this box
        return await chat_completions(req, request)

    # ------------------------------------------------------------------ realtime websocket
    @app.websocket("/v1/realtime")
    async def realtime(ws: WebSocket):
        from .realtime import run_realtime_session

        if state.api_keys and not key_is_valid(extract_key(ws.headers), state.api_keys):
            await ws.close(code=4401)
            return
        await ws.accept()
        try:
            await run_realtime_session(ws, state, _chat_prompt, build_sampling)
        except WebSocketDisconnect:
            pass

    return app
