"""``/v1/realtime`` WebSocket session.

Event vocabulary of the reference (``oxidize-server/src/realtime/protocol.rs:71-117``): the
client sends ``session.update``, ``conversation.item.create``, ``response.create`` and
``response.cancel``; the server answers ``session.created`` / ``session.updated``,
``conversation.item.created``, ``response.created``, ``response.output_item.added``,
``response.text.delta`` / ``response.text.done``, ``response.done`` and ``error``.
"""
from __future__ import annotations

import asyncio
import json
import uuid
from typing import Any, Dict, List, Optional


def _id(prefix: str) -> str:
    return f"{prefix}_{uuid.uuid4().hex[:20]}"


async def run_realtime_session(ws, state, chat_prompt, build_sampling) -> None:
    from .app import PLACEHOLDER_TEXT, ChatCompletionRequest, ChatMessage

    session: Dict[str, Any] = {"id": _id("sess"), "model": state.model_id, "instructions": "", "temperature": None,
                               "max_response_output_tokens": None, "modalities": ["text"]}
    items: List[Dict[str, str]] = []
    current: Optional[asyncio.Task] = None

    async def send(ev: Dict[str, Any]) -> None:
        ev.setdefault("event_id", _id("event"))
        await ws.send_text(json.dumps(ev))

    await send({"type": "session.created", "session": session})

    async def respond() -> None:
        rid, item_id = _id("resp"), _id("item")
        await send({"type": "response.created", "response": {"id": rid, "status": "in_progress"}})
        await send({"type": "response.output_item.added", "response_id": rid,
                    "item": {"id": item_id, "type": "message", "role": "assistant"}})
        msgs = []
        if session["instructions"]:
            msgs.append(ChatMessage(role="system", content=session["instructions"]))
        msgs += [ChatMessage(role=i["role"], content=i["content"]) for i in items]
        text = ""
        status = "completed"
        try:
            if state.engine is None:
                text = PLACEHOLDER_TEXT
                await send({"type": "response.text.delta", "response_id": rid, "item_id": item_id, "delta": text})
            else:
                req = ChatCompletionRequest(model=session["model"], messages=msgs, temperature=session["temperature"],
                                            max_tokens=session["max_response_output_tokens"])
                params = build_sampling(req, state, req.max_tokens)
                async for ev in state.engine.stream(chat_prompt(msgs), params):
                    if ev.error:
                        await send({"type": "error", "error": {"type": "server_error", "message": ev.error}})
                        status = "failed"
                        break
                    if ev.text_delta:
                        text += ev.text_delta
                        await send({"type": "response.text.delta", "response_id": rid, "item_id": item_id,
                                    "delta": ev.text_delta})
        except asyncio.CancelledError:
            status = "cancelled"
        await send({"type": "response.text.done", "response_id": rid, "item_id": item_id, "text": text})
        if status == "completed":
            items.append({"role": "assistant", "content": text})
        await send({"type": "response.done", "response": {"id": rid, "status": status,
                                                          "output": [{"id": item_id, "type": "message",
                                                                      "role": "assistant", "content": text}]}})

    while True:
        raw = await ws.receive_text()
        try:
            ev = json.loads(raw)
            kind = ev.get("type")
        except (ValueError, AttributeError):
            await send({"type": "error", "error": {"type": "invalid_request_error", "message": "malformed JSON event"}})
            continue
        if kind == "session.update":
            upd = ev.get("session") or {}
            for k in ("instructions", "temperature", "max_response_output_tokens", "modalities", "model"):
                if k in upd:
                    session[k] = upd[k]
            await send({"type": "session.updated", "session": session})
        elif kind == "conversation.item.create":
            item = ev.get("item") or {}
            content = item.get("content")
            if isinstance(content, list):
                content = "".join(c.get("text", "") for c in content if isinstance(c, dict))
            rec = {"role": item.get("role", "user"), "content": content or ""}
            items.append(rec)
            await send({"type": "conversation.item.created", "item": {"id": item.get("id") or _id("item"), **rec}})
        elif kind == "response.create":
            if current is not None and not current.done():
                await send({"type": "error", "error": {"type": "invalid_request_error",
                                                       "message": "a response is already in progress"}})
                continue
            current = asyncio.create_task(respond())
        elif kind == "response.cancel":
            if current is not None and not current.done():
                current.cancel()
        else:
            await send({"type": "error", "error": {"type": "invalid_request_error",
                                                   "message": f"unknown event type {kind!r}"}})
