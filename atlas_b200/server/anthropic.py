"""Anthropic Messages dialect: ``POST /v1/messages`` (+SSE) and ``POST /v1/messages/count_tokens``.

Reference parity: ``crates/spark-server/src/anthropic/{handlers,to_ir,translator}.rs`` (events message_start,
content_block_start / delta / stop, message_delta, message_stop).
"""
from __future__ import annotations

import json
import uuid
from typing import Any, Dict, List

from fastapi import Request
from fastapi.responses import JSONResponse, StreamingResponse

from .generation import BadRequest, collect
from .tokenizer import render_chat


def to_openai_messages(body: dict) -> List[dict]:
    msgs: List[dict] = []
    system = body.get("system")
    if isinstance(system, list):
        system = "".join(p.get("text", "") for p in system if isinstance(p, dict))
    if system:
        msgs.append({"role": "system", "content": system})
    for m in body.get("messages") or []:
        role, content = m.get("role"), m.get("content")
        if isinstance(content, str):
            msgs.append({"role": role, "content": content})
            continue
        text, tool_calls, tool_results = [], [], []
        for p in content or []:
            t = p.get("type")
            if t == "text":
                text.append(p.get("text", ""))
            elif t == "thinking":
                continue
            elif t == "tool_use":
                tool_calls.append({"id": p.get("id"), "type": "function",
                                   "function": {"name": p.get("name"), "arguments": json.dumps(p.get("input") or {})}})
            elif t == "tool_result":
                c = p.get("content")
                if isinstance(c, list):
                    c = "".join(x.get("text", "") for x in c if isinstance(x, dict))
                tool_results.append({"role": "tool", "tool_call_id": p.get("tool_use_id"), "content": c if isinstance(c, str) else json.dumps(c)})
            elif t == "image":
                text.append("<|vision_start|><|image_pad|><|vision_end|>")
        if tool_results:
            msgs.extend(tool_results)
            if text:
                msgs.append({"role": role, "content": "".join(text)})
        else:
            msg: Dict[str, Any] = {"role": role, "content": "".join(text)}
            if tool_calls:
                msg["tool_calls"] = tool_calls
            msgs.append(msg)
    return msgs


def to_openai_tools(tools):
    out = []
    for t in tools or []:
        out.append({"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                                     "parameters": t.get("input_schema") or {"type": "object"}}})
    return out or None


_STOP = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use", "timeout": "end_turn", "abort": "end_turn"}


def register(app, S, guard, body_of, gen_request):
    def lower(body: dict):
        if "max_tokens" not in body:
            raise BadRequest("'max_tokens' is required", "max_tokens")
        tc = body.get("tool_choice") or {}
        choice: Any = "auto"
        if tc.get("type") == "any":
            choice = "required"
        elif tc.get("type") == "tool":
            choice = {"type": "function", "function": {"name": tc.get("name")}}
        elif tc.get("type") == "none":
            choice = "none"
        b2 = dict(body)
        b2["messages"] = to_openai_messages(body)
        b2["tools"] = to_openai_tools(body.get("tools"))
        b2["tool_choice"] = choice
        b2["stop"] = body.get("stop_sequences")
        return gen_request(b2)

    @app.post("/v1/messages")
    @guard
    async def messages(request: Request):
        body = await body_of(request)
        if not body.get("messages"):
            raise BadRequest("'messages' is required", "messages")
        req = lower(body)
        S.gen.prepare(req)
        mid = "msg_" + uuid.uuid4().hex[:24]
        model = body.get("model") or S.model_name
        if body.get("stream"):
            async def sse():
                def ev(name, data):
                    return f"event: {name}\ndata: {json.dumps(data)}\n\n".encode()
                yield ev("message_start", {"type": "message_start", "message": {
                    "id": mid, "type": "message", "role": "assistant", "model": model, "content": [],
                    "stop_reason": None, "stop_sequence": None, "usage": {"input_tokens": 0, "output_tokens": 0}}})
                idx, open_kind = -1, None
                usage, reason = {}, "end_turn"

                async def close_block():
                    nonlocal open_kind
                    if open_kind is not None:
                        open_kind = None
                        return ev("content_block_stop", {"type": "content_block_stop", "index": idx})
                    return b""
                async for d in S.gen.stream(req):
                    if d.error:
                        yield ev("error", {"type": "error", "error": {"type": "api_error", "message": d.error}})
                        return
                    for kind, text in (("thinking", d.reasoning), ("text", d.content)):
                        if not text:
                            continue
                        if open_kind != kind:
                            yield await close_block()
                            idx += 1
                            open_kind = kind
                            blk = {"type": "thinking", "thinking": ""} if kind == "thinking" else {"type": "text", "text": ""}
                            yield ev("content_block_start", {"type": "content_block_start", "index": idx, "content_block": blk})
                        delta = {"type": "thinking_delta", "thinking": text} if kind == "thinking" else {"type": "text_delta", "text": text}
                        yield ev("content_block_delta", {"type": "content_block_delta", "index": idx, "delta": delta})
                    for tc in d.tool_calls:
                        yield await close_block()
                        idx += 1
                        yield ev("content_block_start", {"type": "content_block_start", "index": idx, "content_block": {
                            "type": "tool_use", "id": tc.id.replace("call_", "toolu_"), "name": tc.name, "input": {}}})
                        yield ev("content_block_delta", {"type": "content_block_delta", "index": idx,
                                                         "delta": {"type": "input_json_delta", "partial_json": tc.arguments}})
                        yield ev("content_block_stop", {"type": "content_block_stop", "index": idx})
                    if d.finish_reason:
                        reason = _STOP.get(d.finish_reason, "end_turn")
                    if d.usage:
                        usage = d.usage
                yield await close_block()
                yield ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": reason, "stop_sequence": None},
                                           "usage": {"input_tokens": usage.get("prompt_tokens", 0),
                                                     "output_tokens": usage.get("completion_tokens", 0),
                                                     "cache_read_input_tokens": usage.get("prompt_tokens_details", {}).get("cached_tokens", 0)}})
                yield ev("message_stop", {"type": "message_stop"})
            return StreamingResponse(sse(), media_type="text/event-stream")
        o = await collect(S.gen.stream(req))
        if o.error:
            return JSONResponse({"type": "error", "error": {"type": "api_error", "message": o.error}}, status_code=500)
        content = []
        if o.reasoning:
            content.append({"type": "thinking", "thinking": o.reasoning, "signature": ""})
        if o.content:
            content.append({"type": "text", "text": o.content})
        for tc in o.tool_calls:
            try:
                inp = json.loads(tc.arguments)
            except Exception:
                inp = {"_raw": tc.arguments}
            content.append({"type": "tool_use", "id": tc.id.replace("call_", "toolu_"), "name": tc.name, "input": inp})
        u = o.usage or {}
        return JSONResponse({"id": mid, "type": "message", "role": "assistant", "model": model, "content": content,
                             "stop_reason": _STOP.get(o.finish_reason or "stop", "end_turn"), "stop_sequence": None,
                             "usage": {"input_tokens": u.get("prompt_tokens", 0), "output_tokens": u.get("completion_tokens", 0),
                                       "cache_read_input_tokens": u.get("prompt_tokens_details", {}).get("cached_tokens", 0),
                                       "cache_creation_input_tokens": 0}})

    @app.post("/v1/messages/count_tokens")
    @guard
    async def count_tokens(request: Request):
        body = await body_of(request)
        text = render_chat(S.tokenizer, to_openai_messages(body), to_openai_tools(body.get("tools")))
        return {"input_tokens": len(S.tokenizer.encode(text))}
