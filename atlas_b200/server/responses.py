"""OpenAI Responses API (+ Conversations): create (stream / blocking / background), get, delete, cancel, input_items.

Reference parity: ``crates/spark-server/src/api/responses.rs``, ``openai/responses_lowering.rs``, ``api/stored.rs``,
``response_store.rs``, ``conversation_store.rs``.
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, Dict, List, Optional

from fastapi import Request
from fastapi.responses import JSONResponse, StreamingResponse

from .generation import BadRequest, collect


def input_to_messages(inp: Any, instructions: Optional[str]) -> List[dict]:
    msgs: List[dict] = []
    if instructions:
        msgs.append({"role": "system", "content": instructions})
    if isinstance(inp, str):
        msgs.append({"role": "user", "content": inp})
        return msgs
    pending_calls: List[dict] = []
    for it in inp or []:
        t = it.get("type", "message")
        if t == "message":
            role = it.get("role", "user")
            role = "system" if role == "developer" else role
            c = it.get("content")
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if p.get("type") in ("input_text", "output_text", "text"))
            msgs.append({"role": role, "content": c or ""})
        elif t == "function_call":
            pending_calls.append({"id": it.get("call_id"), "type": "function",
                                  "function": {"name": it.get("name"), "arguments": it.get("arguments", "{}")}})
        elif t == "function_call_output":
            if pending_calls:
                msgs.append({"role": "assistant", "content": "", "tool_calls": pending_calls})
                pending_calls = []
            out = it.get("output")
            msgs.append({"role": "tool", "tool_call_id": it.get("call_id"), "content": out if isinstance(out, str) else json.dumps(out)})
        elif t == "reasoning":
            continue
    if pending_calls:
        msgs.append({"role": "assistant", "content": "", "tool_calls": pending_calls})
    return msgs


def tools_to_chat(tools):
    out = []
    for t in tools or []:
        if t.get("type") == "function":
            out.append({"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                                         "parameters": t.get("parameters") or {"type": "object"}}})
    return out or None


def register(app, S, guard, body_of, gen_request):
    def build(body: dict):
        msgs: List[dict] = []
        prev = body.get("previous_response_id")
        if prev:
            old = S.responses.get(prev)
            if old is None:
                raise BadRequest(f"previous response '{prev}' not found", "previous_response_id")
            msgs.extend(old["_messages"])
        conv_id = body.get("conversation")
        if isinstance(conv_id, dict):
            conv_id = conv_id.get("id")
        if conv_id:
            conv = S.conversations.get(conv_id)
            if conv is None:
                raise BadRequest(f"conversation '{conv_id}' not found", "conversation")
            msgs.extend(input_to_messages(conv["items"], None))
        new = input_to_messages(body.get("input"), body.get("instructions") if not prev else None)
        msgs.extend(new)
        if not msgs:
            raise BadRequest("'input' is required", "input")
        b2 = dict(body)
        b2["messages"] = msgs
        b2["tools"] = tools_to_chat(body.get("tools"))
        fmt = (body.get("text") or {}).get("format") or {}
        if fmt.get("type") == "json_schema":
            b2["response_format"] = {"type": "json_schema", "json_schema": {"schema": fmt.get("schema")}}
        elif fmt.get("type") == "json_object":
            b2["response_format"] = {"type": "json_object"}
        tc = body.get("tool_choice", "auto")
        if isinstance(tc, dict) and tc.get("type") == "function":
            tc = {"type": "function", "function": {"name": tc.get("name")}}
        b2["tool_choice"] = tc
        return gen_request(b2), msgs, conv_id

    def envelope(rid, body, status, output, usage, created, error=None):
        u = usage or {}
        return {"id": rid, "object": "response", "created_at": created, "status": status, "model": body.get("model") or S.model_name,
                "output": output, "error": error, "incomplete_details": None, "instructions": body.get("instructions"),
                "metadata": body.get("metadata") or {}, "parallel_tool_calls": body.get("parallel_tool_calls", True),
                "previous_response_id": body.get("previous_response_id"), "temperature": body.get("temperature"),
                "top_p": body.get("top_p"), "tools": body.get("tools") or [], "tool_choice": body.get("tool_choice", "auto"),
                "usage": {"input_tokens": u.get("prompt_tokens", 0), "output_tokens": u.get("completion_tokens", 0),
                          "total_tokens": u.get("total_tokens", 0),
                          "input_tokens_details": {"cached_tokens": u.get("prompt_tokens_details", {}).get("cached_tokens", 0)},
                          "output_tokens_details": {"reasoning_tokens": 0}}}

    def output_items(o):
        items = []
        if o.reasoning:
            items.append({"id": "rs_" + uuid.uuid4().hex[:24], "type": "reasoning", "summary": [],
                          "content": [{"type": "reasoning_text", "text": o.reasoning}]})
        if o.content or not o.tool_calls:
            items.append({"id": "msg_" + uuid.uuid4().hex[:24], "type": "message", "status": "completed", "role": "assistant",
                          "content": [{"type": "output_text", "text": o.content, "annotations": []}]})
        for tc in o.tool_calls:
            items.append({"id": "fc_" + uuid.uuid4().hex[:24], "type": "function_call", "status": "completed",
                          "call_id": tc.id, "name": tc.name, "arguments": tc.arguments})
        return items

    def remember(rid, resp, msgs, o, body, conv_id):
        hist = list(msgs)
        am: Dict[str, Any] = {"role": "assistant", "content": o.content}
        if o.tool_calls:
            am["tool_calls"] = [{"id": tc.id, "type": "function", "function": {"name": tc.name, "arguments": tc.arguments}}
                                for tc in o.tool_calls]
        hist.append(am)
        if body.get("store", True):
            S.responses.put(rid, {**resp, "_messages": hist, "_input": body.get("input")})
        if conv_id:
            ins = body.get("input")
            new_items = [{"type": "message", "role": "user", "content": ins}] if isinstance(ins, str) else list(ins or [])
            S.conversations.add_items(conv_id, new_items + resp["output"])

    @app.post("/v1/responses")
    @guard
    async def create(request: Request):
        body = await body_of(request)
        req, msgs, conv_id = build(body)
        S.gen.prepare(req)
        rid = "resp_" + uuid.uuid4().hex[:32]
        created = int(time.time())
        if body.get("background"):
            S.responses.put(rid, {**envelope(rid, body, "in_progress", [], None, created), "_messages": msgs, "_input": body.get("input")})

            async def run_bg():
                o = await collect(S.gen.stream(req))
                if rid in S.cancelled:
                    return
                status = "failed" if o.error else "completed"
                resp = envelope(rid, body, status, output_items(o), o.usage, created,
                                {"message": o.error, "code": "server_error"} if o.error else None)
                remember(rid, resp, msgs, o, {**body, "store": True}, conv_id)
            asyncio.get_running_loop().create_task(run_bg())
            return JSONResponse(envelope(rid, body, "queued", [], None, created))
        if body.get("stream"):
            async def sse():
                seq = [0]

                def ev(name, data):
                    data = {"type": name, "sequence_number": seq[0], **data}
                    seq[0] += 1
                    return f"event: {name}\ndata: {json.dumps(data)}\n\n".encode()
                shell = envelope(rid, body, "in_progress", [], None, created)
                yield ev("response.created", {"response": shell})
                yield ev("response.in_progress", {"response": shell})
                msg_id = "msg_" + uuid.uuid4().hex[:24]
                opened = False
                from .generation import GenDelta
                agg = GenDelta()
                async for d in S.gen.stream(req):
                    if d.error:
                        yield ev("response.failed", {"response": envelope(rid, body, "failed", [], None, created,
                                                                             {"message": d.error, "code": "server_error"})})
                        return
                    agg.content += d.content
                    agg.reasoning += d.reasoning
                    agg.tool_calls += d.tool_calls
                    if d.reasoning:
                        yield ev("response.reasoning_text.delta", {"item_id": "rs_0", "output_index": 0, "content_index": 0, "delta": d.reasoning})
                    if d.content:
                        if not opened:
                            opened = True
                            yield ev("response.output_item.added", {"output_index": 0, "item": {
                                "id": msg_id, "type": "message", "status": "in_progress", "role": "assistant", "content": []}})
                            yield ev("response.content_part.added", {"item_id": msg_id, "output_index": 0, "content_index": 0,
                                                                     "part": {"type": "output_text", "text": "", "annotations": []}})
                        yield ev("response.output_text.delta", {"item_id": msg_id, "output_index": 0, "content_index": 0, "delta": d.content})
                    if d.finish_reason:
                        agg.finish_reason = d.finish_reason
                    if d.usage:
                        agg.usage = d.usage
                if opened:
                    yield ev("response.output_text.done", {"item_id": msg_id, "output_index": 0, "content_index": 0, "text": agg.content})
                items = output_items(agg)
                for i, it in enumerate(items):
                    if it["type"] == "function_call":
                        yield ev("response.output_item.added", {"output_index": i, "item": {**it, "arguments": ""}})
                        yield ev("response.function_call_arguments.delta", {"item_id": it["id"], "output_index": i, "delta": it["arguments"]})
                        yield ev("response.function_call_arguments.done", {"item_id": it["id"], "output_index": i, "arguments": it["arguments"]})
                    yield ev("response.output_item.done", {"output_index": i, "item": it})
                status = "incomplete" if agg.finish_reason == "length" else "completed"
                resp = envelope(rid, body, status, items, agg.usage, created)
                if status == "incomplete":
                    resp["incomplete_details"] = {"reason": "max_output_tokens"}
                remember(rid, resp, msgs, agg, body, conv_id)
                yield ev("response.completed" if status == "completed" else "response.incomplete", {"response": resp})
            return StreamingResponse(sse(), media_type="text/event-stream")
        o = await collect(S.gen.stream(req))
        if o.error:
            return JSONResponse(envelope(rid, body, "failed", [], None, created, {"message": o.error, "code": "server_error"}),
                                status_code=500)
        status = "incomplete" if o.finish_reason == "length" else "completed"
        resp = envelope(rid, body, status, output_items(o), o.usage, created)
        if status == "incomplete":
            resp["incomplete_details"] = {"reason": "max_output_tokens"}
        remember(rid, resp, msgs, o, body, conv_id)
        return JSONResponse(resp)

    def public(r):
        return {k: v for k, v in r.items() if not k.startswith("_")}

    def nf(what, i):
        return JSONResponse({"error": {"message": f"{what} '{i}' not found", "type": "not_found_error"}}, status_code=404)

    @app.get("/v1/responses/{rid}")
    async def get_response(rid: str):
        r = S.responses.get(rid)
        return JSONResponse(public(r)) if r else nf("response", rid)

    @app.delete("/v1/responses/{rid}")
    async def delete_response(rid: str):
        return {"id": rid, "object": "response", "deleted": True} if S.responses.delete(rid) else nf("response", rid)

    @app.post("/v1/responses/{rid}/cancel")
    async def cancel_response(rid: str):
        r = S.responses.get(rid)
        if r is None:
            return nf("response", rid)
        if r["status"] in ("queued", "in_progress"):
            S.cancelled.add(rid)
            r["status"] = "cancelled"
        return JSONResponse(public(r))

    @app.get("/v1/responses/{rid}/input_items")
    async def input_items(rid: str):
        r = S.responses.get(rid)
        if r is None:
            return nf("response", rid)
        inp = r.get("_input")
        items = [{"id": "msg_in_0", "type": "message", "role": "user", "content": [{"type": "input_text", "text": inp}]}] \
            if isinstance(inp, str) else list(inp or [])
        return {"object": "list", "data": items, "has_more": False}

    # ---- conversations
    @app.post("/v1/conversations")
    @guard
    async def conv_create(request: Request):
        b = await body_of(request)
        c = S.conversations.create(b.get("items"), b.get("metadata"))
        return {k: v for k, v in c.items() if k != "items"}

    @app.get("/v1/conversations/{cid}")
    async def conv_get(cid: str):
        c = S.conversations.get(cid)
        return {k: v for k, v in c.items() if k != "items"} if c else nf("conversation", cid)

    @app.post("/v1/conversations/{cid}")
    @guard
    async def conv_update(request: Request, cid: str):
        b = await body_of(request)
        c = S.conversations.update(cid, b.get("metadata") or {})
        return {k: v for k, v in c.items() if k != "items"} if c else nf("conversation", cid)

    @app.delete("/v1/conversations/{cid}")
    async def conv_delete(cid: str):
        return {"id": cid, "object": "conversation.deleted", "deleted": True} if S.conversations.delete(cid) else nf("conversation", cid)

    @app.get("/v1/conversations/{cid}/items")
    async def conv_items(cid: str):
        c = S.conversations.get(cid)
        return {"object": "list", "data": c["items"], "has_more": False} if c else nf("conversation", cid)

    @app.post("/v1/conversations/{cid}/items")
    @guard
    async def conv_add_items(request: Request, cid: str):
        b = await body_of(request)
        added = S.conversations.add_items(cid, b.get("items") or [])
        return {"object": "list", "data": added} if added is not None else nf("conversation", cid)

    @app.delete("/v1/conversations/{cid}/items/{iid}")
    async def conv_del_item(cid: str, iid: str):
        return {"id": iid, "deleted": True} if S.conversations.delete_item(cid, iid) else nf("item", iid)
