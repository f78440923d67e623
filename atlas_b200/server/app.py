"""HTTP server: OpenAI chat/completions (+stored), legacy completions, Responses, Conversations, Anthropic
messages, models, tokenize/detokenize, llama.cpp dialect, LoRA control, ops endpoints and 501 stubs.

Reference parity: routes of ``crates/spark-server/src/main_modules/serve_router.rs:45-136``; middleware stack
(panic -> 500, CORS any-origin, body limit, auth, rate limit, GPU-fault 503) of ``serve_router.rs:142-169``.
"""
from __future__ import annotations

import asyncio
import functools
import json
import os
import time
import uuid
from typing import Any, AsyncIterator, Dict, List, Optional

from ..utils.trace import TRACER
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..utils.fault import FAULT_LATCH
from .engine_async import AsyncEngine
from .evidence import ChoiceEvidence, combine
from .generation import BadRequest, GenDelta, Generator, GenRequest, collect
from .grammar import GrammarEngine
from .metrics import ServerMetrics
from .middleware import BearerAuth, RateLimiter
from .stores import ConversationStore, LruTtlStore, SessionManager
from .tokenizer import BaseTokenizer, render_chat
from .tool_parsers import default_parser_for

SAMPLING_KEYS = ("max_tokens", "max_completion_tokens", "max_output_tokens", "n_predict", "temperature", "top_p", "top_k",
                 "min_p", "top_n_sigma", "repetition_penalty", "presence_penalty", "frequency_penalty", "logit_bias",
                 "seed", "min_tokens", "stop_token_ids", "ignore_eos", "dry_multiplier", "dry_base", "dry_allowed_length")


class ServerState:
    def __init__(self, engine: AsyncEngine, tokenizer: BaseTokenizer, model_name: str, args: Optional[Dict[str, Any]] = None):
        self.engine, self.tokenizer, self.model_name = engine, tokenizer, model_name
        self.args: Dict[str, Any] = dict(args or {})
        mcfg = engine.engine.mcfg
        self.tool_parser_name = self.args.get("tool_call_parser") or default_parser_for(mcfg.model_type)
        try:
            self.grammar = GrammarEngine(tokenizer, mcfg.vocab_size)
        except Exception:
            self.grammar = None
        self.metrics = ServerMetrics(model_name)
        self.auth = BearerAuth(self.args.get("api_keys"))
        self.limiter = RateLimiter(float(self.args.get("rate_limit_rpm", 0) or 0))
        self.responses = LruTtlStore(int(self.args.get("response_store_capacity", 1024)), float(self.args.get("response_ttl_s", 3600)))
        self.chat_store = LruTtlStore(1024, 3600.0)
        self.conversations = ConversationStore()
        self.sessions = SessionManager()
        self.adapters: Dict[str, dict] = {}
        self.active_adapter: Optional[str] = None
        self.created = int(time.time())
        self.gen = Generator(self)
        self.max_body = int(os.environ.get("ATLAS_MAX_BODY_BYTES", self.args.get("max_body_bytes", 32 << 20)))
        self.cancelled: set = set()


def _err(status: int, message: str, typ: str = "invalid_request_error", param: Optional[str] = None, code: Optional[str] = None):
    return JSONResponse({"error": {"message": message, "type": typ, "param": param, "code": code}}, status_code=status)


def _sse(obj: Any) -> bytes:
    return b"data: " + json.dumps(obj, ensure_ascii=False).encode() + b"\n\n"


def _stops(v) -> List[str]:
    if v is None:
        return []
    return [v] if isinstance(v, str) else [x for x in v if isinstance(x, str)]


def _thinking(body: dict):
    """(enable_thinking, budget) from the several spellings clients use."""
    en, budget = body.get("enable_thinking"), body.get("thinking_token_budget")
    th = body.get("thinking")
    if isinstance(th, dict):
        if th.get("type") == "enabled":
            en = True
            budget = th.get("budget_tokens", budget)
        elif th.get("type") == "disabled":
            en = False
    elif isinstance(th, bool):
        en = th
    kw = body.get("chat_template_kwargs") or {}
    if "enable_thinking" in kw:
        en = bool(kw["enable_thinking"])
    r = body.get("reasoning") or {}
    eff = body.get("reasoning_effort") or (r.get("effort") if isinstance(r, dict) else None)
    if eff is not None:
        en = eff not in ("none", "minimal") if en is None else en
        budget = budget or {"low": 1024, "medium": 4096, "high": 16384}.get(eff)
    return en, budget


def create_app(state: ServerState) -> FastAPI:
    app = FastAPI(title="atlas-b200", docs_url=None, redoc_url=None)
    app.state.atlas = state
    S = state

    # ------------------------------------------------------------------ middleware stack
    @app.middleware("http")
    async def stack(request: Request, call_next):
        t0 = time.monotonic()
        path = request.url.path
        try:
            if request.method == "OPTIONS":
                resp = PlainTextResponse("", status_code=204)
            else:
                cl = request.headers.get("content-length")
                if cl and int(cl) > S.max_body:
                    resp = _err(413, f"request body exceeds {S.max_body} bytes")
                elif FAULT_LATCH.tripped and not path.startswith(("/health", "/metrics")):
                    resp = _err(503, f"GPU context lost: {FAULT_LATCH.reason}", "server_error", code="gpu_fault")
                else:
                    ident = "anonymous"
                    open_path = path in ("/health", "/health/live", "/metrics", "/")
                    if S.auth.enabled and not open_path:
                        got = S.auth.identity(request.headers.get("authorization"), request.headers.get("x-api-key"))
                        if got is None:
                            resp = _err(401, "missing or invalid API key", "authentication_error", code="invalid_api_key")
                            raise _Short(resp)
                        ident = got
                    if not open_path and not S.limiter.allow(ident):
                        raise _Short(_err(429, "rate limit exceeded", "rate_limit_error", code="rate_limit_exceeded"))
                    request.state.identity = ident
                    resp = await call_next(request)
        except _Short as s:
            resp = s.resp
        except Exception as e:        # the "panic -> 500" layer
            resp = _err(500, f"internal error: {e.__class__.__name__}: {e}", "server_error")
        resp.headers["access-control-allow-origin"] = "*"
        resp.headers["access-control-allow-headers"] = "*"
        resp.headers["access-control-allow-methods"] = "*"
        S.metrics.on_http(path, resp.status_code, time.monotonic() - t0, int(request.headers.get("content-length") or 0))
        return resp

    async def body_of(request: Request) -> dict:
        raw = await request.body()
        if len(raw) > S.max_body:
            raise BadRequest(f"request body exceeds {S.max_body} bytes")
        try:
            b = json.loads(raw or b"{}")
        except Exception as e:
            raise BadRequest(f"invalid JSON body: {e}")
        if not isinstance(b, dict):
            raise BadRequest("the request body must be a JSON object")
        return b

    def guard(fn):
        @functools.wraps(fn)
        async def wrapped(request: Request, **kw):
            try:
                if not S.engine.accepting and request.method == "POST":
                    return _err(503, "the engine is draining or stopped", "server_error")
                return await fn(request, **kw)
            except BadRequest as e:
                return _err(400, str(e), "invalid_request_error", e.param, e.code if e.code != "invalid_request_error" else None)
        return wrapped

    def gen_request(body: dict, **over) -> GenRequest:
        en, budget = _thinking(body)
        so = body.get("stream_options") or {}
        tc = body.get("tool_choice", "auto")
        to = body.get("timeout")
        r = GenRequest(messages=body.get("messages"), tools=body.get("tools"), tool_choice=tc,
                       parallel_tool_calls=bool(body.get("parallel_tool_calls", True)),
                       sampling={k: body[k] for k in SAMPLING_KEYS if k in body},
                       response_format=body.get("response_format"), stop=_stops(body.get("stop")),
                       enable_thinking=en, thinking_budget=budget,
                       chat_template_kwargs={k: v for k, v in (body.get("chat_template_kwargs") or {}).items() if k != "enable_thinking"},
                       logprobs=bool(body.get("logprobs")) and not isinstance(body.get("logprobs"), int) or body.get("logprobs") is True,
                       top_logprobs=int(body.get("top_logprobs") or 0), timeout_s=float(to) if to else S.args.get("request_timeout"),
                       cache_key=body.get("prompt_cache_key") or body.get("user"), adapter=body.get("adapter"),
                       disable_spec=(body.get("atlas_speculative") is False), confidence=bool(body.get("atlas_confidence")))
        for k, v in over.items():
            setattr(r, k, v)
        return r

    def lp_openai(entries: Optional[list]) -> Optional[dict]:
        if not entries:
            return None
        content = []
        for e in entries:
            if e is None:
                continue
            piece = S.tokenizer.token_to_piece(e["token"])
            content.append({"token": piece, "logprob": e["logprob"], "bytes": list(piece.encode()),
                            "top_logprobs": [{"token": S.tokenizer.token_to_piece(t), "logprob": lp,
                                              "bytes": list(S.tokenizer.token_to_piece(t).encode())} for t, lp in e.get("top", [])]})
        return {"content": content}

    # ------------------------------------------------------------------ OpenAI chat completions
    @app.post("/v1/chat/completions")
    @guard
    async def chat_completions(request: Request):
        body = await body_of(request)
        if "messages" not in body:
            raise BadRequest("'messages' is required", "messages")
        n = int(body.get("n") or 1)
        if n < 1 or n > 8:
            raise BadRequest("'n' must be between 1 and 8", "n")
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        model = body.get("model") or S.model_name
        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
        want_ids = bool(body.get("return_token_ids"))
        reqs = [gen_request(body) for _ in range(n)]
        if n > 1 and body.get("seed") is not None:
            for i, r in enumerate(reqs):
                r.sampling["seed"] = int(body["seed"]) + i
        for r in reqs:
            S.gen.prepare(r)       # validate before any bytes are sent
        want_evidence = bool(body.get("atlas_evidence"))
        stop_ids = S.engine.engine.mcfg.eos_ids() if want_evidence else ()
        if body.get("stream"):
            async def sse() -> AsyncIterator[bytes]:
                base = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model}
                usage_tot: Dict[str, Any] = {}
                ev_tok, ev_out = [], []
                for idx, r in enumerate(reqs):
                    yield _sse({**base, "choices": [{"index": idx, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]})
                    ev, fin = ChoiceEvidence(stop_ids), ""
                    async for d in S.gen.stream(r):
                        ev.add(d.token_ids, d.content, d.reasoning)
                        fin = d.finish_reason or fin
                        if d.error:
                            yield _sse({"error": {"message": d.error, "type": "server_error"}})
                            break
                        delta: Dict[str, Any] = {}
                        if d.content:
                            delta["content"] = d.content
                        if d.reasoning:
                            delta["reasoning_content"] = d.reasoning
                        if d.tool_calls:
                            delta["tool_calls"] = [tc.to_openai(i) for i, tc in enumerate(d.tool_calls)]
                        if delta or d.finish_reason:
                            ch: Dict[str, Any] = {"index": idx, "delta": delta, "finish_reason": d.finish_reason}
                            if d.logprobs and r.logprobs:
                                ch["logprobs"] = lp_openai(d.logprobs)
                            if want_ids and d.token_ids:
                                ch["token_ids"] = d.token_ids
                            yield _sse({**base, "choices": [ch]})
                        if d.usage:
                            for k, v in d.usage.items():
                                if isinstance(v, (int, float)):
                                    usage_tot[k] = usage_tot.get(k, 0) + v if k != "prompt_tokens" else v
                                else:
                                    usage_tot[k] = v
                    ev_tok.append(ev.token_digest(fin))
                    ev_out.append(ev.output_digest())
                if want_evidence:
                    usage_tot["atlas_token_sha"], usage_tot["atlas_output_sha256"] = combine(ev_tok), combine(ev_out)
                if include_usage or want_evidence:
                    usage_tot["total_tokens"] = usage_tot.get("prompt_tokens", 0) + usage_tot.get("completion_tokens", 0)
                    yield _sse({**base, "choices": [], "usage": usage_tot})
                yield b"data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        outs = await asyncio.gather(*[collect(S.gen.stream(r)) for r in reqs])
        choices = []
        usage = {"prompt_tokens": 0, "completion_tokens": 0}
        ev_tok, ev_out = [], []
        for idx, (r, o) in enumerate(zip(reqs, outs)):
            if o.error:
                return _err(500, o.error, "server_error")
            if want_evidence:
                ev = ChoiceEvidence(stop_ids)
                ev.add(o.token_ids, o.content, o.reasoning)
                ev_tok.append(ev.token_digest(o.finish_reason or ""))
                ev_out.append(ev.output_digest())
            msg: Dict[str, Any] = {"role": "assistant", "content": o.content if (o.content or not o.tool_calls) else None}
            if o.reasoning:
                msg["reasoning_content"] = o.reasoning
            if o.tool_calls:
                msg["tool_calls"] = [{k: v for k, v in tc.to_openai(i).items() if k != "index"} for i, tc in enumerate(o.tool_calls)]
            ch = {"index": idx, "message": msg, "finish_reason": o.finish_reason,
                  "logprobs": lp_openai(o.logprobs) if r.logprobs else None}
            if want_ids:
                ch["token_ids"] = o.token_ids
            if r.confidence:
                from .confidence import confidence_summary
                ch["atlas_confidence"] = confidence_summary(o.logprobs)
                usage.setdefault("atlas_confidence", ch["atlas_confidence"])        # the first choice's, as in `usage`
                S.metrics.on_confidence(ch["atlas_confidence"])
            choices.append(ch)
            u = o.usage or {}
            usage["prompt_tokens"] = u.get("prompt_tokens", 0)
            usage["completion_tokens"] += u.get("completion_tokens", 0)
            for k in ("prompt_tokens_details", "completion_tokens_details", "time_to_first_token_ms", "decode_time_ms"):
                if k in u:
                    usage[k] = u[k]
        usage["total_tokens"] = usage["prompt_tokens"] + usage["completion_tokens"]
        if want_evidence:
            usage["atlas_token_sha"], usage["atlas_output_sha256"] = combine(ev_tok), combine(ev_out)
        resp = {"id": cid, "object": "chat.completion", "created": created, "model": model, "choices": choices,
                "usage": usage, "system_fingerprint": "atlas-b200"}
        if body.get("store"):
            S.chat_store.put(cid, {**resp, "metadata": body.get("metadata") or {}, "request": {"messages": body["messages"]}})
        return JSONResponse(resp)

    @app.get("/v1/chat/completions/{cid}")
    async def chat_get(cid: str):
        r = S.chat_store.get(cid)
        return JSONResponse(r) if r else _err(404, f"no stored completion '{cid}'", "not_found_error")

    # ------------------------------------------------------------------ legacy completions
    @app.post("/v1/completions")
    @guard
    async def completions(request: Request):
        body = await body_of(request)
        prompt = body.get("prompt")
        if prompt is None:
            raise BadRequest("'prompt' is required", "prompt")
        toks = None
        if isinstance(prompt, list):
            if prompt and all(isinstance(x, int) for x in prompt):
                toks, prompt = prompt, None
            elif len(prompt) == 1 and isinstance(prompt[0], str):
                prompt = prompt[0]
            else:
                raise BadRequest("batched prompts are not supported; send one prompt per request", "prompt")
        req = gen_request(body, messages=None, prompt=prompt, prompt_tokens=toks, echo=bool(body.get("echo")))
        if isinstance(body.get("logprobs"), int) and not isinstance(body.get("logprobs"), bool):
            req.logprobs, req.top_logprobs = True, int(body["logprobs"])
        S.gen.prepare(req)
        cid = "cmpl-" + uuid.uuid4().hex[:24]
        want_ids = bool(body.get("return_token_ids"))
        created, model = int(time.time()), body.get("model") or S.model_name

        def lp_legacy(entries):
            if not entries:
                return None
            ents = [e for e in entries if e]
            return {"tokens": [S.tokenizer.token_to_piece(e["token"]) for e in ents],
                    "token_logprobs": [e["logprob"] for e in ents],
                    "top_logprobs": [{S.tokenizer.token_to_piece(t): lp for t, lp in e.get("top", [])} for e in ents],
                    "text_offset": []}
        if body.get("stream"):
            async def sse():
                async for d in S.gen.stream(req):
                    if d.error:
                        yield _sse({"error": {"message": d.error, "type": "server_error"}})
                        break
                    if d.content or d.reasoning or d.finish_reason or (want_ids and d.token_ids):
                        yield _sse({"id": cid, "object": "text_completion", "created": created, "model": model,
                                    "choices": [{"index": 0, "text": d.reasoning + d.content, "finish_reason": d.finish_reason,
                                                 "logprobs": lp_legacy(d.logprobs) if req.logprobs else None,
                                                 **({"token_ids": d.token_ids} if want_ids and d.token_ids else {})}],
                                    **({"usage": d.usage} if d.usage else {})})
                yield b"data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        o = await collect(S.gen.stream(req))
        if o.error:
            return _err(500, o.error, "server_error")
        return JSONResponse({"id": cid, "object": "text_completion", "created": created, "model": model,
                             "choices": [{"index": 0, "text": o.reasoning + o.content, "finish_reason": o.finish_reason,
                                          "logprobs": lp_legacy(o.logprobs) if req.logprobs else None,
                                          **({"token_ids": o.token_ids} if want_ids else {})}],
                             "usage": o.usage})

    # ------------------------------------------------------------------ models / tokenize
    def model_card():
        return {"id": S.model_name, "object": "model", "created": S.created, "owned_by": "atlas-b200",
                "max_model_len": S.engine.engine.cfg.max_seq_len, "vocab_size": S.engine.engine.mcfg.vocab_size}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [model_card()]}

    @app.get("/v1/models/{mid:path}")
    async def model_get(mid: str):
        return model_card() if mid == S.model_name else _err(404, f"model '{mid}' not found", "not_found_error")

    @app.post("/tokenize")
    @guard
    async def tokenize(request: Request):
        b = await body_of(request)
        if "messages" in b:
            text = render_chat(S.tokenizer, b["messages"], b.get("tools"), add_generation_prompt=b.get("add_generation_prompt", True))
        else:
            text = b.get("prompt", b.get("content", b.get("text", "")))
        ids = S.tokenizer.encode(text, add_special_tokens=bool(b.get("add_special_tokens", False)))
        return {"tokens": ids, "count": len(ids), "max_model_len": S.engine.engine.cfg.max_seq_len}

    @app.post("/detokenize")
    @guard
    async def detokenize(request: Request):
        b = await body_of(request)
        ids = b.get("tokens")
        if not isinstance(ids, list):
            raise BadRequest("'tokens' must be an array of ids", "tokens")
        text = S.tokenizer.decode([int(i) for i in ids], skip_special_tokens=False)
        return {"prompt": text, "content": text}

    # ------------------------------------------------------------------ llama.cpp dialect
    @app.post("/completion")
    @app.post("/completions")
    @guard
    async def llama_completion(request: Request):
        b = await body_of(request)
        req = gen_request(b, messages=None, prompt=b.get("prompt", ""))
        S.gen.prepare(req)
        if b.get("stream"):
            async def sse():
                async for d in S.gen.stream(req):
                    yield _sse({"content": d.reasoning + d.content, "stop": d.finish_reason is not None,
                                **({"tokens_predicted": d.usage["completion_tokens"], "tokens_evaluated": d.usage["prompt_tokens"],
                                    "stop_type": "limit" if d.finish_reason == "length" else "eos"} if d.usage else {})})
            return StreamingResponse(sse(), media_type="text/event-stream")
        o = await collect(S.gen.stream(req))
        u = o.usage or {}
        return {"content": o.reasoning + o.content, "stop": True, "model": S.model_name,
                "tokens_predicted": u.get("completion_tokens", 0), "tokens_evaluated": u.get("prompt_tokens", 0),
                "stop_type": "limit" if o.finish_reason == "length" else "eos", "truncated": False,
                "timings": {"prompt_ms": u.get("time_to_first_token_ms"), "predicted_ms": u.get("decode_time_ms")}}

    @app.get("/props")
    async def props():
        return {"default_generation_settings": {"n_ctx": S.engine.engine.cfg.max_seq_len, "model": S.model_name},
                "total_slots": S.engine.engine.cfg.max_num_seqs, "model_path": S.model_name,
                "chat_template": S.tokenizer.chat_template or "", "build_info": "atlas-b200"}

    @app.post("/apply-template")
    @guard
    async def apply_template(request: Request):
        b = await body_of(request)
        return {"prompt": render_chat(S.tokenizer, b.get("messages") or [], b.get("tools"))}

    @app.post("/embedding")
    @app.post("/embeddings")
    async def llama_embedding():
        return _err(501, "embeddings are not supported by this server", "not_implemented")

    # ------------------------------------------------------------------ LoRA control
    @app.get("/v1/lora/active")
    async def lora_active():
        return {"active": S.active_adapter, "loaded": sorted(S.adapters)}

    @app.post("/v1/lora/load")
    @guard
    async def lora_load(request: Request):
        b = await body_of(request)
        name, path = b.get("name"), b.get("path")
        if not name:
            raise BadRequest("'name' is required", "name")
        try:
            path = path or S.adapters[name]["path"]
            slot = S.engine.engine.load_adapter(name, path)      # resident on every rank from now on, addressed by slot
            S.adapters[name] = {"path": path, "slot": slot}
        except KeyError:
            return _err(404, f"adapter '{name}' is not loaded and no path was given", "not_found_error")
        except Exception as e:
            raise BadRequest(f"could not load adapter: {e}", "path")
        if b.get("activate", True):
            S.active_adapter = name
        return {"active": S.active_adapter, "loaded": sorted(S.adapters)}

    # ------------------------------------------------------------------ ops
    @app.get("/health")
    async def health():
        if FAULT_LATCH.tripped:
            return JSONResponse({"status": "fault", "reason": FAULT_LATCH.reason}, status_code=503)
        return {"status": "ok" if S.engine.accepting else "draining", "model": S.model_name,
                "uptime_s": round(time.time() - S.engine.started_at, 1)}

    @app.get("/health/live")
    async def live():
        return {"status": "alive"}

    @app.get("/metrics")
    async def metrics():
        S.metrics.observe_engine(S.engine.engine)
        return PlainTextResponse(S.metrics.render(), media_type="text/plain; version=0.0.4")

    @app.get("/hardware")
    async def hardware():
        from ..utils.hardware import fingerprint
        return fingerprint()

    @app.get("/serve-config")
    async def serve_config():
        e = S.engine.engine
        import dataclasses
        return {"model": S.model_name, "engine": dataclasses.asdict(e.cfg), "scheduler": e.snapshot(),
                "tool_call_parser": S.tool_parser_name, "grammar_backend": S.grammar.backend if S.grammar else None,
                "kv_cache_dtype": str(e.kv_dtype), "num_kv_blocks": e.pool.num_blocks,
                "serve_plan": S.args.get("serve_plan"), "trace": TRACER.summary()}

    @app.get("/trace")
    async def trace_dump():
        return TRACER.chrome_trace()

    for stub in ("/v1/embeddings", "/v1/batches", "/v1/files", "/v1/audio/speech", "/v1/audio/transcriptions",
                 "/v1/audio/translations", "/v1/images/generations", "/v1/images/edits", "/v1/moderations",
                 "/v1/fine_tuning/jobs"):
        def make(path):
            async def not_impl():
                return _err(501, f"{path} is not implemented by this server", "not_implemented", code="not_implemented")
            return not_impl
        app.add_api_route(stub, make(stub), methods=["GET", "POST"])

    from .anthropic import register as reg_anthropic
    from .responses import register as reg_responses
    reg_anthropic(app, S, guard, body_of, gen_request)
    reg_responses(app, S, guard, body_of, gen_request)
    return app


class _Short(Exception):
    def __init__(self, resp):
        self.resp = resp
