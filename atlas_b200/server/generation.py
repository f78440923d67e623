"""Protocol-independent generation pipeline used by every HTTP dialect.

``prepare`` lowers a dialect-neutral :class:`GenRequest` (messages or a raw prompt, tools, sampling fields,
response format, thinking switches) into prompt tokens + :class:`SamplingParams` + grammar / logits processors;
``stream`` drives the engine and yields :class:`GenDelta` items after detokenisation, stop-string handling,
reasoning splitting and tool-call parsing.

Reference parity: the protocol IR of ``crates/spark-server/src/ir/*``, ``api/chat/{msg_entry,sampling_setup,
thinking,levers}.rs``, ``api/chat_stream/handle_token.rs`` and ``api/inference_impl.rs``.
"""
from __future__ import annotations

import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Dict, List, Optional

from ..sampling import SamplingParams
from .grammar import GrammarSpec
from .reasoning import ReasoningSplitter, ThinkingBudget
from .logit_processors import ThinkToolPipeline, repeated_tool_call
from .loop_detector import LoopDetector
from .compaction import compact_messages
from .sanitizer import ContentSanitizer, StreamGuards, guarded_stops
from .tokenizer import IncrementalDetokenizer, render_chat
from .tool_parsers import StreamingToolParser, ToolCall, get_parser, dedupe_calls


@dataclass
class GenRequest:
    messages: Optional[List[dict]] = None
    prompt: Optional[str] = None
    prompt_tokens: Optional[List[int]] = None
    tools: Optional[List[dict]] = None
    tool_choice: Any = "auto"
    parallel_tool_calls: bool = True
    sampling: Dict[str, Any] = field(default_factory=dict)       # raw request fields
    response_format: Optional[dict] = None
    stop: List[str] = field(default_factory=list)
    enable_thinking: Optional[bool] = None
    thinking_budget: Optional[int] = None
    chat_template_kwargs: Dict[str, Any] = field(default_factory=dict)
    echo: bool = False
    logprobs: bool = False
    top_logprobs: int = 0
    confidence: bool = False             # attach the confidence summary of the first tokens (server/confidence.py)
    timeout_s: Optional[float] = None
    cache_key: Optional[str] = None
    adapter: Optional[str] = None
    disable_spec: bool = False
    request_id: str = field(default_factory=lambda: uuid.uuid4().hex[:24])


@dataclass
class GenDelta:
    content: str = ""
    reasoning: str = ""
    tool_calls: List[ToolCall] = field(default_factory=list)
    token_ids: List[int] = field(default_factory=list)
    logprobs: Optional[list] = None
    finish_reason: Optional[str] = None
    usage: Optional[dict] = None
    error: Optional[str] = None


class BadRequest(ValueError):
    def __init__(self, message: str, param: Optional[str] = None, code: str = "invalid_request_error"):
        super().__init__(message)
        self.param, self.code = param, code


def sampling_from_fields(f: Dict[str, Any], defaults: Optional[Dict[str, Any]] = None, max_default: int = 1024) -> SamplingParams:
    d = dict(defaults or {})
    d.update({k: v for k, v in f.items() if v is not None})

    def num(name, default, cast=float):
        v = d.get(name, default)
        try:
            return cast(v)
        except (TypeError, ValueError):
            raise BadRequest(f"'{name}' must be a number", name)
    max_tokens = d.get("max_completion_tokens", d.get("max_tokens", d.get("max_output_tokens", d.get("n_predict", max_default))))
    if max_tokens is None or int(max_tokens) < 0:
        max_tokens = max_default
    lb = {}
    for k, v in (d.get("logit_bias") or {}).items():
        try:
            lb[int(k)] = float(v)
        except (TypeError, ValueError):
            raise BadRequest("logit_bias keys must be token ids", "logit_bias")
    sp = SamplingParams(
        temperature=num("temperature", 1.0), top_k=num("top_k", 0, int), top_p=num("top_p", 1.0), min_p=num("min_p", 0.0),
        top_n_sigma=num("top_n_sigma", 0.0), repetition_penalty=num("repetition_penalty", 1.0),
        presence_penalty=num("presence_penalty", 0.0), frequency_penalty=num("frequency_penalty", 0.0),
        dry_multiplier=num("dry_multiplier", 0.0), dry_base=num("dry_base", 1.75), dry_allowed_length=num("dry_allowed_length", 2, int),
        logit_bias=lb, max_tokens=max(1, int(max_tokens)), min_tokens=num("min_tokens", 0, int),
        stop_token_ids=[int(x) for x in (d.get("stop_token_ids") or [])], ignore_eos=bool(d.get("ignore_eos", False)),
        seed=d.get("seed"), logprobs=bool(d.get("logprobs")), top_logprobs=num("top_logprobs", 0, int) if d.get("top_logprobs") else 0,
    )
    if isinstance(d.get("logprobs"), int) and not isinstance(d.get("logprobs"), bool):     # legacy completions: logprobs=N
        sp.logprobs, sp.top_logprobs = True, int(d["logprobs"])
    try:
        sp.validate()
    except ValueError as e:
        raise BadRequest(str(e))
    return sp


class Generator:
    def __init__(self, state):
        self.s = state

    # ------------------------------------------------------------------ lowering
    def prepare(self, req: GenRequest):
        s = self.s
        tk = s.tokenizer
        thinking = req.enable_thinking
        if thinking is None:
            thinking = s.args.get("default_thinking", False)
        if s.args.get("disable_thinking"):
            thinking = False
        tools = req.tools if (req.tools and req.tool_choice != "none") else None
        if req.prompt_tokens is not None:
            toks = list(req.prompt_tokens)
            text = None
        elif req.messages is not None:
            if not isinstance(req.messages, list) or not req.messages:
                raise BadRequest("'messages' must be a non-empty array", "messages")
            def render(msgs):
                return render_chat(tk, msgs, tools, add_generation_prompt=True, enable_thinking=thinking,
                                   **req.chat_template_kwargs)
            try:
                text = render(req.messages)
            except Exception as e:
                raise BadRequest(f"chat template failed: {e}", "messages")
            toks = tk.encode(text)
            if s.args.get("context_compaction"):
                reserve = int(s.args.get("compaction_reserve_tokens") or 256)
                budget = s.engine.engine.cfg.max_seq_len - reserve
                if len(toks) > budget:
                    msgs, self.last_compaction = compact_messages(req.messages, lambda m: len(tk.encode(render(m))), budget)
                    text = render(msgs)
                    toks = tk.encode(text)
        else:
            text = req.prompt or ""
            toks = tk.encode(text, add_special_tokens=bool(tk.bos_token_id is not None and s.args.get("add_bos", False)))
        if not toks:
            toks = [tk.bos_token_id if tk.bos_token_id is not None else 0]
        req._images = []
        model = s.engine.engine.model
        if req.messages is not None and getattr(model, "vision", None) is not None:
            from .multimodal import ImageError, prepare_images
            try:
                toks, req._images = prepare_images(req.messages, toks, model.cfg.vision, model.cfg.image_token_id)
            except ImageError as e:
                raise BadRequest(str(e), "messages")
        presets = s.args.get("sampling_presets", {})
        sp = sampling_from_fields(req.sampling, presets, max_default=s.args.get("default_max_tokens", 1024))
        if req.logprobs:
            sp.logprobs, sp.top_logprobs = True, max(sp.top_logprobs, req.top_logprobs)
        if req.confidence or s.args.get("conf_summary"):
            from .confidence import INTERNAL_TOP
            req.confidence = True
            sp.logprobs, sp.top_logprobs = True, max(sp.top_logprobs, INTERNAL_TOP)     # returned only if the client asked
        room = s.engine.engine.cfg.max_seq_len - len(toks)
        if room <= 0:
            raise BadRequest(f"prompt has {len(toks)} tokens; the context window is {s.engine.engine.cfg.max_seq_len}", "messages",
                             "context_length_exceeded")
        sp.max_tokens = min(sp.max_tokens, room)
        grammar = None
        spec = None
        rf = req.response_format or {}
        if rf.get("type") == "json_object":
            spec = GrammarSpec("json_object")
        elif rf.get("type") == "json_schema":
            schema = (rf.get("json_schema") or {}).get("schema") or rf.get("schema")
            if not isinstance(schema, dict):
                raise BadRequest("response_format.json_schema.schema must be an object", "response_format")
            spec = GrammarSpec("json_schema", schema=schema)
        elif rf.get("type") == "ebnf" or rf.get("type") == "grammar":
            spec = GrammarSpec("ebnf", ebnf=rf.get("grammar") or rf.get("ebnf"))
        require_tool = tools and (req.tool_choice == "required" or isinstance(req.tool_choice, dict))
        if require_tool and s.tool_parser_name in ("bare_json", "llama3_json"):
            chosen = tools
            if isinstance(req.tool_choice, dict):
                name = (req.tool_choice.get("function") or req.tool_choice).get("name")
                chosen = [t for t in tools if (t.get("function", t)).get("name") == name] or tools
            spec = GrammarSpec("tool_call", tools=chosen)
        if spec is not None and s.grammar is not None:
            try:
                grammar = s.grammar.matcher(spec)
            except Exception as e:
                raise BadRequest(f"could not compile the grammar: {e}", "response_format")
        procs = []
        if thinking and (req.thinking_budget or s.args.get("max_thinking_budget")):
            budget = min(x for x in (req.thinking_budget, s.args.get("max_thinking_budget")) if x)
            close_ids = tk.encode("</think>")
            procs.append(ThinkingBudget(close_ids, int(budget)))
        loop = bool(tools) and repeated_tool_call(req.messages)
        if not s.args.get("no_logit_pipeline") and (thinking or (tools and (require_tool or loop))):
            marker = next((m for m in get_parser(s.tool_parser_name, tools).markers if len(m) > 1), None) if tools else None
            procs.append(ThinkToolPipeline(
                think_open=tk.encode("<think>") if thinking else (), think_close=tk.encode("</think>") if thinking else (),
                tool_open=tk.encode(marker) if marker else (), token_text=lambda t: tk.decode([t]),
                starts_in_think=bool(thinking) and text.rstrip().endswith("<think>"), require_tool_call=bool(require_tool),
                suppress_tool_call=loop, streak=int(s.args.get("think_confidence_streak") or 0),
                margin=bool(s.args.get("margin_counter")), guard_pinned=bool(procs)))
        ns = s.sessions.namespace(req.cache_key)
        return toks, sp, grammar, procs, ns, thinking, tools, text

    # ------------------------------------------------------------------ streaming
    async def stream(self, req: GenRequest) -> AsyncIterator[GenDelta]:
        s = self.s
        toks, sp, grammar, procs, ns, thinking, tools, prompt_text = self.prepare(req)
        detok = IncrementalDetokenizer(s.tokenizer)
        reasoning = ReasoningSplitter(starts_in_reasoning=False) if (thinking or s.args.get("always_split_reasoning")) else None
        tool_stream = StreamingToolParser(get_parser(s.tool_parser_name, tools)) if tools else None
        stops = guarded_stops(req.stop, enabled=not s.args.get("no_output_sanitizer"))
        hold = max((len(x) for x in stops), default=0)
        pending = ""              # text held back while it could be the start of a stop string
        stopped = False
        n_out = 0
        t0 = time.monotonic()
        ttft = None
        lora = getattr(s.engine.engine.model, "lora", None)
        adapter_slot = lora.slot_of(req.adapter or s.active_adapter) if lora is not None else 0
        if req.adapter and not adapter_slot:
            raise ValueError(f"adapter '{req.adapter}' is not loaded")
        extra = {"images": req._images} if getattr(req, "_images", None) else {}
        gen_iter = s.engine.generate(toks, sp, request_id="req-" + req.request_id, namespace=ns, adapter_slot=adapter_slot, **extra,
                                     grammar=_GrammarAdapter(grammar) if grammar else None,
                                     logits_processors=procs, timeout_s=req.timeout_s, disable_spec=req.disable_spec,
                                     stop_checker=(LoopDetector(span=int(s.args.get("loop_guard_span") or 128))
                                                   if s.args.get("loop_guard") else None))
        final = None
        if req.echo and prompt_text:
            yield GenDelta(content=prompt_text)

        sanitize = not s.args.get("no_output_sanitizer")
        content_filter = ContentSanitizer() if sanitize else None
        guards = StreamGuards() if sanitize else None

        def clean(c: str) -> str:
            """Content channel only: leftover markup out, repetition watchdog fed with what the client will see."""
            if content_filter is not None and c:
                c = content_filter.feed(c)
            if guards is not None and c:
                guards.on_text(c)
            return c

        def route(text: str) -> GenDelta:
            d = GenDelta()
            if not text:
                return d
            r, c = (reasoning.push(text) if reasoning else ("", text))
            d.reasoning = r
            if c:
                d.content = clean(tool_stream.push(c) if tool_stream else c)
            return d

        async for ev in gen_iter:
            if ev.kind == "error":
                yield GenDelta(error=ev.error, finish_reason="error")
                return
            if ev.kind == "token":
                if ttft is None:
                    ttft = time.monotonic() - t0
                n_out += len(ev.tokens)
                text = detok.push(ev.tokens)
                out_text = text
                if stops and text:
                    pending += text
                    cut = min((pending.find(x) for x in stops if x in pending), default=-1)
                    if cut >= 0:
                        out_text, pending, stopped = pending[:cut], "", True
                    else:
                        keep = 0
                        for x in stops:
                            for k in range(min(len(x) - 1, len(pending)), 0, -1):
                                if pending.endswith(x[:k]):
                                    keep = max(keep, k)
                                    break
                        out_text, pending = pending[:len(pending) - keep], pending[len(pending) - keep:]
                d = route(out_text)
                d.token_ids, d.logprobs = list(ev.tokens), ev.logprobs
                if d.content or d.reasoning or d.token_ids:
                    yield d
                if guards is not None and guards.tripped and not stopped:
                    stopped = True                      # the visible text started to loop: end the turn here
                if stopped:
                    s.engine.abort("req-" + req.request_id)
                    break
            elif ev.kind == "done":
                final = ev.output
                break
        tail = "" if stopped else (pending + detok.flush())
        d = route(tail)
        if reasoning:
            r2, c2 = reasoning.finish()
            d.reasoning += r2
            if c2:
                d.content += clean(tool_stream.push(c2) if tool_stream else c2)
        calls: List[ToolCall] = []
        if tool_stream:
            rest, calls = tool_stream.finish()
            calls = dedupe_calls(calls)
            d.content += clean(rest)
            if calls and not req.parallel_tool_calls:
                calls = calls[:1]
            if guards is not None and len(calls) > guards.max_tool_calls:
                calls = calls[:guards.max_tool_calls]    # a response with dozens of calls is a failure mode, not a plan
        if content_filter is not None:
            d.content += content_filter.flush()
        d.tool_calls = calls
        reason = "stop" if stopped else (final.finish_reason if final else "stop")
        if calls:
            reason = "tool_calls"
        d.finish_reason = reason
        cached = final.cached_tokens if final else 0
        d.usage = {"prompt_tokens": len(toks), "completion_tokens": n_out, "total_tokens": len(toks) + n_out,
                   "prompt_tokens_details": {"cached_tokens": cached},
                   "completion_tokens_details": {"reasoning_tokens": 0,
                                                 "accepted_prediction_tokens": final.accepted_prediction_tokens if final else 0},
                   "time_to_first_token_ms": round((ttft or 0.0) * 1e3, 3),
                   "decode_time_ms": round((time.monotonic() - t0 - (ttft or 0.0)) * 1e3, 3)}
        s.metrics.on_request_done(len(toks), n_out, ttft)
        yield d


class _GrammarAdapter:
    """What the engine sees: ``token_mask(vocab)`` before sampling, ``accept(token)`` right after (both on the
    scheduler thread, so the matcher state never races the HTTP side)."""

    def __init__(self, matcher):
        self.m = matcher

    def token_mask(self, vocab: int):
        return self.m.token_mask(vocab)

    def accept(self, token: int) -> bool:
        return self.m.accept(token)


async def collect(gen: AsyncIterator[GenDelta]) -> GenDelta:
    """Aggregate a delta stream into one final delta (non-streaming responses)."""
    out = GenDelta()
    lps: list = []
    async for d in gen:
        out.content += d.content
        out.reasoning += d.reasoning
        out.tool_calls += d.tool_calls
        out.token_ids += d.token_ids
        if d.logprobs:
            lps += d.logprobs
        if d.finish_reason:
            out.finish_reason = d.finish_reason
        if d.usage:
            out.usage = d.usage
        if d.error:
            out.error = d.error
    out.logprobs = lps or None
    return out
