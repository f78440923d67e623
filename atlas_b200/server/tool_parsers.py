"""Tool-call parsers (complete-text and streaming) for the model dialects the server speaks.

Each parser turns generated text into ``(visible_content, [ToolCall])``.  The streaming wrapper holds text
back only while it could still be the start of a tool-call marker, so ordinary content streams through
immediately and tool calls are emitted once their block closes.

Dialects: ``hermes`` (``<tool_call>{json}</tool_call>``), ``qwen3_coder`` / ``qwen3_xml``
(``<tool_call><function=name><parameter=k>v</parameter></function></tool_call>``), ``mistral``
(``[TOOL_CALLS][{...}]``), ``llama3_json`` / ``bare_json`` (a bare JSON object / array with name+arguments),
``minimax_xml`` (``<minimax:tool_call><invoke name=..><parameter name=..>``), ``deepseek_dsml``
(``<｜tool▁call▁begin｜>name<｜tool▁sep｜>{json}<｜tool▁call▁end｜>``), ``gemma`` (```` ```tool_code```` blocks).

Reference parity: ``crates/spark-server/src/tool_parser/*`` (hermes, qwen3_coder, qwen3_xml, mistral, gemma4,
minimax_xml, deepseek_v4_dsml, bare_json, lfm3, poolside_v1) and the streaming emitters used by ``api/chat_stream/handle_token.rs``.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class ToolCall:
    name: str
    arguments: str                      # JSON text
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_openai(self, index: int = 0) -> Dict[str, Any]:
        return {"index": index, "id": self.id, "type": "function",
                "function": {"name": self.name, "arguments": self.arguments}}


def dedupe_calls(calls: List["ToolCall"]) -> List["ToolCall"]:
    """Drop repeated calls of one turn that name the same function with the same arguments (compared as parsed JSON, so
    key order and whitespace do not matter); the first occurrence stays.  Models in a repetition loop emit the same
    call several times, and executing it more than once is never what the client wants.
    Reference behaviour replaced: ``crates/spark-server/src/tool_arg_dedup.rs``."""
    seen, out = set(), []
    for c in calls:
        try:
            key = (c.name, json.dumps(json.loads(c.arguments), sort_keys=True))
        except (ValueError, TypeError):
            key = (c.name, c.arguments)
        if key not in seen:
            seen.add(key)
            out.append(c)
    return out


def _json_args(v: Any) -> str:
    if isinstance(v, str):
        try:
            json.loads(v)
            return v
        except Exception:
            return json.dumps(v)
    return json.dumps(v if v is not None else {}, ensure_ascii=False)


def _coerce_param(v: str, schema: Optional[dict]) -> Any:
    """XML-style dialects carry parameters as text: coerce by the declared JSON-schema type, else by literal."""
    t = (schema or {}).get("type")
    s = v.strip("\n")
    if t == "string":
        return s
    if t in ("integer", "number", "boolean", "object", "array", "null") or t is None:
        try:
            return json.loads(s)
        except Exception:
            if t == "integer":
                try:
                    return int(s)
                except Exception:
                    pass
            if t == "boolean":
                return s.strip().lower() == "true"
    return s


class ToolParser:
    name = "base"
    markers: Tuple[str, ...] = ()           # strings whose prefix must be held back while streaming
    system_prompt_tools = True              # False: the model's own chat template renders the tool schemas

    def __init__(self, tools: Optional[List[dict]] = None):
        self.tools = tools or []
        self.schemas: Dict[str, dict] = {}
        for t in self.tools:
            fn = t.get("function", t)
            if "name" in fn:
                self.schemas[fn["name"]] = (fn.get("parameters") or fn.get("input_schema") or {}).get("properties", {})

    def parse(self, text: str) -> Tuple[str, List[ToolCall]]:
        raise NotImplementedError


class HermesParser(ToolParser):
    name = "hermes"
    markers = ("<tool_call>",)
    _re = re.compile(r"<tool_call>\s*(.*?)\s*(?:</tool_call>|$)", re.S)

    def parse(self, text):
        calls = []
        for m in self._re.finditer(text):
            body = m.group(1).strip()
            try:
                obj = json.loads(body)
            except Exception:
                obj = _lenient_json(body)
            if isinstance(obj, dict) and "name" in obj:
                calls.append(ToolCall(obj["name"], _json_args(obj.get("arguments", obj.get("parameters", {})))))
        content = self._re.sub("", text).strip() if calls else text
        return content, calls


class Qwen3CoderParser(ToolParser):
    name = "qwen3_coder"
    markers = ("<tool_call>", "<function=")
    _fn = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|$)", re.S)
    _pa = re.compile(r"<parameter=([^>\s]+)>(.*?)(?:</parameter>|(?=<parameter=)|$)", re.S)

    def parse(self, text):
        calls = []
        for m in self._fn.finditer(text):
            name, body = m.group(1), m.group(2)
            props = self.schemas.get(name, {})
            args = {pm.group(1): _coerce_param(pm.group(2), props.get(pm.group(1))) for pm in self._pa.finditer(body)}
            calls.append(ToolCall(name, json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        content = re.sub(r"<tool_call>.*?(?:</tool_call>|$)", "", text, flags=re.S)
        content = self._fn.sub("", content).strip()
        return content, calls


class Lfm3Parser(Qwen3CoderParser):
    """LFM3 emits the qwen3_coder block form (``<tool_call><function=NAME><parameter=K>V</parameter></function>``), so
    extraction and typed coercion are shared; what differs is the prompt side: the checkpoint's own chat template
    already renders the tool schemas, so this dialect adds no tool instructions of its own
    (``system_prompt_tools`` is False; reference: ``crates/spark-server/src/tool_parser/lfm3.rs``)."""
    name = "lfm3"
    system_prompt_tools = False


class PoolsideV1Parser(ToolParser):
    """``<tool_call>NAME<arg_key>K</arg_key><arg_value>V</arg_value>...</tool_call>``; values are text, coerced by the
    declared schema type (reference: ``crates/spark-server/src/tool_parser/poolside_v1.rs``)."""
    name = "poolside_v1"
    markers = ("<tool_call>",)
    system_prompt_tools = False
    _call = re.compile(r"<tool_call>\s*([^<\s]+)\s*(.*?)(?:</tool_call>|$)", re.S)
    _kv = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)(?:</arg_value>|(?=<arg_key>)|$)", re.S)

    def parse(self, text):
        calls = []
        for m in self._call.finditer(text):
            name, body = m.group(1), m.group(2)
            props = self.schemas.get(name, {})
            args = {k.strip(): _coerce_param(v, props.get(k.strip())) for k, v in self._kv.findall(body)}
            calls.append(ToolCall(name, json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        return self._call.sub("", text).strip(), calls

    @staticmethod
    def format_tool_calls(calls: List[dict]) -> str:
        """Earlier assistant tool calls rendered back into the dialect (for templates that expect raw text)."""
        out = []
        for c in calls:
            fn = c.get("function", c)
            try:
                args = json.loads(fn.get("arguments") or "{}")
            except ValueError:
                args = {}
            body = "".join(f"<arg_key>{k}</arg_key><arg_value>{v if isinstance(v, str) else json.dumps(v)}</arg_value>"
                           for k, v in (args.items() if isinstance(args, dict) else []))
            out.append(f"<tool_call>{fn.get('name', '')}{body}</tool_call>")
        return "".join(out)


class MistralParser(ToolParser):
    name = "mistral"
    markers = ("[TOOL_CALLS]",)

    def parse(self, text):
        if "[TOOL_CALLS]" not in text:
            return text, []
        head, _, tail = text.partition("[TOOL_CALLS]")
        tail = tail.strip()
        calls = []
        try:
            arr = json.loads(tail)
        except Exception:
            arr = _lenient_json(tail)
        if isinstance(arr, dict):
            arr = [arr]
        if isinstance(arr, list):
            for o in arr:
                if isinstance(o, dict) and "name" in o:
                    calls.append(ToolCall(o["name"], _json_args(o.get("arguments", {}))))
        else:   # newer dialect: name{json}
            m = re.match(r"([\w\-\.]+)\s*(\{.*\})", tail, re.S)
            if m:
                calls.append(ToolCall(m.group(1), _json_args(m.group(2))))
        return head.strip(), calls


class BareJsonParser(ToolParser):
    name = "bare_json"
    markers = ("{", "[")

    def parse(self, text):
        s = text.strip()
        if s.startswith("<|python_tag|>"):
            s = s[len("<|python_tag|>"):].strip()
        if not s or s[0] not in "{[":
            return text, []
        try:
            obj = json.loads(s)
        except Exception:
            obj = _lenient_json(s)
        objs = obj if isinstance(obj, list) else [obj]
        calls = []
        for o in objs:
            if isinstance(o, dict) and "name" in o and ("arguments" in o or "parameters" in o):
                if not self.schemas or o["name"] in self.schemas:
                    calls.append(ToolCall(o["name"], _json_args(o.get("arguments", o.get("parameters")))))
        return ("", calls) if calls else (text, [])


class MinimaxXmlParser(ToolParser):
    name = "minimax_xml"
    markers = ("<minimax:tool_call>",)
    _inv = re.compile(r"<invoke name=\"([^\"]+)\">(.*?)(?:</invoke>|$)", re.S)
    _pa = re.compile(r"<parameter name=\"([^\"]+)\">(.*?)</parameter>", re.S)

    def parse(self, text):
        calls = []
        for m in self._inv.finditer(text):
            props = self.schemas.get(m.group(1), {})
            args = {p.group(1): _coerce_param(p.group(2), props.get(p.group(1))) for p in self._pa.finditer(m.group(2))}
            calls.append(ToolCall(m.group(1), json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        return re.sub(r"<minimax:tool_call>.*?(?:</minimax:tool_call>|$)", "", text, flags=re.S).strip(), calls


class DeepseekDsmlParser(ToolParser):
    name = "deepseek_dsml"
    markers = ("<｜tool▁calls▁begin｜>", "<｜tool▁call▁begin｜>")
    _re = re.compile(r"<｜tool▁call▁begin｜>(?:function<｜tool▁sep｜>)?([^\n<]+?)(?:<｜tool▁sep｜>|\n```json\n)(.*?)(?:```)?\s*<｜tool▁call▁end｜>", re.S)

    def parse(self, text):
        calls = [ToolCall(m.group(1).strip(), _json_args(m.group(2).strip())) for m in self._re.finditer(text)]
        if not calls:
            return text, []
        return text.split("<｜tool▁calls▁begin｜>")[0].split("<｜tool▁call▁begin｜>")[0].strip(), calls


class GemmaParser(ToolParser):
    name = "gemma"
    markers = ("```tool_code", "```tool_call")
    _re = re.compile(r"```tool_(?:code|call)\s*\n(.*?)```", re.S)
    _call = re.compile(r"(?:print\()?\s*([\w\.]+)\((.*)\)\s*\)?\s*$", re.S)

    def parse(self, text):
        calls = []
        for m in self._re.finditer(text):
            body = m.group(1).strip()
            try:
                o = json.loads(body)
                if isinstance(o, dict) and "name" in o:
                    calls.append(ToolCall(o["name"], _json_args(o.get("arguments", o.get("parameters", {})))))
                    continue
            except Exception:
                pass
            cm = self._call.match(body)
            if cm:
                args: Dict[str, Any] = {}
                for kv in _split_top_level(cm.group(2)):
                    if "=" in kv:
                        k, v = kv.split("=", 1)
                        try:
                            args[k.strip()] = json.loads(v.strip().replace("'", '"'))
                        except Exception:
                            args[k.strip()] = v.strip().strip("'\"")
                calls.append(ToolCall(cm.group(1), json.dumps(args)))
        if not calls:
            return text, []
        return self._re.sub("", text).strip(), calls


def _split_top_level(s: str) -> List[str]:
    out, depth, cur, q = [], 0, "", None
    for ch in s:
        if q:
            cur += ch
            if ch == q:
                q = None
            continue
        if ch in "'\"":
            q = ch
        elif ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur)
    return out


def _lenient_json(s: str) -> Any:
    """Best effort for truncated / trailing-garbage JSON: longest prefix that parses after closing brackets."""
    s = s.strip()
    dec = json.JSONDecoder()
    try:
        obj, _ = dec.raw_decode(s)
        return obj
    except Exception:
        pass
    stack, in_str, esc = [], False, False
    for ch in s:
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        elif ch in "{[":
            stack.append("}" if ch == "{" else "]")
        elif ch in "}]" and stack:
            stack.pop()
    fixed = s + ('"' if in_str else "") + "".join(reversed(stack))
    try:
        return json.loads(fixed)
    except Exception:
        return None


PARSERS = {c.name: c for c in (HermesParser, Qwen3CoderParser, MistralParser, BareJsonParser, MinimaxXmlParser,
                               DeepseekDsmlParser, GemmaParser, Lfm3Parser, PoolsideV1Parser)}
PARSERS["poolside"] = PoolsideV1Parser
PARSERS["qwen3_xml"] = Qwen3CoderParser
PARSERS["llama3_json"] = BareJsonParser
PARSERS["gemma4"] = GemmaParser
PARSERS["deepseek_v4_dsml"] = DeepseekDsmlParser


def get_parser(name: Optional[str], tools: Optional[List[dict]] = None) -> ToolParser:
    cls = PARSERS.get((name or "hermes").lower())
    if cls is None:
        raise ValueError(f"unknown tool-call parser '{name}' (known: {sorted(PARSERS)})")
    return cls(tools)


def default_parser_for(model_type: str) -> str:
    mt = model_type.lower()
    if mt.startswith("qwen3_next") or "coder" in mt:
        return "qwen3_coder"
    if mt.startswith(("mistral", "mixtral")):
        return "mistral"
    if mt.startswith("llama"):
        return "llama3_json"
    if mt.startswith("gemma"):
        return "gemma"
    if mt.startswith("minimax"):
        return "minimax_xml"
    if mt.startswith("deepseek"):
        return "deepseek_dsml"
    if mt.startswith("lfm"):
        return "lfm3"
    if mt.startswith(("laguna", "poolside")):
        return "poolside_v1"
    return "hermes"


class StreamingToolParser:
    """Feeds text deltas; returns the content that may be shown now.  Text from the first tool-call marker on
    is buffered; :meth:`finish` parses it into tool calls."""

    def __init__(self, parser: ToolParser):
        self.parser = parser
        self.buf = ""            # undecided tail (could be a marker prefix) or the tool-call block
        self.in_tool = False
        self.emitted = ""

    def push(self, delta: str) -> str:
        self.buf += delta
        if self.in_tool:
            return ""
        markers = [m for m in self.parser.markers if len(m) > 1]
        if not markers:
            # bare-json dialects: the whole message is either content or a call; decide on the first character
            if self.emitted == "" and self.buf.lstrip()[:1] in ("{", "["):
                self.in_tool = True
                return ""
            out, self.buf = self.buf, ""
            self.emitted += out
            return out
        idx = min((self.buf.find(m) for m in markers if m in self.buf), default=-1)
        if idx >= 0:
            out, self.buf = self.buf[:idx], self.buf[idx:]
            self.in_tool = True
            self.emitted += out
            return out
        hold = 0
        for m in markers:
            for k in range(min(len(m) - 1, len(self.buf)), 0, -1):
                if self.buf.endswith(m[:k]):
                    hold = max(hold, k)
                    break
        out = self.buf[:len(self.buf) - hold] if hold else self.buf
        self.buf = self.buf[len(out):]
        self.emitted += out
        return out

    def finish(self) -> Tuple[str, List[ToolCall]]:
        """Returns (remaining visible content, tool calls)."""
        if not self.buf:
            return "", []
        content, calls = self.parser.parse(self.buf)
        self.buf = ""
        if calls:
            return content, calls
        return content, []
