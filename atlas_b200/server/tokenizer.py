"""Tokenizers, incremental detokenisation and chat-template rendering.

* :class:`HFTokenizer` loads ``tokenizer.json`` (+ ``tokenizer_config.json`` / ``chat_template.jinja``) from a model
  directory.
* :class:`ByteTokenizer` is a dependency-free UTF-8 byte tokenizer used with random-init models and in tests.
* :func:`render_chat` renders OpenAI-style messages (+tools) through the model's Jinja chat template, falling back
  to ChatML.

Reference parity: ``crates/spark-server/src/tokenizer/*`` (tokenizer + minijinja ``chat_render.rs``),
``api/chat/template.rs``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence

CHATML_TEMPLATE = (
    "{%- if tools %}{{- '<|im_start|>system\\n' }}{%- if messages[0].role == 'system' %}{{- messages[0].content + '\\n\\n' }}{%- endif %}"
    "{{- '# Tools\\n\\nYou may call one or more functions to assist with the user query.\\n\\nYou are provided with function "
    "signatures within <tools></tools> XML tags:\\n<tools>' }}{%- for tool in tools %}{{- '\\n' }}{{- tool | tojson }}{%- endfor %}"
    "{{- '\\n</tools>\\n\\nFor each function call, return a json object with function name and arguments within "
    "<tool_call></tool_call> XML tags:\\n<tool_call>\\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\\n</tool_call>"
    "<|im_end|>\\n' }}{%- elif messages[0].role == 'system' %}{{- '<|im_start|>system\\n' + messages[0].content + '<|im_end|>\\n' }}{%- endif %}"
    "{%- for message in messages %}{%- if message.role == 'system' and loop.first %}{%- elif message.role == 'tool' %}"
    "{{- '<|im_start|>user\\n<tool_response>\\n' + (message.content | string) + '\\n</tool_response><|im_end|>\\n' }}"
    "{%- elif message.role == 'assistant' %}{{- '<|im_start|>assistant\\n' }}{%- if message.content %}{{- message.content }}{%- endif %}"
    "{%- if message.tool_calls %}{%- for tc in message.tool_calls %}{{- '\\n<tool_call>\\n{\"name\": \"' + tc.function.name + '\", \"arguments\": ' }}"
    "{%- if tc.function.arguments is string %}{{- tc.function.arguments }}{%- else %}{{- tc.function.arguments | tojson }}{%- endif %}"
    "{{- '}\\n</tool_call>' }}{%- endfor %}{%- endif %}{{- '<|im_end|>\\n' }}"
    "{%- else %}{{- '<|im_start|>' + message.role + '\\n' + (message.content | string) + '<|im_end|>\\n' }}{%- endif %}{%- endfor %}"
    "{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}{%- if enable_thinking is defined and enable_thinking is false %}"
    "{{- '<think>\\n\\n</think>\\n\\n' }}{%- endif %}{%- endif %}"
)


class BaseTokenizer:
    vocab_size: int = 0
    eos_token_ids: List[int] = []
    bos_token_id: Optional[int] = None
    chat_template: Optional[str] = None

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]: raise NotImplementedError
    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str: raise NotImplementedError
    def token_to_piece(self, tid: int) -> str:
        return self.decode([tid], skip_special_tokens=False)
    def token_id(self, text: str) -> Optional[int]:
        ids = self.encode(text)
        return ids[0] if len(ids) == 1 else None


class ByteTokenizer(BaseTokenizer):
    """ids 0..2 = pad / bos / eos, id 3+b = byte b; ids above 258 decode to nothing."""

    def __init__(self, vocab_size: int = 1024):
        self.vocab_size = vocab_size
        self.bos_token_id, self.eos_token_ids = 1, [2]
        self.chat_template = None

    def encode(self, text, add_special_tokens=False):
        ids = [3 + b for b in text.encode("utf-8")]
        return ([1] + ids) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens=True):
        bs = bytes(i - 3 for i in ids if 3 <= i < 259)
        return bs.decode("utf-8", errors="replace")


class HFTokenizer(BaseTokenizer):
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        tj = os.path.join(path, "tokenizer.json") if os.path.isdir(path) else path
        self.tk = Tokenizer.from_file(tj)
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        base = os.path.dirname(tj)
        cfg: Dict[str, Any] = {}
        for name in ("tokenizer_config.json",):
            p = os.path.join(base, name)
            if os.path.exists(p):
                with open(p) as f:
                    cfg = json.load(f)
        self.chat_template = cfg.get("chat_template")
        if isinstance(self.chat_template, list):      # named templates
            self.chat_template = next((t["template"] for t in self.chat_template if t.get("name") == "default"),
                                      self.chat_template[0]["template"])
        jt = os.path.join(base, "chat_template.jinja")
        if os.path.exists(jt):
            with open(jt) as f:
                self.chat_template = f.read()

        def tok_str(v):
            return v.get("content") if isinstance(v, dict) else v
        self.bos_token = tok_str(cfg.get("bos_token"))
        self.eos_token = tok_str(cfg.get("eos_token"))
        self.bos_token_id = self.tk.token_to_id(self.bos_token) if self.bos_token else None
        eos = set()
        if self.eos_token and self.tk.token_to_id(self.eos_token) is not None:
            eos.add(self.tk.token_to_id(self.eos_token))
        gc = os.path.join(base, "generation_config.json")
        if os.path.exists(gc):
            with open(gc) as f:
                g = json.load(f).get("eos_token_id")
            if isinstance(g, int):
                eos.add(g)
            elif isinstance(g, list):
                eos.update(int(x) for x in g)
        self.eos_token_ids = sorted(eos)

    def encode(self, text, add_special_tokens=False):
        return self.tk.encode(text, add_special_tokens=add_special_tokens).ids

    def decode(self, ids, skip_special_tokens=True):
        return self.tk.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def token_id(self, text):
        return self.tk.token_to_id(text)


def load_tokenizer(path: Optional[str], vocab_size: int = 1024) -> BaseTokenizer:
    if path and (os.path.exists(os.path.join(path, "tokenizer.json")) or path.endswith(".json")):
        return HFTokenizer(path)
    return ByteTokenizer(vocab_size)


class IncrementalDetokenizer:
    """Streams text for a growing token list without re-decoding everything and without emitting half a
    multi-byte character (holds output back while the tail decodes to U+FFFD)."""

    def __init__(self, tokenizer: BaseTokenizer, skip_special_tokens: bool = True, window: int = 6):
        self.tk, self.skip, self.window = tokenizer, skip_special_tokens, window
        self.ids: List[int] = []
        self.prefix_offset = 0
        self.read_offset = 0
        self.text = ""

    def push(self, new_ids: Sequence[int]) -> str:
        self.ids.extend(new_ids)
        prefix_text = self.tk.decode(self.ids[self.prefix_offset:self.read_offset], self.skip)
        new_text = self.tk.decode(self.ids[self.prefix_offset:], self.skip)
        if len(new_text) > len(prefix_text) and not new_text.endswith("\ufffd"):
            delta = new_text[len(prefix_text):]
            self.prefix_offset = self.read_offset
            self.read_offset = len(self.ids)
            self.text += delta
            return delta
        return ""

    def flush(self) -> str:
        """Whatever is still held back (e.g. a dangling partial character) at end of stream."""
        prefix_text = self.tk.decode(self.ids[self.prefix_offset:self.read_offset], self.skip)
        new_text = self.tk.decode(self.ids[self.prefix_offset:], self.skip)
        delta = new_text[len(prefix_text):]
        self.prefix_offset = self.read_offset = len(self.ids)
        self.text += delta
        return delta


# ----------------------------------------------------------------------------- chat templates
_env = None


def _jinja_env():
    global _env
    if _env is None:
        import datetime
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(msg):
            raise ValueError(msg)
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = raise_exception
        env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
        env.filters["tojson"] = lambda v, indent=None, ensure_ascii=False: json.dumps(v, ensure_ascii=ensure_ascii, indent=indent)
        _env = env
    return _env


def normalise_messages(messages: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """Flatten content-part lists to text (image / video parts become placeholders) and parse tool-call argument
    strings so templates that iterate ``arguments`` as a mapping work."""
    out = []
    for m in messages:
        m = dict(m)
        c = m.get("content")
        if isinstance(c, list):
            parts = []
            for p in c:
                t = p.get("type")
                if t in ("text", "input_text", "output_text"):
                    parts.append(p.get("text", ""))
                elif t in ("image_url", "image", "input_image"):
                    parts.append("<|vision_start|><|image_pad|><|vision_end|>")
                elif t in ("video_url", "video"):
                    parts.append("<|vision_start|><|video_pad|><|vision_end|>")
                elif t == "tool_result":
                    parts.append(json.dumps(p.get("content")) if not isinstance(p.get("content"), str) else p["content"])
            m["content"] = "".join(parts)
        elif c is None:
            m["content"] = ""
        if m.get("tool_calls"):
            tcs = []
            for tc in m["tool_calls"]:
                tc = json.loads(json.dumps(tc))
                fn = tc.get("function", {})
                if isinstance(fn.get("arguments"), str):
                    try:
                        fn["arguments"] = json.loads(fn["arguments"])
                    except Exception:
                        pass
                tcs.append(tc)
            m["tool_calls"] = tcs
        out.append(m)
    return out


def render_chat(tokenizer: BaseTokenizer, messages: List[Dict[str, Any]], tools: Optional[List[dict]] = None,
                add_generation_prompt: bool = True, template: Optional[str] = None, **kwargs) -> str:
    tpl = template or tokenizer.chat_template or CHATML_TEMPLATE
    t = _jinja_env().from_string(tpl)
    return t.render(messages=normalise_messages(messages), tools=tools or None,
                    add_generation_prompt=add_generation_prompt,
                    bos_token=getattr(tokenizer, "bos_token", "") or "", eos_token=getattr(tokenizer, "eos_token", "") or "",
                    **kwargs)
