"""Constrained decoding: JSON-object / JSON-schema / tool-call / EBNF grammars compiled to per-step token masks.

Default backend: the engine's own matcher (``server/ebnf.py`` over the native ``csrc/runtime/grammar.cpp``): grammars
are compiled once per distinct spec, the tokenizer's vocabulary once per engine.  ``ATLAS_GRAMMAR_BACKEND=xgrammar``
selects the upstream ``xgrammar`` package instead when it is importable.

Reference parity: ``crates/xgrammar`` + ``crates/spark-server/src/grammar/{engine,compile_tools,mask_cache}.rs``;
``GrammarSpec::{ToolCall, JsonObject, JsonSchema, Ebnf}`` (``api/inference_types.rs``).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch


@dataclass
class GrammarSpec:
    kind: str                      # json_object | json_schema | tool_call | ebnf
    schema: Optional[dict] = None
    ebnf: Optional[str] = None
    tools: Optional[List[dict]] = None


def tools_to_schema(tools: List[dict], allow_multiple: bool = False) -> dict:
    """JSON schema of ``{"name": <one of the tools>, "arguments": <that tool's parameters>}``."""
    alts = []
    for t in tools:
        fn = t.get("function", t)
        alts.append({"type": "object", "properties": {"name": {"const": fn["name"]},
                                                        "arguments": fn.get("parameters") or {"type": "object"}},
                     "required": ["name", "arguments"], "additionalProperties": False})
    one = {"anyOf": alts} if len(alts) != 1 else alts[0]
    return {"type": "array", "items": one, "minItems": 1} if allow_multiple else one


class GrammarEngine:
    def __init__(self, tokenizer, vocab_size: int):
        self.tokenizer, self.vocab_size = tokenizer, vocab_size
        self._xgr = None
        self._compiler = None
        self._cache: Dict[str, Any] = {}
        self._vocab = None                       # ebnf.Vocabulary, built on first use
        import os
        if os.environ.get("ATLAS_GRAMMAR_BACKEND", "native") != "xgrammar":
            return
        try:
            import xgrammar as xgr
            tk = getattr(tokenizer, "tk", None)
            if tk is not None:
                vocab = [None] * tokenizer.vocab_size
                for tok, i in tk.get_vocab(with_added_tokens=True).items():
                    if i < len(vocab):
                        vocab[i] = tok
                info = xgr.TokenizerInfo([v if v is not None else "" for v in vocab], vocab_size=vocab_size,
                                         stop_token_ids=list(tokenizer.eos_token_ids) or None)
                self._compiler = xgr.GrammarCompiler(info)
                self._xgr = xgr
        except Exception:
            self._xgr = None

    @property
    def backend(self) -> str:
        return "xgrammar" if self._xgr is not None else "native"

    def matcher(self, spec: GrammarSpec):
        if self._xgr is not None:
            key = json.dumps([spec.kind, spec.schema, spec.ebnf, spec.tools], sort_keys=True, default=str)
            cg = self._cache.get(key)
            if cg is None:
                if spec.kind == "json_object":
                    cg = self._compiler.compile_builtin_json_grammar()
                elif spec.kind == "json_schema":
                    cg = self._compiler.compile_json_schema(json.dumps(spec.schema))
                elif spec.kind == "tool_call":
                    cg = self._compiler.compile_json_schema(json.dumps(tools_to_schema(spec.tools or [])))
                elif spec.kind == "ebnf":
                    cg = self._compiler.compile_grammar(spec.ebnf)
                else:
                    raise ValueError(f"unknown grammar kind {spec.kind}")
                self._cache[key] = cg
            return _XgrMatcher(self._xgr, cg, self.vocab_size)
        from . import ebnf
        if self._vocab is None:
            toks = ebnf.token_bytes(self.tokenizer, self.vocab_size)
            if not any(toks):
                return None                      # a tokenizer whose token bytes are unknown cannot be masked
            self._vocab = ebnf.Vocabulary(toks, list(getattr(self.tokenizer, "eos_token_ids", []) or []))
        key = json.dumps([spec.kind, spec.schema, spec.ebnf, spec.tools], sort_keys=True, default=str)
        cg = self._cache.get(key)
        if cg is None:
            if spec.kind == "json_object":
                text = ebnf.JSON_OBJECT_GRAMMAR
            elif spec.kind == "json_schema":
                text = ebnf.schema_to_ebnf(spec.schema or {})
            elif spec.kind == "tool_call":
                text = ebnf.schema_to_ebnf(tools_to_schema(spec.tools or []))
            elif spec.kind == "ebnf":
                text = spec.ebnf or ""
            else:
                raise ValueError(f"unknown grammar kind {spec.kind}")
            cg = self._cache[key] = ebnf.CompiledGrammar(text)
        return ebnf.EbnfMatcher(cg, self._vocab)


class _XgrMatcher:
    def __init__(self, xgr, compiled, vocab_size: int):
        self.xgr = xgr
        self.m = xgr.GrammarMatcher(compiled)
        self.vocab_size = vocab_size
        self.bitmask = xgr.allocate_token_bitmask(1, vocab_size)

    def token_mask(self, vocab: int) -> Optional[torch.Tensor]:
        if self.m.is_terminated():
            return None
        self.m.fill_next_token_bitmask(self.bitmask)
        bits = self.bitmask[0]
        idx = torch.arange(vocab)
        return ((bits[idx // 32] >> (idx % 32)) & 1).bool()

    def accept(self, token: int) -> bool:
        return self.m.accept_token(int(token))

    def terminated(self) -> bool:
        return self.m.is_terminated()


class _ByteJsonMatcher:
    """Byte-level pushdown check that the output stays a prefix of one JSON object; after it closes only EOS."""

    def __init__(self, vocab_size: int):
        self.vocab_size = vocab_size
        self.stack: List[str] = []
        self.in_str = self.esc = False
        self.started = self.closed = False

    def token_mask(self, vocab: int) -> Optional[torch.Tensor]:
        mask = torch.zeros(vocab, dtype=torch.bool)
        if self.closed:
            mask[2] = True
            return mask
        if not self.started:
            for ch in b" \n{":
                mask[3 + ch] = True
            return mask
        mask[3:259] = True
        if not self.in_str:
            for ch in b"}]":
                ok = bool(self.stack) and self.stack[-1] == chr(ch)
                mask[3 + ch] = ok
        return mask

    def accept(self, token: int) -> bool:
        if not (3 <= token < 259):
            return token == 2 and self.closed
        ch = chr(token - 3)
        if self.in_str:
            if self.esc:
                self.esc = False
            elif ch == "\\":
                self.esc = True
            elif ch == '"':
                self.in_str = False
            return True
        if ch == '"':
            self.in_str = True
        elif ch in "{[":
            self.started = True
            self.stack.append("}" if ch == "{" else "]")
        elif ch in "}]":
            if not self.stack or self.stack[-1] != ch:
                return False
            self.stack.pop()
            if not self.stack:
                self.closed = True
        return True

    def terminated(self) -> bool:
        return self.closed
