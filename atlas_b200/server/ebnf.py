"""The engine's own grammar backend: EBNF grammars (and JSON schemas lowered to EBNF) compiled by the native matcher in
``csrc/runtime/grammar.cpp`` and turned into per-step token masks over the tokenizer's byte-level vocabulary.

``schema_to_ebnf`` covers the JSON-schema subset tool calls and structured outputs use: ``type`` (object / array /
string / number / integer / boolean / null, or a list of them), ``properties`` + ``required`` +
``additionalProperties``, ``items`` + ``minItems`` / ``maxItems``, ``enum``, ``const``, ``anyOf`` / ``oneOf``,
``$ref`` into ``$defs`` / ``definitions``, string ``minLength`` / ``maxLength``.  Object properties are emitted in
declaration order (required ones always, optional ones may be skipped), which is how models are prompted to write them.

Reference parity: ``crates/xgrammar`` (grammar compiler, JSON-schema front end, token-mask cache) and
``crates/spark-server/src/grammar/compile_tools.rs`` (tool list -> schema).
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Dict, List, Optional, Sequence

import torch

from .. import runtime_native as rn

JSON_PRELUDE = r'''
ws ::= [ \t\n\r]*
json-string ::= "\"" json-char* "\""
json-char ::= [^"\\\x00-\x1f] | "\\" (["\\/bfnrt] | "u" [0-9a-fA-F]{4})
json-int ::= "-"? ("0" | [1-9] [0-9]*)
json-number ::= json-int ("." [0-9]+)? ([eE] [-+]? [0-9]+)?
json-bool ::= "true" | "false"
json-null ::= "null"
json-value ::= json-object | json-array | json-string | json-number | json-bool | json-null
json-object ::= "{" ws (json-string ws ":" ws json-value (ws "," ws json-string ws ":" ws json-value)*)? ws "}"
json-array ::= "[" ws (json-value (ws "," ws json-value)*)? ws "]"
'''

JSON_OBJECT_GRAMMAR = "root ::= ws json-object ws\n" + JSON_PRELUDE


def _lit(s: str) -> str:
    """EBNF literal matching the JSON text ``s`` exactly."""
    out = []
    for ch in s:
        if ch == '"':
            out.append('\\"')
        elif ch == "\\":
            out.append("\\\\")
        elif ch == "\n":
            out.append("\\n")
        elif ch == "\r":
            out.append("\\r")
        elif ch == "\t":
            out.append("\\t")
        elif ord(ch) < 0x20:
            out.append("\\x%02x" % ord(ch))
        else:
            out.append(ch)
    return '"' + "".join(out) + '"'


class _SchemaLowering:
    def __init__(self, root_schema: dict):
        self.root_schema = root_schema
        self.rules: List[str] = []
        self.named: Dict[str, str] = {}          # $ref target -> rule name
        self.n = 0

    def fresh(self, hint: str) -> str:
        self.n += 1
        return f"s{self.n}-{hint}"

    def resolve(self, ref: str) -> dict:
        if not ref.startswith("#/"):
            raise ValueError(f"only local $ref is supported: {ref}")
        node = self.root_schema
        for part in ref[2:].split("/"):
            node = node[part.replace("~1", "/").replace("~0", "~")]
        return node

    def lower(self, sch, hint: str = "v") -> str:
        """Returns an EBNF expression (a rule name or an inline expression) for ``sch``."""
        if sch is True or sch == {} or sch is None:
            return "json-value"
        if sch is False:
            raise ValueError("schema 'false' admits nothing")
        if "$ref" in sch:
            ref = sch["$ref"]
            if ref not in self.named:
                name = self.fresh("ref")
                self.named[ref] = name
                self.rules.append(f"{name} ::= {self.lower(self.resolve(ref), 'ref')}")
            return self.named[ref]
        if "const" in sch:
            return _lit(json.dumps(sch["const"], ensure_ascii=False))
        if "enum" in sch:
            return "(" + " | ".join(_lit(json.dumps(v, ensure_ascii=False)) for v in sch["enum"]) + ")"
        for key in ("anyOf", "oneOf"):
            if key in sch:
                return "(" + " | ".join(self.lower(s, hint) for s in sch[key]) + ")"
        if "allOf" in sch and len(sch["allOf"]) == 1:
            return self.lower(sch["allOf"][0], hint)
        t = sch.get("type")
        if isinstance(t, list):
            return "(" + " | ".join(self.lower({**sch, "type": one}, hint) for one in t) + ")"
        if t is None:
            t = "object" if "properties" in sch else "array" if "items" in sch else None
        if t == "string":
            lo, hi = sch.get("minLength"), sch.get("maxLength")
            if lo is None and hi is None:
                return "json-string"
            rep = "{%d,%s}" % (lo or 0, "" if hi is None else hi)
            return '("\\"" json-char' + rep + ' "\\"")'
        if t == "integer":
            return "json-int"
        if t == "number":
            return "json-number"
        if t == "boolean":
            return "json-bool"
        if t == "null":
            return "json-null"
        if t == "array":
            item = self.lower(sch.get("items", True), "item")
            lo, hi = int(sch.get("minItems", 0)), sch.get("maxItems")
            name = self.fresh("arr")
            more = f'(ws "," ws {item})'
            if hi is not None and int(hi) == 0:
                body = ""
            elif lo == 0:
                tail = "*" if hi is None else "{0,%d}" % (int(hi) - 1)
                body = f"({item} {more}{tail})?"
            else:
                tail = "{%d,%s}" % (lo - 1, "" if hi is None else int(hi) - 1)
                body = f"{item} {more}{tail}"
            self.rules.append(f'{name} ::= "[" ws {body} ws "]"')
            return name
        if t == "object":
            return self.lower_object(sch)
        return "json-value"

    def lower_object(self, sch: dict) -> str:
        props = sch.get("properties") or {}
        required = set(sch.get("required") or [])
        extra = sch.get("additionalProperties", True)
        name = self.fresh("obj")
        if not props:
            if extra is False:
                self.rules.append(f'{name} ::= "{{" ws "}}"')
                return name
            return "json-object"
        pairs = []
        for key, sub in props.items():
            pairs.append((key in required, f'{_lit(json.dumps(key, ensure_ascii=False))} ws ":" ws {self.lower(sub, "p")}'))
        if extra is not False:
            extra_val = "json-value" if extra is True else self.lower(extra, "x")
            pairs.append((False, f'json-string ws ":" ws {extra_val}'))
            repeat_last = True
        else:
            repeat_last = False
        # members in declaration order; rule k = "what may follow once a member has been written, from member k on"
        n = len(pairs)
        rest_names = [self.fresh("rest") for _ in range(n + 1)]
        self.rules.append(f"{rest_names[n]} ::= \"\"")
        for k in range(n - 1, -1, -1):
            req, pair = pairs[k]
            here = f'ws "," ws {pair}'
            if repeat_last and k == n - 1:
                self.rules.append(f"{rest_names[k]} ::= ({here})*")
            elif req:
                self.rules.append(f"{rest_names[k]} ::= {here} {rest_names[k + 1]}")
            else:
                self.rules.append(f"{rest_names[k]} ::= ({here})? {rest_names[k + 1]}")
        # first member: the first one actually written has no leading comma
        alts = []
        for k in range(n):
            req, pair = pairs[k]
            if repeat_last and k == n - 1:
                alts.append(f"{pair} {rest_names[k]}")
            else:
                alts.append(f"{pair} {rest_names[k + 1]}")
            if req:
                break
        else:
            alts.append('""')                                        # every member optional: {} is fine
        self.rules.append(f'{name} ::= "{{" ws ({" | ".join(alts)}) ws "}}"')
        return name


def schema_to_ebnf(schema: dict) -> str:
    low = _SchemaLowering(schema)
    root = low.lower(schema, "root")
    return f"root ::= ws {root} ws\n" + "\n".join(low.rules) + "\n" + JSON_PRELUDE


# ----------------------------------------------------------------------------- vocabulary bytes
def _gpt2_byte_decoder() -> Dict[str, int]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("\xa1"), ord("\xac") + 1)) + list(range(ord("\xae"), ord("\xff") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {chr(c): b for b, c in zip(bs, cs)}


def token_bytes(tokenizer, vocab_size: int) -> List[bytes]:
    """Byte string of every token id (``b""`` for special / unknown ids, which a grammar never allows)."""
    out = [b""] * vocab_size
    if tokenizer.__class__.__name__ == "ByteTokenizer":
        for b in range(256):
            if 3 + b < vocab_size:
                out[3 + b] = bytes([b])
        return out
    tk = getattr(tokenizer, "tk", None)
    if tk is None:
        return out
    spec = json.loads(tk.to_str())
    blob = json.dumps([spec.get("decoder"), spec.get("pre_tokenizer")])
    byte_level = '"ByteLevel"' in blob
    special = {int(t["id"]) for t in spec.get("added_tokens", []) if t.get("special", True)}
    dec = _gpt2_byte_decoder() if byte_level else None
    for tok, i in tk.get_vocab(with_added_tokens=True).items():
        if i >= vocab_size or i in special:
            continue
        if byte_level:
            try:
                out[i] = bytes(dec[ch] for ch in tok)
            except KeyError:
                out[i] = tok.encode("utf-8")
        elif len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
            out[i] = bytes([int(tok[3:5], 16)])
        else:
            out[i] = tok.replace("▁", " ").encode("utf-8")
    return out


# ----------------------------------------------------------------------------- native binding
_BOUND = False


def _lib():
    global _BOUND
    L = rn.lib()
    if not _BOUND:
        vp = C.c_void_p
        L.atlas_grammar_compile.restype = vp
        L.atlas_grammar_compile.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_int]
        L.atlas_grammar_destroy.argtypes = [vp]
        L.atlas_grammar_num_rules.argtypes = [vp]
        L.atlas_vocab_create.restype = vp
        L.atlas_vocab_create.argtypes = [vp, vp, C.c_int]
        L.atlas_vocab_destroy.argtypes = [vp]
        L.atlas_vocab_num_nodes.argtypes = [vp]
        L.atlas_matcher_create.restype = vp
        L.atlas_matcher_create.argtypes = [vp, vp]
        L.atlas_matcher_destroy.argtypes = [vp]
        for f in ("atlas_matcher_can_end", "atlas_matcher_exhausted", "atlas_matcher_num_stacks"):
            getattr(L, f).argtypes = [vp]
        L.atlas_matcher_mask.argtypes = [vp, vp, C.c_int]
        L.atlas_matcher_accept_bytes.argtypes = [vp, C.c_char_p, C.c_int]
        L.atlas_matcher_rollback.argtypes = [vp, C.c_int]
        _BOUND = True
    return L


class GrammarSyntaxError(ValueError):
    pass


class CompiledGrammar:
    def __init__(self, text: str, root: str = "root"):
        err = C.create_string_buffer(512)
        self._h = _lib().atlas_grammar_compile(text.encode("utf-8"), root.encode(), err, 512)
        if not self._h:
            raise GrammarSyntaxError(err.value.decode("utf-8", "replace"))
        self.text = text

    @property
    def num_rules(self) -> int:
        return _lib().atlas_grammar_num_rules(self._h)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            try:
                _lib().atlas_grammar_destroy(h)
            except Exception:                       # interpreter shutdown
                pass


class Vocabulary:
    """Byte trie of a tokenizer's vocabulary (built once per tokenizer)."""

    def __init__(self, tokens: Sequence[bytes], eos_ids: Sequence[int] = ()):
        self.tokens = list(tokens)
        self.eos_ids = [int(e) for e in eos_ids]
        blob = b"".join(self.tokens)
        offs = [0]
        for t in self.tokens:
            offs.append(offs[-1] + len(t))
        self._blob = C.create_string_buffer(blob, max(1, len(blob)))
        self._offs = (C.c_int64 * len(offs))(*offs)
        self._h = _lib().atlas_vocab_create(C.cast(self._blob, C.c_void_p), C.cast(self._offs, C.c_void_p), len(self.tokens))

    def __len__(self) -> int:
        return len(self.tokens)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            try:
                _lib().atlas_vocab_destroy(h)
            except Exception:                       # interpreter shutdown
                pass


class EbnfMatcher:
    """Per-request matcher with the interface the sampler uses (``token_mask`` / ``accept`` / ``terminated``)."""

    def __init__(self, grammar: CompiledGrammar, vocab: Vocabulary):
        self.grammar, self.vocab = grammar, vocab
        self._h = _lib().atlas_matcher_create(grammar._h, vocab._h)
        self._words = (len(vocab) + 31) // 32
        self._bits = torch.zeros(self._words, dtype=torch.int32)
        self._done = False

    def token_mask(self, vocab: int) -> Optional[torch.Tensor]:
        """Boolean mask over ``vocab`` ids, or None once the sentence has ended."""
        if self._done:
            return None
        n = _lib().atlas_matcher_mask(self._h, self._bits.data_ptr(), self._words)
        if n < 0:
            raise RuntimeError("grammar exceeded the matcher's bounds (left recursion or too many simultaneous parses)")
        idx = torch.arange(min(vocab, len(self.vocab)))
        mask = torch.zeros(vocab, dtype=torch.bool)
        mask[:idx.numel()] = ((self._bits[idx // 32] >> (idx % 32)) & 1).bool()
        if _lib().atlas_matcher_can_end(self._h):
            for e in self.vocab.eos_ids:
                if e < vocab:
                    mask[e] = True
        return mask

    def accept(self, token: int) -> bool:
        token = int(token)
        if token in self.vocab.eos_ids:
            ok = bool(_lib().atlas_matcher_can_end(self._h))
            self._done = self._done or ok
            return ok
        if not (0 <= token < len(self.vocab)) or not self.vocab.tokens[token]:
            return False
        b = self.vocab.tokens[token]
        return bool(_lib().atlas_matcher_accept_bytes(self._h, b, len(b)))

    def rollback(self, n: int) -> int:
        return _lib().atlas_matcher_rollback(self._h, int(n))

    def terminated(self) -> bool:
        return self._done or bool(_lib().atlas_matcher_exhausted(self._h))

    def can_end(self) -> bool:
        return bool(_lib().atlas_matcher_can_end(self._h))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            try:
                _lib().atlas_matcher_destroy(h)
            except Exception:                       # interpreter shutdown
                pass
