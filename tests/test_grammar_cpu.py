"""The engine's own grammar backend: EBNF parsing, JSON-schema lowering, token masks over a byte-level and a BPE
vocabulary, UTF-8 across token boundaries, rollback, bounds on pathological grammars, and the engine glue."""
import json

import pytest
import torch

from atlas_b200.server import ebnf
from atlas_b200.server.grammar import GrammarEngine, GrammarSpec
from atlas_b200.server.tokenizer import ByteTokenizer


def _byte_vocab(extra=()):
    toks = [b""] * 3 + [bytes([b]) for b in range(256)] + list(extra)
    return ebnf.Vocabulary(toks, eos_ids=[2]), toks


def _accepts(grammar, text, vocab):
    m = ebnf.EbnfMatcher(grammar, vocab)
    for b in text.encode():
        if not m.accept(3 + b):
            return False
    return m.can_end()


def test_ebnf_syntax_and_matching():
    v, toks = _byte_vocab([b"yes", b"no", b"no1", b"ye", "é".encode(), "éß".encode(), "éa".encode()])
    g = ebnf.CompiledGrammar('# comment\nroot ::= "yes" | "no" [0-9]+ ws\n     | "é" [^a-z]\nws ::= " "*\n')
    m = ebnf.EbnfMatcher(g, v)
    allowed = {toks[i] for i in m.token_mask(len(toks)).nonzero().flatten().tolist()}
    # single bytes that start a sentence, whole-word tokens, the lead byte of "é"; never an overlong lead byte, never "éa"
    assert allowed == {b"y", b"n", b"\xc3", b"yes", b"no", b"no1", b"ye", "é".encode(), "éß".encode()}
    assert m.accept(3 + 0xC3)
    assert {toks[i] for i in m.token_mask(len(toks)).nonzero().flatten().tolist()} == {b"\xa9"}
    assert m.accept(3 + 0xA9) and not m.accept(3 + ord("q")) and m.accept(3 + ord("Q")) and m.can_end()
    assert m.token_mask(len(toks)).nonzero().flatten().tolist() == [2]           # only EOS can follow
    assert m.accept(2) and m.terminated() and m.token_mask(len(toks)) is None
    for text, ok in [("yes", True), ("no42  ", True), ("no", False), ("maybe", False)]:
        assert _accepts(g, text, v) == ok, text
    # repetition bounds and groups
    g = ebnf.CompiledGrammar('root ::= ("ab" | [x-z]){2,3} "!"?')
    for text, ok in [("abx", True), ("xyz!", True), ("ab", False), ("ababxy", False), ("abab!", True)]:
        assert _accepts(g, text, v) == ok, text
    with pytest.raises(ebnf.GrammarSyntaxError):
        ebnf.CompiledGrammar('root ::= "unterminated')
    with pytest.raises(ebnf.GrammarSyntaxError):
        ebnf.CompiledGrammar("root ::= missing-rule")


def test_rollback_and_left_recursion_is_bounded():
    v, toks = _byte_vocab()
    g = ebnf.CompiledGrammar('root ::= [a-c]+ "."')
    m = ebnf.EbnfMatcher(g, v)
    for ch in b"ab.":
        assert m.accept(3 + ch)
    assert m.can_end() and m.rollback(2) == 2 and not m.can_end()
    assert m.accept(3 + ord("c")) and m.accept(3 + ord(".")) and m.can_end()
    bad = ebnf.EbnfMatcher(ebnf.CompiledGrammar('root ::= root "a" | "b"'), v)
    with pytest.raises(RuntimeError):
        bad.token_mask(len(toks))


def test_json_schema_lowering():
    v, _ = _byte_vocab()
    sch = {"type": "object",
           "properties": {"name": {"const": "get_weather"},
                          "arguments": {"type": "object",
                                        "properties": {"city": {"type": "string"}, "days": {"type": "integer"},
                                                       "unit": {"enum": ["c", "f"]},
                                                       "tags": {"type": "array", "items": {"$ref": "#/$defs/tag"}, "maxItems": 2}},
                                        "required": ["city"], "additionalProperties": False}},
           "required": ["name", "arguments"], "additionalProperties": False,
           "$defs": {"tag": {"type": "string", "maxLength": 3}}}
    g = ebnf.CompiledGrammar(ebnf.schema_to_ebnf(sch))
    good = ['{"name": "get_weather", "arguments": {"city": "Zürich", "days": 3}}',
            '{"name":"get_weather","arguments":{"city":"x","unit":"f","tags":["ab","c"]}}',
            ' {"name":"get_weather","arguments":{"city":"\\u00e9\\n"}} ']
    bad = ['{"name":"get_weather","arguments":{"days":3}}',                       # required member missing
           '{"name":"other","arguments":{"city":"x"}}',                            # const violated
           '{"name":"get_weather","arguments":{"city":"x","zzz":1}}',              # additionalProperties false
           '{"name":"get_weather","arguments":{"city":"x","tags":["abcd"]}}',      # maxLength
           '{"name":"get_weather","arguments":{"city":"x","tags":["a","b","c"]}}',  # maxItems
           '{"name":"get_weather","arguments":{"city":"x","days":1.5}}']
    for t in good:
        json.loads(t)
        assert _accepts(g, t, v), t
    for t in bad:
        assert not _accepts(g, t, v), t
    obj = ebnf.CompiledGrammar(ebnf.JSON_OBJECT_GRAMMAR)
    assert _accepts(obj, '{"a": [1, -2.5e3, {"b": null}], "c": "q\\"x"}', v)
    assert not _accepts(obj, "[1]", v) and not _accepts(obj, '{"a": }', v) and not _accepts(obj, '{"a": 01}', v)
    anyof = ebnf.CompiledGrammar(ebnf.schema_to_ebnf({"anyOf": [{"type": "boolean"}, {"type": ["integer", "null"]}]}))
    assert all(_accepts(anyof, t, v) for t in ("true", "-12", "null")) and not _accepts(anyof, '"x"', v)


def test_bpe_vocabulary_bytes_and_masks():
    """A byte-level BPE tokenizer built in place: token bytes come back through the GPT-2 byte map, merged tokens are
    masked as whole words, special tokens are never allowed."""
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tk = Tokenizer(models.BPE())
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tk.decoder = decoders.ByteLevel()
    corpus = ['{"name": "get_weather", "arguments": {"city": "Zürich"}}', "true false null 12345 yes no"] * 50
    tk.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=["<eos>"],
                                                       initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))

    class Wrap:
        pass
    w = Wrap()
    w.tk, w.vocab_size, w.eos_token_ids = tk, tk.get_vocab_size(), [tk.token_to_id("<eos>")]
    toks = ebnf.token_bytes(w, w.vocab_size)
    assert toks[w.eos_token_ids[0]] == b""
    ids = tk.encode('{"city": "Zürich"}').ids
    assert b"".join(toks[i] for i in ids) == '{"city": "Zürich"}'.encode()
    eng = GrammarEngine(w, w.vocab_size)
    assert eng.backend == "native"
    m = eng.matcher(GrammarSpec(kind="json_schema", schema={"type": "object", "properties": {"city": {"type": "string"}},
                                                            "required": ["city"], "additionalProperties": False}))
    for i in ids:
        mask = m.token_mask(w.vocab_size)
        assert bool(mask[i]), toks[i]
        assert m.accept(i)
    mask = m.token_mask(w.vocab_size)
    assert bool(mask[w.eos_token_ids[0]]) and m.accept(w.eos_token_ids[0]) and m.terminated()
    # a second matcher of the same spec reuses the compiled grammar and the trie
    assert eng.matcher(GrammarSpec(kind="json_schema", schema={"type": "object", "properties": {"city": {"type": "string"}},
                                                               "required": ["city"], "additionalProperties": False})).grammar is m.grammar


def test_engine_glue_with_byte_tokenizer_constrains_sampling():
    tok = ByteTokenizer(1024)
    eng = GrammarEngine(tok, 1024)
    m = eng.matcher(GrammarSpec(kind="ebnf", ebnf='root ::= "A" [0-9]{3}'))
    out = []
    g = torch.Generator().manual_seed(0)
    for _ in range(8):
        mask = m.token_mask(1024)
        if mask is None:
            break
        logits = torch.randn(1024, generator=g)
        logits[~mask] = float("-inf")
        t = int(logits.argmax())
        assert m.accept(t)
        if t == 2:
            break
        out.append(t)
    text = tok.decode(out)
    assert len(text) == 4 and text[0] == "A" and text[1:].isdigit()
