"""HTTP API surface on CPU (FastAPI test client over a tiny random-init model with the byte tokenizer): OpenAI chat /
completions (streaming and not), Anthropic messages, Responses + Conversations, llama.cpp dialect, ops routes, stubs,
auth, rate limiting and the fault latch."""
import json

import pytest
from fastapi.testclient import TestClient

from atlas_b200.config import EngineConfig, tiny_dense
from atlas_b200.engine import LLMEngine
from atlas_b200.models import build_model
from atlas_b200.server.app import ServerState, create_app
from atlas_b200.server.engine_async import AsyncEngine
from atlas_b200.server.tokenizer import load_tokenizer
from atlas_b200.utils.fault import FAULT_LATCH


def _client(args=None):
    eng = LLMEngine(build_model(tiny_dense()).init_random(0), EngineConfig(num_kv_blocks=256, max_num_seqs=8, max_seq_len=1024))
    aeng = AsyncEngine(eng)
    aeng.start()
    state = ServerState(aeng, load_tokenizer(None, 1024), "tiny", args or {})
    return TestClient(create_app(state)), aeng, state


@pytest.fixture(scope="module")
def ctx():
    c, aeng, state = _client()
    yield c, state
    aeng.shutdown(drain=False)


def _sse(resp):
    out = []
    for line in resp.iter_lines():
        if line.startswith("data:"):
            d = line[5:].strip()
            if d != "[DONE]":
                out.append(json.loads(d))
    return out


def test_chat_completion_and_usage(ctx):
    c, _ = ctx
    r = c.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "hi"}],
                                              "max_tokens": 6, "temperature": 0, "logprobs": True, "top_logprobs": 2})
    assert r.status_code == 200, r.text
    j = r.json()
    ch = j["choices"][0]
    assert j["object"] == "chat.completion" and ch["finish_reason"] == "length"
    assert j["usage"]["completion_tokens"] == 6 and j["usage"]["prompt_tokens"] > 0
    assert "cached_tokens" in j["usage"]["prompt_tokens_details"]
    assert len(ch["logprobs"]["content"]) == 6 and len(ch["logprobs"]["content"][0]["top_logprobs"]) == 2
    # deterministic at temperature 0, and the second call hits the prefix cache
    r2 = c.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "hi"}],
                                               "max_tokens": 6, "temperature": 0}).json()
    assert r2["choices"][0]["message"]["content"] == ch["message"]["content"]


def test_chat_stream_matches_blocking(ctx):
    c, _ = ctx
    body = {"model": "tiny", "messages": [{"role": "user", "content": "stream me"}], "max_tokens": 8, "temperature": 0}
    full = c.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"]
    with c.stream("POST", "/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}}) as r:
        evs = _sse(r)
    text = "".join((e["choices"][0]["delta"].get("content") or "") for e in evs if e.get("choices"))
    assert text == full
    assert any(e.get("usage") for e in evs)
    assert [e for e in evs if e.get("choices") and e["choices"][0].get("finish_reason")][-1]["choices"][0]["finish_reason"] == "length"


def test_completions_with_token_ids_and_stop(ctx):
    c, _ = ctx
    r = c.post("/v1/completions", json={"model": "tiny", "prompt": [5, 6, 7, 8, 9], "max_tokens": 5, "temperature": 0,
                                         "return_token_ids": True, "ignore_eos": True})
    assert r.status_code == 200, r.text
    ch = r.json()["choices"][0]
    assert len(ch["token_ids"]) == 5
    first = ch["token_ids"][0]
    r = c.post("/v1/completions", json={"model": "tiny", "prompt": [5, 6, 7, 8, 9], "max_tokens": 5, "temperature": 0,
                                         "stop_token_ids": [ch["token_ids"][1]], "return_token_ids": True})
    ch2 = r.json()["choices"][0]
    assert ch2["finish_reason"] == "stop" and ch2["token_ids"][0] == first and len(ch2["token_ids"]) <= 2
    with c.stream("POST", "/v1/completions", json={"model": "tiny", "prompt": [5, 6, 7, 8, 9], "max_tokens": 5, "temperature": 0,
                                                    "stream": True, "return_token_ids": True, "ignore_eos": True}) as s:
        ids = [t for e in _sse(s) for t in (e["choices"][0].get("token_ids") or [])]
    assert ids == ch["token_ids"]


def test_validation_errors(ctx):
    c, _ = ctx
    assert c.post("/v1/chat/completions", json={"model": "tiny", "messages": []}).status_code == 400
    assert c.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "x"}],
                                                 "temperature": -1}).status_code == 400
    r = c.post("/v1/completions", json={"model": "tiny", "prompt": [1] * 5000, "max_tokens": 4})
    assert r.status_code == 400 and "error" in r.json()


def test_json_mode_emits_valid_json(ctx):
    c, state = ctx
    if state.grammar is None:
        pytest.skip("no grammar backend")
    r = c.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "json please"}],
                                              "max_tokens": 48, "temperature": 0, "response_format": {"type": "json_object"}})
    assert r.status_code == 200, r.text
    txt = r.json()["choices"][0]["message"]["content"]
    if r.json()["choices"][0]["finish_reason"] == "stop":
        json.loads(txt)
    else:                                   # cut by max_tokens: still a prefix of a JSON document
        assert txt.lstrip()[:1] in ("{", "[", "")


def test_anthropic_messages(ctx):
    c, _ = ctx
    r = c.post("/v1/messages", json={"model": "tiny", "max_tokens": 5, "messages": [{"role": "user", "content": "hello"}],
                                      "system": "be brief", "temperature": 0})
    assert r.status_code == 200, r.text
    j = r.json()
    assert j["type"] == "message" and j["role"] == "assistant" and j["stop_reason"] == "max_tokens"
    assert j["usage"]["output_tokens"] == 5 and all(b["type"] == "text" for b in j["content"])
    n = c.post("/v1/messages/count_tokens", json={"model": "tiny", "messages": [{"role": "user", "content": "hello"}]}).json()
    assert n["input_tokens"] > 0
    with c.stream("POST", "/v1/messages", json={"model": "tiny", "max_tokens": 5, "stream": True, "temperature": 0,
                                                 "messages": [{"role": "user", "content": "hello"}]}) as s:
        types = [e["type"] for e in _sse(s)]
    # (a random-init model may emit bytes that never complete a UTF-8 character, so text deltas are optional)
    assert types[0] == "message_start" and "message_delta" in types and types[-1] == "message_stop"


def test_responses_and_conversations(ctx):
    c, _ = ctx
    r = c.post("/v1/responses", json={"model": "tiny", "input": "say something", "max_output_tokens": 5, "temperature": 0})
    assert r.status_code == 200, r.text
    j = r.json()
    assert j["object"] == "response" and j["status"] in ("completed", "incomplete")
    rid = j["id"]
    assert c.get(f"/v1/responses/{rid}").json()["id"] == rid
    assert c.get(f"/v1/responses/{rid}/input_items").status_code == 200
    r2 = c.post("/v1/responses", json={"model": "tiny", "input": "and more", "previous_response_id": rid, "max_output_tokens": 4})
    assert r2.status_code == 200 and r2.json()["usage"]["input_tokens"] > j["usage"]["input_tokens"]
    assert c.delete(f"/v1/responses/{rid}").status_code == 200
    assert c.get(f"/v1/responses/{rid}").status_code == 404
    conv = c.post("/v1/conversations", json={"metadata": {"k": "v"}}).json()
    cid = conv["id"]
    c.post(f"/v1/conversations/{cid}/items", json={"items": [{"type": "message", "role": "user", "content": "hi"}]})
    items = c.get(f"/v1/conversations/{cid}/items").json()["data"]
    assert len(items) == 1
    assert c.delete(f"/v1/conversations/{cid}/items/{items[0]['id']}").status_code == 200
    assert c.delete(f"/v1/conversations/{cid}").status_code == 200


def test_models_tokenize_llamacpp_and_ops(ctx):
    c, _ = ctx
    models = c.get("/v1/models").json()["data"]
    assert models[0]["id"] == "tiny" and c.get("/v1/models/tiny").status_code == 200
    toks = c.post("/tokenize", json={"content": "abc"}).json()["tokens"]
    assert c.post("/detokenize", json={"tokens": toks}).json()["content"] == "abc"
    r = c.post("/completion", json={"prompt": "abc", "n_predict": 4, "temperature": 0})
    assert r.status_code == 200 and r.json()["tokens_predicted"] == 4
    assert "default_generation_settings" in c.get("/props").json()
    assert c.post("/apply-template", json={"messages": [{"role": "user", "content": "x"}]}).status_code == 200
    assert c.post("/embedding", json={"content": "x"}).status_code in (400, 501)
    assert c.get("/health").json()["status"] == "ok" and c.get("/health/live").status_code == 200
    m = c.get("/metrics").text
    assert "atlas_requests_total" in m and "atlas_generation_tokens_total" in m
    sc = c.get("/serve-config").json()
    assert sc["engine"]["block_size"] == 16 and "scheduler" in sc and "trace" in sc
    assert "gpus" in c.get("/hardware").json() or "hardware" in c.get("/hardware").json() or c.get("/hardware").status_code == 200
    for stub in ("/v1/embeddings", "/v1/batches", "/v1/files", "/v1/audio/speech", "/v1/images/generations", "/v1/moderations"):
        r = c.post(stub, json={})
        assert r.status_code == 501 and r.json()["error"]["type"]


def test_auth_and_rate_limit():
    c, aeng, _ = _client({"api_keys": ["sekret"], "rate_limit_rpm": 2})
    try:
        body = {"model": "tiny", "messages": [{"role": "user", "content": "x"}], "max_tokens": 2}
        assert c.post("/v1/chat/completions", json=body).status_code == 401
        assert c.get("/health").status_code == 200              # probes stay open
        h = {"Authorization": "Bearer sekret"}
        codes = [c.post("/v1/chat/completions", json=body, headers=h).status_code for _ in range(4)]
        assert codes[0] == 200 and 429 in codes
    finally:
        aeng.shutdown(drain=False)


def test_fault_latch_turns_service_unavailable():
    c, aeng, _ = _client()
    try:
        FAULT_LATCH.reset_for_tests()
        FAULT_LATCH.trip("test: context lost")
        r = c.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "x"}], "max_tokens": 2})
        assert r.status_code == 503
        h = c.get("/health")
        assert h.status_code == 503 and "context lost" in json.dumps(h.json())
    finally:
        FAULT_LATCH.reset_for_tests()
        aeng.shutdown(drain=False)


def test_over_long_chat_is_compacted_or_rejected():
    """Without compaction an over-long conversation is a 400 (context_length_exceeded); with it the old turns are
    elided / dropped and the request is served."""
    msgs = [{"role": "system", "content": "be brief"}]
    for i in range(12):
        msgs.append({"role": "user", "content": f"question {i} " + "lorem ipsum " * 8})
        msgs.append({"role": "assistant", "content": f"answer {i} " + "dolor sit " * 8})
    msgs.append({"role": "user", "content": "final?"})
    body = {"model": "tiny", "messages": msgs, "max_tokens": 4}
    c, aeng, _ = _client()
    try:
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 400 and r.json()["error"]["code"] == "context_length_exceeded"
    finally:
        aeng.shutdown(drain=False)
    c, aeng, state = _client({"context_compaction": True, "compaction_reserve_tokens": 64})
    try:
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        assert r.json()["usage"]["prompt_tokens"] <= 1024 - 64
    finally:
        aeng.shutdown(drain=False)


def test_image_parts_are_decoded_patchified_and_placeholders_widened():
    import base64
    import io

    import numpy as np
    from PIL import Image

    from atlas_b200.models.vision import VisionConfig, mrope_positions
    from atlas_b200.server.multimodal import ImageError, expand_placeholders, extract_images, prepare_images
    rng = np.random.default_rng(0)
    buf = io.BytesIO()
    Image.fromarray((rng.random((37, 50, 3)) * 255).astype(np.uint8)).save(buf, format="PNG")
    b64 = base64.b64encode(buf.getvalue()).decode()
    msgs = [{"role": "user", "content": [{"type": "text", "text": "look"},
                                         {"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64}},
                                         {"type": "image", "source": {"type": "base64", "media_type": "image/png", "data": b64}}]}]
    imgs = extract_images(msgs)
    assert len(imgs) == 2 and imgs[0].shape == (37, 50, 3) and (imgs[0] == imgs[1]).all()
    cfg = VisionConfig(patch_size=4, spatial_merge_size=2, temporal_patch_size=2, hidden_size=64, depth=1, num_heads=4,
                       intermediate_size=128, out_hidden_size=256, num_position_embeddings=64)
    toks, pairs = prepare_images(msgs, [1, 500, 2, 500, 3], cfg, 500)
    (p0, g0), (p1, g1) = pairs
    assert g0 == (1, 10, 12) and p0.shape == (120, 3 * 2 * 4 * 4) and toks.count(500) == 2 * 30
    pos, delta = mrope_positions(toks, 500, [g0, g1], 2)
    assert pos.shape == (3, len(toks)) and delta == (1 + 6 + 1 + 6 + 1) - len(toks)
    assert pos[:, 0].tolist() == [0, 0, 0] and pos[1, 1:31].max() == 1 + 4 and pos[2, 1:31].max() == 1 + 5
    with pytest.raises(ImageError):
        expand_placeholders([1, 2], 500, [4])
    with pytest.raises(ImageError):
        extract_images([{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "https://example.com/x.png"}}]}])


def test_output_sanitizer_rules():
    """Streaming content filter (markers split across chunks, suppressed envelopes, held tails), the complete-string
    scrubbers and the per-response guards."""
    from atlas_b200.server.sanitizer import (ContentSanitizer, StreamGuards, marker_prefix_hold, scrub_think_markers,
                                             scrub_tool_tags, strip_orphan_tool_markup, DEFAULT_MARKERS)
    s = ContentSanitizer()
    chunks = ["Hello <to", 'ol_call>{"name": 1}</tool', "_call> world </thi", "nk>  done <func", "tion=foo> x </function> y <"]
    shown = [s.feed(c) for c in chunks]
    assert shown[0] == "Hello " and "".join(shown) + s.flush() == "Hello  world done  x  y "
    # every prefix of the stream: nothing that later turns out to be markup is ever shown
    text = 'ok <tool_call>{"a": 1}</tool_call> fine'
    for cut in range(1, len(text)):
        f = ContentSanitizer()
        assert f.feed(text[:cut]) + f.feed(text[cut:]) + f.flush() == "ok  fine", cut
    f = ContentSanitizer()
    assert f.feed("text <tool_call>{never closed") == "text " and f.flush() == "" and f.dropped > 0
    f = ContentSanitizer()
    assert f.feed("a < b and c <") == "a < b and c " and f.flush() == ""        # a lone "<" could start a tag: held, then dropped
    f = ContentSanitizer()
    assert f.feed("1 <= 2") + f.flush() == "1 <= 2"
    assert marker_prefix_hold("abc</tool", DEFAULT_MARKERS.all) == 6 and marker_prefix_hold("abc", DEFAULT_MARKERS.all) == 0
    assert scrub_tool_tags("a<function=x>b</function>c<parameter=q") == "abc"
    assert scrub_think_markers("391.</think>  17 x 23") == "391.17 x 23"
    assert strip_orphan_tool_markup('the story."<tool_call>catch({})') == 'the story."'
    g = StreamGuards()
    line = "The quick brown fox jumps.\n"
    assert not any(g.on_text(line) for _ in range(3)) and g.on_text(line) and g.tripped == "repeated_line"
    g = StreamGuards()
    assert not any(g.on_tool_call() for _ in range(12)) and g.on_tool_call() and g.tripped == "tool_call_cap"
    g = StreamGuards()
    assert not g.on_text("a perfectly ordinary paragraph without any repetition in it at all, just prose.")
    assert g.on_text(" and again the same thirty-something characters" * 4) and g.tripped == "repeated_phrase"


def test_lora_control_routes_load_an_adapter_and_requests_use_it(tmp_path):
    """``/v1/lora/load`` reads a PEFT directory through the engine (every rank would), ``/v1/lora/active`` lists it, a
    request can name it, and a request without a name runs on the active adapter."""
    from tests.test_lora_cpu import _write_adapter
    c, aeng, state = _client()
    try:
        path = _write_adapter(str(tmp_path / "ad"), tiny_dense())
        assert c.post("/v1/lora/load", json={"name": "nope"}).status_code == 404
        r = c.post("/v1/lora/load", json={"name": "ad", "path": path, "activate": False})
        assert r.status_code == 200 and r.json() == {"active": None, "loaded": ["ad"]}
        body = {"model": "tiny", "prompt": "hello there", "max_tokens": 8, "temperature": 0}
        base = c.post("/v1/completions", json=body).json()["choices"][0]["text"]
        with_ad = c.post("/v1/completions", json=dict(body, adapter="ad")).json()["choices"][0]["text"]
        assert with_ad != base
        assert c.post("/v1/completions", json=dict(body, adapter="missing")).status_code >= 400
        assert c.post("/v1/lora/load", json={"name": "ad"}).json()["active"] == "ad"      # already resident: activate it
        assert c.get("/v1/lora/active").json() == {"active": "ad", "loaded": ["ad"]}
        assert c.post("/v1/completions", json=body).json()["choices"][0]["text"] == with_ad
    finally:
        aeng.shutdown(drain=False)


def test_confidence_summary_extension(ctx):
    """``atlas_confidence``: the three figures over the first tokens, computed from internally requested top-2
    log-probabilities that are not returned unless the client asked for them; the figures feed ``/metrics``."""
    from atlas_b200.server.confidence import confidence_summary
    import math
    ents = [{"logprob": math.log(0.9), "top": [(1, math.log(0.9)), (2, math.log(0.05))]},
            {"logprob": math.log(0.4), "top": [(3, math.log(0.4)), (4, math.log(0.35))]}]
    s = confidence_summary(ents)
    assert s["tokens"] == 2 and abs(s["mean_top1"] - 0.65) < 1e-9 and abs(s["min_margin"] - 0.05) < 1e-9 and s["low_frac"] == 0.5
    assert confidence_summary(ents, k=1)["low_frac"] == 0.0 and confidence_summary(None) is None
    c, state = ctx
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0}
    plain = c.post("/v1/chat/completions", json=body).json()["choices"][0]
    assert "atlas_confidence" not in plain
    r = c.post("/v1/chat/completions", json=dict(body, atlas_confidence=True)).json()["choices"][0]
    conf = r["atlas_confidence"]
    assert conf["tokens"] == 6 and 0 < conf["mean_top1"] <= 1 and 0 <= conf["min_margin"] <= 1 and 0 <= conf["low_frac"] <= 1
    assert r["logprobs"] is None and r["message"]["content"] == plain["message"]["content"]
    both = c.post("/v1/chat/completions", json=dict(body, atlas_confidence=True, logprobs=True, top_logprobs=3)).json()["choices"][0]
    assert len(both["logprobs"]["content"]) == 6 and both["atlas_confidence"]["tokens"] == 6
    assert "atlas_confidence_mean_top1_count 2.0" in c.get("/metrics").text


def test_evidence_fingerprints_blocking_and_streaming(ctx):
    """``atlas_evidence``: the token and output fingerprints follow their definition, are equal for two identical greedy
    requests (blocking and streamed alike, whatever the chunking), differ for another prompt, and combine over choices."""
    import hashlib
    import struct
    from atlas_b200.server.evidence import ChoiceEvidence, combine
    c, state = ctx
    body = {"model": "tiny", "messages": [{"role": "user", "content": "fingerprint me"}], "max_tokens": 8, "temperature": 0,
            "atlas_evidence": True, "return_token_ids": True}
    a = c.post("/v1/chat/completions", json=body).json()
    b = c.post("/v1/chat/completions", json=body).json()
    ua, ub = a["usage"], b["usage"]
    assert ua["atlas_token_sha"] == ub["atlas_token_sha"] and ua["atlas_output_sha256"] == ub["atlas_output_sha256"]
    content = a["choices"][0]["message"]["content"] or ""
    want_out = hashlib.sha256(hashlib.sha256(content.encode()).digest() + hashlib.sha256(b"").digest()).hexdigest()
    assert ua["atlas_output_sha256"] == want_out
    other = c.post("/v1/chat/completions", json=dict(body, messages=[{"role": "user", "content": "something else"}])).json()
    assert other["usage"]["atlas_token_sha"] != ua["atlas_token_sha"]
    assert "atlas_token_sha" not in c.post("/v1/chat/completions", json={k: v for k, v in body.items() if k != "atlas_evidence"}).json()["usage"]
    with c.stream("POST", "/v1/chat/completions", json=dict(body, stream=True)) as r:
        chunks = _sse(r)
    us = [ch["usage"] for ch in chunks if ch.get("usage")][-1]
    assert us["atlas_token_sha"] == ua["atlas_token_sha"] and us["atlas_output_sha256"] == ua["atlas_output_sha256"]
    # the definition itself: stop token dropped only on a "stop" finish, several choices hash their digests
    ev = ChoiceEvidence(stop_ids=[2])
    ev.add([5, 6], "ab")
    ev.add([2], "c", "why")
    assert ev.token_digest("stop") == hashlib.sha256(struct.pack("<2I", 5, 6)).digest()
    assert ev.token_digest("length") == hashlib.sha256(struct.pack("<3I", 5, 6, 2)).digest()
    assert ev.output_digest() == hashlib.sha256(hashlib.sha256(b"abc").digest() + hashlib.sha256(b"why").digest()).digest()
    d1, d2 = ev.token_digest("stop"), ev.token_digest("length")
    assert combine([d1]) == d1.hex() and combine([d1, d2]) == hashlib.sha256(d1 + d2).hexdigest()
