"""Command line and boot path on CPU: recipes layering, ``doctor``, and a real ``serve`` process — single rank and two
gloo ranks (rank 0 serves HTTP, rank 1 follows over the control plane) — answering an OpenAI chat request."""
import json
import os
import socket
import subprocess
import sys
import time

import pytest

from atlas_b200 import cli, recipes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_recipe_layering_and_validation(tmp_path):
    y = tmp_path / "fam" / "demo.yaml"
    y.parent.mkdir()
    y.write_text("model: preset:tiny-dense\nmin_nodes: 2\ndefaults:\n  tp_size: 2\n  max_num_seqs: 4\n  speculative: true\n"
                 "env:\n  ATLAS_GEMM_SPLITS: 2\n")
    r = recipes.load(str(y))
    assert r.id == "fam/demo" and r.min_ranks == 2
    args, rec = cli.resolve_serve_args(["--recipe", str(y), "--max-num-seqs", "9"])
    assert args.model == "preset:tiny-dense" and args.tp_size == 2 and args.speculative
    assert args.max_num_seqs == 9                     # an explicit flag beats the recipe
    env = {}
    assert rec.export_env(env) == {"ATLAS_GEMM_SPLITS": "2"} and rec.export_env(env) == {}
    with pytest.raises(recipes.RecipeError):
        recipes.from_dict({"model": "m", "defaults": {"bogus": 1}})
    with pytest.raises(recipes.RecipeError):
        recipes.from_dict({"model": "m", "defaults": {"tp_size": 4}})      # needs 4 ranks, min_ranks says 1
    for rid in recipes.BUILTIN:
        assert recipes.builtin(rid).argv()[0].startswith("preset:")


def test_doctor_reports():
    rep = cli.doctor_report()
    names = {c["name"] for c in rep["checks"]}
    assert {"kernel library", "gpu", "peer access", "python deps"} <= names
    assert "hardware" in rep


def _wait_http(port, procs, timeout=120.0):
    import urllib.request
    t0 = time.time()
    while time.time() - t0 < timeout:
        for p in procs:
            if p.poll() is not None:
                raise AssertionError(f"server process exited early with {p.returncode}: {p.stderr.read()[-2000:] if p.stderr else ''}")
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1.0) as r:
                if r.status == 200:
                    return
        except Exception:
            time.sleep(0.3)
    raise AssertionError("server did not come up")


def _chat(port, content="hello", max_tokens=8):
    import urllib.request
    body = json.dumps({"model": "x", "messages": [{"role": "user", "content": content}], "max_tokens": max_tokens,
                       "temperature": 0}).encode()
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body,
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=60) as r:
        return json.loads(r.read())


def _spawn(argv, env_extra):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", **env_extra)
    return subprocess.Popen([sys.executable, "-m", "atlas_b200", "serve"] + argv, cwd=ROOT, env=env,
                            stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, text=True)


def _stop(procs):
    for p in procs:
        if p.poll() is None:
            p.terminate()
    for p in procs:
        try:
            p.wait(timeout=15)
        except subprocess.TimeoutExpired:
            p.kill()


def test_serve_single_rank():
    port = _free_port()
    procs = [_spawn(["preset:tiny-dense", "--port", str(port), "--bind", "127.0.0.1", "--num-kv-blocks", "64",
                     "--max-seq-len", "256"], {})]
    try:
        _wait_http(port, procs)
        out = _chat(port)
        assert out["usage"]["completion_tokens"] == 8 and out["choices"][0]["finish_reason"] == "length"
    finally:
        _stop(procs)


def test_serve_two_ranks_gloo():
    port, mport = _free_port(), _free_port()
    common = ["preset:tiny-dense", "--port", str(port), "--bind", "127.0.0.1", "--num-kv-blocks", "64", "--max-seq-len", "256",
              "--world-size", "2", "--tp-size", "2", "--master-addr", "127.0.0.1", "--master-port", str(mport)]
    procs = [_spawn(common + ["--rank", str(r)], {"ATLAS_CONTROL_TIMEOUT_S": "20"}) for r in range(2)]
    try:
        _wait_http(port, procs)
        a = _chat(port, "first")
        b = _chat(port, "first")
        assert a["usage"]["completion_tokens"] == 8
        assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
        # the single-rank engine gives the same greedy text (TP sharding is exact in fp32 up to summation order)
        assert procs[1].poll() is None
    finally:
        _stop(procs)


def test_recipe_sync_from_an_index(tmp_path, monkeypatch, capsys):
    """``recipes --sync``: an index with checksums, fetched over file://; a synced recipe resolves by id; a checksum
    mismatch or an invalid recipe writes nothing (the earlier copy stays)."""
    import hashlib
    import json
    src, dest = tmp_path / "remote", tmp_path / "local"
    (src / "fam").mkdir(parents=True)
    good = b"model: preset:llama3-8b\ndescription: synced\ndefaults:\n  max_num_seqs: 32\n  mtp_vocab: 4096\n"
    (src / "fam" / "a.yaml").write_bytes(good)
    index = {"recipes": [{"id": "fam/a", "url": "fam/a.yaml", "sha256": hashlib.sha256(good).hexdigest()}]}
    (src / "index.json").write_text(json.dumps(index))
    url = (src / "index.json").as_uri()
    assert cli.main(["recipes", "--sync", url, "--dest", str(dest)]) == 0
    assert capsys.readouterr().out.strip() == "fam/a"
    monkeypatch.setenv("ATLAS_RECIPES_DIR", str(dest))
    r = recipes.resolve("fam/a")
    assert r.description == "synced" and "--mtp-vocab" in r.argv() and "32" in r.argv()
    # a tampered file: nothing is replaced
    (src / "fam" / "a.yaml").write_bytes(good.replace(b"32", b"64"))
    with pytest.raises(recipes.RecipeError, match="checksum"):
        recipes.sync(url, str(dest))
    assert "32" in recipes.resolve("fam/a").argv()
    # an invalid recipe (unknown key) and a path-escaping id are refused before anything is written
    bad = b"model: m\ndefaults:\n  bogus: 1\n"
    (src / "fam" / "b.yaml").write_bytes(bad)
    (src / "index.json").write_text(json.dumps({"recipes": [{"id": "fam/b", "url": "fam/b.yaml"}]}))
    with pytest.raises(recipes.RecipeError):
        recipes.sync(url, str(dest))
    assert not (dest / "fam" / "b.yaml").exists()
    (src / "index.json").write_text(json.dumps({"recipes": [{"id": "../x", "url": "fam/a.yaml"}]}))
    with pytest.raises(recipes.RecipeError, match="bad recipe id"):
        recipes.sync(url, str(dest))
