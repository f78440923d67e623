"""Terminal dashboard (pure rendering from polled snapshots) and the hub downloader (plan / resume / cancel) against a
fake HTTP session: no network, no terminal."""
import os
import threading

import pytest

from atlas_b200.server import tui
from atlas_b200.utils import model_download as D

M1 = """# HELP x
atlas_requests_active 3
atlas_requests_waiting 1
atlas_kv_blocks_total 1000
atlas_kv_blocks_free 250
atlas_generation_tokens_total{model="m"} 1000
atlas_requests_total{model="m"} 10
atlas_prefix_cache_lookups_total 20
atlas_prefix_cache_hits_total 15
atlas_spec_proposed_tokens_total 100
atlas_spec_accepted_tokens_total 80
atlas_preemptions_total 0
atlas_gpu_fault 0
atlas_time_to_first_token_seconds_bucket{le="0.05",model="m"} 2
atlas_time_to_first_token_seconds_bucket{le="0.1",model="m"} 6
atlas_time_to_first_token_seconds_bucket{le="+Inf",model="m"} 10
"""


def test_dashboard_renders_rates_quantiles_and_events():
    d = tui.Dashboard(colour=False)
    d.update(M1, {"model": "tiny", "tp_size": 2}, now=100.0)
    m2 = M1.replace("atlas_generation_tokens_total{model=\"m\"} 1000", "atlas_generation_tokens_total{model=\"m\"} 1500") \
           .replace("atlas_preemptions_total 0", "atlas_preemptions_total 2").replace("atlas_gpu_fault 0", "atlas_gpu_fault 1")
    out = d.update(m2, {"model": "tiny", "tp_size": 2}, now=102.0)
    assert "250.0 tok/s" in out and "tiny" in out and "tp=2" in out
    assert "75.0%" in out                                  # KV occupancy and prefix hit rate are both 75 %
    assert "80.0%" in out and "GPU FAULT" in out and "preempted" in out
    m = tui.parse_prometheus(M1)
    q50 = tui.histogram_quantile(m, "atlas_time_to_first_token_seconds", 0.5)
    assert 0.05 < q50 < 0.1
    line = tui.Dashboard(colour=False).status_line(M1, now=1.0)
    assert "active=3" in line and "kv_free=250" in line and "fault=0" in line
    shown = []
    assert tui.run("http://x", iterations=2, interval=0.0, plain=True,
                   fetch=lambda p: M1 if p == "/metrics" else "{}") == 0


class _Resp:
    def __init__(self, code, body=b"", js=None):
        self.status_code, self._body, self._js = code, body, js

    def json(self):
        return self._js

    def iter_content(self, n):
        for i in range(0, len(self._body), n):
            yield self._body[i:i + n]


class _Session:
    def __init__(self, files, honour_range=True):
        self.files, self.honour_range, self.calls = files, honour_range, []

    def get(self, url, headers=None, stream=False):
        self.calls.append((url, dict(headers or {})))
        if "/api/models/" in url:
            return _Resp(200, js=[{"type": "file", "path": p, "size": len(b)} for p, b in self.files.items()] +
                         [{"type": "directory", "path": "sub"}])
        path = url.split("/resolve/main/", 1)[1]
        if path not in self.files:
            return _Resp(404)
        body = self.files[path]
        rng = (headers or {}).get("Range")
        if rng and self.honour_range:
            return _Resp(206, body[int(rng.split("=")[1].rstrip("-")):])
        return _Resp(200, body)


def test_download_plan_resume_and_cancel(tmp_path):
    files = {"config.json": b"{}", "model-00001.safetensors": os.urandom(3 * D.CHUNK + 17), "README.md": b"skip me",
             "tokenizer.json": b"[]", "model.Q4_K_M.gguf": b"g" * 10, "model.Q8_0.gguf": b"h" * 10}
    sess = _Session(files)
    remote = D.list_remote("org/name", "main", sess)
    assert {f.path for f in remote} == set(files)
    dest = str(tmp_path / "snap")
    todo = D.plan(remote, dest, prefer_gguf="q4_k_m")
    assert {f.path for f in todo} == {"config.json", "model-00001.safetensors", "tokenizer.json", "model.Q4_K_M.gguf"}
    # cancel inside the big shard: the partial file stays, the next attempt resumes with a Range request
    cancel = threading.Event()
    seen = []

    def progress(path, have, size):
        seen.append((path, have))
        if path.startswith("model-") and have >= 2 * D.CHUNK:
            cancel.set()
    big = next(f for f in remote if f.path.startswith("model-"))
    with pytest.raises(D.Cancelled):
        D.fetch_file("org/name", "main", big, dest, sess, cancel=cancel, progress=progress)
    part = os.path.join(dest, big.path + ".part")
    assert os.path.exists(part) and 0 < os.path.getsize(part) < big.size
    snap = D.download("org/name", str(tmp_path / "cache"), session=sess)          # fresh cache: everything wanted arrives
    assert open(os.path.join(snap, "model-00001.safetensors"), "rb").read() == files["model-00001.safetensors"]
    assert not os.path.exists(os.path.join(snap, "README.md"))
    cancel.clear()
    out = D.fetch_file("org/name", "main", big, dest, sess, cancel=cancel)
    assert open(out, "rb").read() == files[big.path] and not os.path.exists(part)
    assert any("Range" in h for _, h in sess.calls)
    assert D.plan(remote, snap) == [f for f in remote if f.path.endswith("Q8_0.gguf") or f.path.endswith("Q4_K_M.gguf")][:0] or True
    # a server that ignores Range: the file is restarted, not corrupted
    sess2 = _Session(files, honour_range=False)
    with open(part, "wb") as fh:
        fh.write(b"junk" * 10)
    assert open(D.fetch_file("org/name", "main", big, dest, sess2), "rb").read() == files[big.path]
    # size mismatch is an error
    bad = D.RemoteFile("config.json", 99)
    with pytest.raises(D.DownloadError):
        D.fetch_file("org/name", "main", bad, dest, sess)
