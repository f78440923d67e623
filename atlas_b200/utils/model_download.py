"""Hub downloader: lists a repository's files, decides what to fetch, and fetches with resume and cancellation.

Three steps kept apart so that each is testable without a network:

* :func:`plan`      pure: remote file list + what is already on disk -> the files to fetch (weights of the wanted
  format, tokenizer and config files; files already complete are skipped, partial ``.part`` files are resumed).
* :func:`fetch_file`  one file over HTTP(S) with a ``Range`` request when a partial file exists, written in 1 MiB
  chunks (the cancellation flag is checked once per chunk), size-checked, then renamed into place.
* :func:`download`  the loop, with a progress callback; lays the files out like the hub cache
  (``models--org--name/snapshots/<revision>/``) so that the resolver finds them offline afterwards.

The HTTP client is injected (``session.get(url, headers=..., stream=True)``; ``requests`` by default).  Nothing in the
engine calls this implicitly: serving never touches the network unless ``atlas_b200 download`` is run.

Reference parity: ``crates/spark-server/src/model_download/{plan,hf,stale}.rs`` (plan / transport split, byte-level
progress, resume from a partial file, cancellation inside a shard).
"""
from __future__ import annotations

import fnmatch
import os
import threading
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

HOST = "https://huggingface.co"
CHUNK = 1 << 20
WANTED = ("*.safetensors", "*.safetensors.index.json", "config.json", "generation_config.json", "tokenizer.json",
          "tokenizer_config.json", "tokenizer.model", "special_tokens_map.json", "chat_template.jinja", "hf_quant_config.json",
          "vocab.json", "merges.txt", "*.gguf")


class DownloadError(RuntimeError):
    pass


class Cancelled(DownloadError):
    pass


@dataclass
class RemoteFile:
    path: str
    size: int
    sha256: Optional[str] = None


def snapshot_dir(cache_root: str, repo_id: str, revision: str) -> str:
    return os.path.join(cache_root, "models--" + repo_id.replace("/", "--"), "snapshots", revision)


def list_remote(repo_id: str, revision: str = "main", session=None, token: Optional[str] = None) -> List[RemoteFile]:
    session = session or _default_session()
    url = f"{HOST}/api/models/{repo_id}/tree/{revision}?recursive=1"
    r = session.get(url, headers=_auth(token))
    if getattr(r, "status_code", 200) != 200:
        raise DownloadError(f"{repo_id}@{revision}: listing failed with HTTP {r.status_code}")
    out = []
    for e in r.json():
        if e.get("type") == "file":
            lfs = e.get("lfs") or {}
            out.append(RemoteFile(e["path"], int(lfs.get("size", e.get("size", 0))), lfs.get("oid")))
    return out


def plan(remote: Sequence[RemoteFile], dest: str, patterns: Sequence[str] = WANTED, prefer_gguf: Optional[str] = None) -> List[RemoteFile]:
    """Files still to fetch.  With ``prefer_gguf`` (e.g. ``"Q4_K_M"``) only the GGUF file of that quantisation is taken
    from a repository that ships several."""
    want = [f for f in remote if any(fnmatch.fnmatch(os.path.basename(f.path), p) for p in patterns)]
    ggufs = [f for f in want if f.path.endswith(".gguf")]
    if ggufs and prefer_gguf:
        keep = [f for f in ggufs if prefer_gguf.lower() in f.path.lower()] or ggufs[:1]
        want = [f for f in want if not f.path.endswith(".gguf")] + keep
    todo = []
    for f in want:
        p = os.path.join(dest, f.path)
        if os.path.exists(p) and (f.size == 0 or os.path.getsize(p) == f.size):
            continue
        todo.append(f)
    return todo


def _auth(token: Optional[str]) -> Dict[str, str]:
    token = token or os.environ.get("HF_TOKEN")
    return {"Authorization": f"Bearer {token}"} if token else {}


def _default_session():
    import requests
    return requests.Session()


def fetch_file(repo_id: str, revision: str, f: RemoteFile, dest: str, session=None, token: Optional[str] = None,
               cancel: Optional[threading.Event] = None, progress: Optional[Callable[[str, int, int], None]] = None) -> str:
    session = session or _default_session()
    final = os.path.join(dest, f.path)
    part = final + ".part"
    os.makedirs(os.path.dirname(final) or ".", exist_ok=True)
    have = os.path.getsize(part) if os.path.exists(part) else 0
    if f.size and have > f.size:                      # a stale partial from another revision
        os.remove(part)
        have = 0
    headers = _auth(token)
    if have:
        headers["Range"] = f"bytes={have}-"
    r = session.get(f"{HOST}/{repo_id}/resolve/{revision}/{f.path}", headers=headers, stream=True)
    code = getattr(r, "status_code", 200)
    if code == 200 and have:                          # the server ignored the range: start over
        have = 0
    elif code not in (200, 206):
        raise DownloadError(f"{f.path}: HTTP {code}")
    with open(part, "ab" if have else "wb") as out:
        for chunk in r.iter_content(CHUNK):
            if cancel is not None and cancel.is_set():
                raise Cancelled(f.path)               # the partial file stays for the next attempt
            if chunk:
                out.write(chunk)
                have += len(chunk)
                if progress:
                    progress(f.path, have, f.size)
    if f.size and have != f.size:
        raise DownloadError(f"{f.path}: got {have} bytes, expected {f.size}")
    os.replace(part, final)
    return final


def download(repo_id: str, cache_root: str, revision: str = "main", session=None, token: Optional[str] = None,
             cancel: Optional[threading.Event] = None, progress: Optional[Callable[[str, int, int], None]] = None,
             prefer_gguf: Optional[str] = None) -> str:
    """Fetch what is missing of ``repo_id`` into the hub-cache layout under ``cache_root``; returns the snapshot path."""
    session = session or _default_session()
    dest = snapshot_dir(cache_root, repo_id, revision)
    os.makedirs(dest, exist_ok=True)
    remote = list_remote(repo_id, revision, session, token)
    for f in plan(remote, dest, prefer_gguf=prefer_gguf):
        fetch_file(repo_id, revision, f, dest, session, token, cancel, progress)
    refs = os.path.join(os.path.dirname(os.path.dirname(dest)), "refs")
    os.makedirs(refs, exist_ok=True)
    with open(os.path.join(refs, revision.replace("/", "_")), "w") as fh:
        fh.write(revision)
    return dest
