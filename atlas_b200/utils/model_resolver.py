"""Model reference -> local checkpoint directory.

``serve`` accepts a directory, a ``preset:<name>`` (random weights), or a hub-style id ``org/name``.  Hub ids are
resolved offline, in this order: ``<dir>/<org>/<name>`` and ``<dir>/<name>`` for every directory in ``ATLAS_MODEL_DIRS``
(``os.pathsep``-separated), then the Hugging Face cache layout (``$HF_HUB_CACHE`` or ``$HF_HOME/hub`` or
``~/.cache/huggingface/hub``): ``models--org--name/snapshots/<revision>``, taking the revision named by ``refs/main``
when present and otherwise the most recently modified snapshot that contains a ``config.json``.  Nothing is downloaded:
a miss raises with the list of places that were searched.

Reference behaviour replaced: ``crates/spark-server/src/model_resolver.rs`` (the resolution order); the downloader of
``model_download/`` has no counterpart here.
"""
from __future__ import annotations

import os
from typing import List, Optional


class ModelNotFound(FileNotFoundError):
    pass


def _is_checkpoint(path: str) -> bool:
    return os.path.isfile(os.path.join(path, "config.json"))


def hub_cache_dirs() -> List[str]:
    out = []
    if os.environ.get("HF_HUB_CACHE"):
        out.append(os.environ["HF_HUB_CACHE"])
    if os.environ.get("HF_HOME"):
        out.append(os.path.join(os.environ["HF_HOME"], "hub"))
    out.append(os.path.join(os.path.expanduser("~"), ".cache", "huggingface", "hub"))
    return out


def _from_hub_cache(cache: str, repo_id: str, revision: Optional[str]) -> Optional[str]:
    root = os.path.join(cache, "models--" + repo_id.replace("/", "--"))
    snaps = os.path.join(root, "snapshots")
    if not os.path.isdir(snaps):
        return None
    want = revision
    if want is None:
        ref = os.path.join(root, "refs", "main")
        if os.path.isfile(ref):
            with open(ref) as f:
                want = f.read().strip()
    if want and _is_checkpoint(os.path.join(snaps, want)):
        return os.path.join(snaps, want)
    if revision is not None:
        return None
    cands = [os.path.join(snaps, d) for d in os.listdir(snaps)]
    cands = [c for c in cands if _is_checkpoint(c)]
    return max(cands, key=os.path.getmtime) if cands else None


def resolve_model(ref: str, revision: Optional[str] = None) -> str:
    """Local directory for ``ref`` (unchanged for ``preset:`` references)."""
    if ref.startswith("preset:"):
        return ref
    if os.path.isdir(ref):
        if not _is_checkpoint(ref):
            raise ModelNotFound(f"'{ref}' is a directory without a config.json")
        return ref
    searched: List[str] = []
    name = ref.rstrip("/").split("/")[-1]
    for base in [d for d in os.environ.get("ATLAS_MODEL_DIRS", "").split(os.pathsep) if d]:
        for cand in (os.path.join(base, ref), os.path.join(base, name)):
            searched.append(cand)
            if os.path.isdir(cand) and _is_checkpoint(cand):
                return cand
    if ref.count("/") == 1 and not ref.startswith((".", "/")):
        for cache in hub_cache_dirs():
            searched.append(os.path.join(cache, "models--" + ref.replace("/", "--")))
            hit = _from_hub_cache(cache, ref, revision)
            if hit:
                return hit
    raise ModelNotFound(f"model '{ref}' was not found locally (no download is attempted); searched: " + ", ".join(searched))
