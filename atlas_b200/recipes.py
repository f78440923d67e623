"""Serving recipes: a validated serve configuration for one checkpoint (model id, flag defaults, environment levers,
rank requirement and the rationale), read from YAML or from the built-in table, and turned into ``serve`` argv.

Precedence when serving: built-in flag defaults < recipe ``defaults`` < explicit command-line flags; ``env`` entries are
exported only when the variable is not already set by the operator.

Reference parity: ``crates/spark-server/src/recipe/{mod,schema,yaml}.rs`` (recipe struct, key -> flag mapping,
``min_nodes`` outside ``defaults``) and ``recipe/sync.rs`` (``sync``: an index of recipe files with checksums, fetched
into a local directory that ``resolve`` searches; ``file://`` indexes serve hermetic deployments).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

# recipe key -> (flag, kind).  kind: "value" (--flag v) or "switch" (--flag when truthy)
SCHEMA: Dict[str, tuple] = {
    "port": ("--port", "value"), "bind": ("--bind", "value"), "max_seq_len": ("--max-seq-len", "value"),
    "block_size": ("--block-size", "value"), "kv_cache_dtype": ("--kv-cache-dtype", "value"),
    "gpu_memory_utilization": ("--gpu-memory-utilization", "value"), "max_num_seqs": ("--max-num-seqs", "value"),
    "max_batch_size": ("--max-batch-size", "value"), "max_prefill_tokens": ("--max-prefill-tokens", "value"),
    "scheduling_policy": ("--scheduling-policy", "value"), "tbt_deadline_ms": ("--tbt-deadline-ms", "value"),
    "enable_prefix_caching": ("--enable-prefix-caching", "switch"), "speculative": ("--speculative", "switch"),
    "num_drafts": ("--num-drafts", "value"), "mtp_gate": ("--mtp-gate", "switch"),
    "ngram_speculative": ("--ngram-speculative", "switch"),
    "tp_size": ("--tp-size", "value"), "ep_size": ("--ep-size", "value"),
    "ssm_cache_slots": ("--ssm-cache-slots", "value"), "ssm_checkpoint_interval": ("--ssm-checkpoint-interval", "value"),
    "tool_call_parser": ("--tool-call-parser", "value"), "disable_thinking": ("--disable-thinking", "switch"),
    "max_thinking_budget": ("--max-thinking-budget", "value"), "request_timeout": ("--request-timeout", "value"),
    "quantization": ("--quantization", "value"), "comm": ("--comm", "value"), "no_cuda_graphs": ("--no-cuda-graphs", "switch"),
    "self_speculative": ("--self-speculative", "switch"), "self_spec_keep": ("--self-spec-keep", "value"),
    "mtp_vocab": ("--mtp-vocab", "value"), "mtp_vocab_rank": ("--mtp-vocab-rank", "value"),
    "think_confidence_streak": ("--think-confidence-streak", "value"),
}

ENV_PREFIX = "ATLAS_"


class RecipeError(ValueError):
    pass


@dataclass
class Recipe:
    id: str
    model: str
    version: str = "1"
    description: str = ""
    min_ranks: int = 1
    quantization: str = ""
    kv_dtype: str = ""
    defaults: Dict[str, Any] = field(default_factory=dict)
    env: Dict[str, str] = field(default_factory=dict)

    def validate(self) -> "Recipe":
        for k in self.defaults:
            if k not in SCHEMA:
                raise RecipeError(f"recipe {self.id}: unknown defaults key '{k}'")
        for k in self.env:
            if not k.startswith(ENV_PREFIX) and not k.startswith("NCCL_"):
                raise RecipeError(f"recipe {self.id}: env key '{k}' is not an {ENV_PREFIX}* / NCCL_* lever")
        tp, ep = int(self.defaults.get("tp_size", 1)), int(self.defaults.get("ep_size", 1))
        need = tp if tp == ep else tp * ep        # overlapping mesh (tp == ep == world) or orthogonal (tp x ep)
        if need > self.min_ranks:
            raise RecipeError(f"recipe {self.id}: tp_size {tp} / ep_size {ep} need {need} ranks but min_ranks is {self.min_ranks}")
        return self

    def argv(self) -> List[str]:
        """``serve`` arguments (model first)."""
        out = [self.model]
        for k, v in self.defaults.items():
            flag, kind = SCHEMA[k]
            if kind == "switch":
                if v in (True, "true", "True", 1, "1", "yes"):
                    out.append(flag)
            else:
                out += [flag, str(v)]
        return out

    def export_env(self, environ: Optional[dict] = None) -> Dict[str, str]:
        environ = os.environ if environ is None else environ
        applied = {}
        for k, v in self.env.items():
            if k not in environ:
                environ[k] = str(v)
                applied[k] = str(v)
        return applied


def from_dict(d: Dict[str, Any], rid: Optional[str] = None) -> Recipe:
    if "model" not in d:
        raise RecipeError("recipe has no 'model'")
    md = d.get("metadata") or {}
    r = Recipe(id=rid or d.get("id") or str(d["model"]), model=str(d["model"]), version=str(d.get("version", "1")),
               description=str(d.get("description", md.get("description", ""))),
               min_ranks=int(d.get("min_ranks", d.get("min_nodes", 1))),
               quantization=str(md.get("quantization", d.get("quantization", ""))),
               kv_dtype=str(md.get("kv_dtype", "")), defaults=dict(d.get("defaults") or {}),
               env={str(k): str(v) for k, v in (d.get("env") or {}).items()})
    return r.validate()


def load(path: str) -> Recipe:
    import yaml
    with open(path) as f:
        d = yaml.safe_load(f)
    if not isinstance(d, dict):
        raise RecipeError(f"{path}: a recipe is a mapping")
    stem = os.path.splitext(os.path.basename(path))[0]
    parent = os.path.basename(os.path.dirname(os.path.abspath(path)))
    return from_dict(d, f"{parent}/{stem}")


# Shapes this engine is tuned and benchmarked on (random-init presets; swap ``model`` for a checkpoint directory).
BUILTIN: Dict[str, Dict[str, Any]] = {
    "llama/llama3-8b-fp8": {"model": "preset:llama3-8b", "description": "dense 8B, FP8 block-scaled weights, FP8 KV, one GPU",
                            "defaults": {"max_seq_len": 8192, "max_num_seqs": 128, "max_batch_size": 128,
                                         "kv_cache_dtype": "fp8", "quantization": "fp8_block"}},
    "llama/llama3-70b-fp8-tp8": {"model": "preset:llama3-70b", "min_ranks": 8,
                                 "description": "dense 70B over 8 GPUs, row-parallel GEMMs fused with their all-reduce",
                                 "defaults": {"tp_size": 8, "max_seq_len": 32768, "max_prefill_tokens": 32768,
                                              "max_num_seqs": 64, "max_batch_size": 64, "kv_cache_dtype": "fp8",
                                              "quantization": "fp8_block", "comm": "p2p"}},
    "qwen/qwen3-30b-a3b-nvfp4-ep8": {"model": "preset:qwen3-30b-a3b", "min_ranks": 8,
                                     "description": "128-expert MoE, NVFP4 experts, expert parallel over 8 GPUs",
                                     "defaults": {"ep_size": 8, "tp_size": 8, "max_seq_len": 8192, "kv_cache_dtype": "fp8",
                                                  "quantization": "nvfp4", "tool_call_parser": "hermes"}},
    "qwen/qwen3-next-80b-a3b-fp8": {"model": "preset:qwen3-next-80b", "min_ranks": 2,
                                    "description": "hybrid GDN/attention MoE with a 1-layer MTP head, depth-3 speculation, prefix cache",
                                    "defaults": {"tp_size": 2, "ep_size": 2, "max_seq_len": 32768, "speculative": True,
                                                 "num_drafts": 3, "mtp_gate": True, "enable_prefix_caching": True,
                                                 "ssm_cache_slots": 32, "kv_cache_dtype": "fp8", "quantization": "fp8_block",
                                                 "tool_call_parser": "qwen3_coder"}},
}


def builtin(rid: str) -> Recipe:
    if rid not in BUILTIN:
        raise RecipeError(f"unknown recipe '{rid}'; known: {', '.join(sorted(BUILTIN))}")
    return from_dict(BUILTIN[rid], rid)


def synced_dir() -> str:
    return os.environ.get("ATLAS_RECIPES_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "atlas_b200", "recipes")


def resolve(spec: str) -> Recipe:
    """A path to a YAML file, the id of a synced recipe (``family/name`` under ``synced_dir()``), or a built-in id."""
    if os.path.exists(spec):
        return load(spec)
    local = os.path.join(synced_dir(), spec + ".yaml")
    if ".." not in spec.split("/") and os.path.exists(local):
        return load(local)
    return builtin(spec)


def sync(index_url: str, dest: Optional[str] = None, timeout_s: float = 30.0) -> List[str]:
    """Fetch a recipe index and the recipes it lists into ``dest`` (default ``synced_dir()``); returns the ids written.

    The index is JSON: ``{"recipes": [{"id": "family/name", "url": "...", "sha256": "..."}]}``; relative urls are taken
    against the index's own location, ``file://`` works like ``https://``.  A file is written only after its checksum
    matched and it parsed as a valid recipe, under a temporary name that is renamed into place, so a failed sync leaves
    the previous copy of every recipe untouched."""
    import hashlib
    import json
    import urllib.parse
    import urllib.request
    dest = dest or synced_dir()

    def fetch(url: str) -> bytes:
        with urllib.request.urlopen(url, timeout=timeout_s) as r:
            return r.read()
    index = json.loads(fetch(index_url).decode())
    entries = index.get("recipes") if isinstance(index, dict) else index
    if not isinstance(entries, list):
        raise RecipeError("the recipe index lists no recipes")
    staged = []
    for e in entries:
        rid = str(e.get("id", ""))
        parts = rid.split("/")
        if len(parts) != 2 or not all(p and p not in (".", "..") and os.sep not in p for p in parts):
            raise RecipeError(f"bad recipe id in the index: '{rid}'")
        data = fetch(urllib.parse.urljoin(index_url, str(e["url"])))
        digest = hashlib.sha256(data).hexdigest()
        if e.get("sha256") and digest != str(e["sha256"]).lower():
            raise RecipeError(f"{rid}: checksum mismatch (index {e['sha256']}, file {digest})")
        import yaml
        from_dict(yaml.safe_load(data.decode()), rid)        # raises on an invalid recipe
        staged.append((rid, data))
    written = []
    for rid, data in staged:
        path = os.path.join(dest, rid + ".yaml")
        os.makedirs(os.path.dirname(path), exist_ok=True)
        tmp = path + ".part"
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, path)
        written.append(rid)
    return written
