"""Bindings of the MoE, Gated-DeltaNet and NVFP4 translation units of the kernel library."""
from __future__ import annotations

import torch


def bind(lib) -> None:
    pass


def _missing(name):
    raise NotImplementedError(f"{name}: sm_100a kernel not built yet")


def gemm_nvfp4(x, packed, bscale, gscale, out=None):
    _missing("gemm_nvfp4")


def moe_route(logits, top_k, norm_topk, scoring):
    _missing("moe_route")


def moe_forward(x, topk_w, topk_ids, experts, e_lo, pctx, ep_mode):
    _missing("moe_forward")


def gdn_forward(layer, mixed, a, b, batch, state, commit):
    _missing("gdn_forward")


def gdn_commit(layer, mixed, a, b, qlens, slots, has_state, state, num_accepted_rows):
    _missing("gdn_commit")
