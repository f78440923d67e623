"""model_type dispatch (single site, like ``crates/spark-model/src/factory.rs:68-160``)."""
from __future__ import annotations

from typing import List, Optional

from ..config import ModelConfig, _FAMILY_ALIASES
from ..layers import ParallelCtx
from .decoder import DecoderLM


def supported_model_types() -> List[str]:
    return sorted(_FAMILY_ALIASES)


def build_model(cfg: ModelConfig, pctx: Optional[ParallelCtx] = None, device="cpu", ep_mode: str = "auto",
                with_mtp: Optional[bool] = None) -> DecoderLM:
    """Construct the (weight-less) model for ``cfg``; raises ``ValueError`` for unknown families."""
    if cfg.model_type not in _FAMILY_ALIASES:
        raise ValueError(f"Unsupported model_type '{cfg.model_type}'")
    return DecoderLM(cfg, pctx, device, ep_mode, with_mtp)
