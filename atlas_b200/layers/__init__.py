"""Decoder building blocks: attention, Gated DeltaNet, dense FFN, MoE, MTP head."""
from .common import ParallelCtx, make_weight, randn_weight  # noqa: F401
from .attention import Attention  # noqa: F401
from .mla import MLAttention  # noqa: F401
from .mlp import DenseMLP  # noqa: F401
from .moe import MoE  # noqa: F401
from .gdn import GatedDeltaNet  # noqa: F401
from .mamba2 import Mamba2Mixer  # noqa: F401
