"""atlas_b200: a Blackwell (sm_100a) native LLM inference engine.

Public entry points:

* :class:`atlas_b200.engine.LLMEngine` — continuous-batching engine (``add_request`` / ``step`` / ``generate``).
* :mod:`atlas_b200.server` — OpenAI / Anthropic / Responses compatible HTTP server.
* :mod:`atlas_b200.ops` — fused ops (sm_100a kernels on GPU, plain PyTorch restatement on CPU).
"""
__version__ = "0.1.0"

from .config import EngineConfig, ModelConfig, QuantConfig, PRESETS  # noqa: F401
