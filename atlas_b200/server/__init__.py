"""HTTP serving layer (OpenAI / Anthropic / Responses / llama.cpp dialects)."""
from .app import ServerState, create_app  # noqa: F401
from .engine_async import AsyncEngine  # noqa: F401
