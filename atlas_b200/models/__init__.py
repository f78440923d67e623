"""Model definitions and the model_type -> builder factory."""
from .batch import ForwardBatch  # noqa: F401
from .decoder import CacheStore, DecoderLM  # noqa: F401
from .factory import build_model, supported_model_types  # noqa: F401
