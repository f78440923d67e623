"""Checkpoint loading: safetensors shards, HF weight names, quantised formats, TP / EP sharding."""
from .checkpoint import Checkpoint  # noqa: F401
from .load import load_model, load_weights  # noqa: F401
from .qtensor import QTensor  # noqa: F401
