"""Parallelism: rank topology, collective backends (baseline + in-kernel), worker control plane."""
from .comm import CommBackend, CommError, FakeComm, FakeWorld, SingleGpuBackend, TorchDistBackend  # noqa: F401
from .topology import Topology, init_distributed  # noqa: F401
