"""Serving-box fingerprint for ``/hardware`` (GPU name, driver, clocks, memory) — read-only queries.

Reference parity: ``crates/avarok-plugin/src/hardware/*``.
"""
from __future__ import annotations

import platform
from typing import Any, Dict


def fingerprint() -> Dict[str, Any]:
    out: Dict[str, Any] = {"host": platform.node(), "python": platform.python_version(), "gpus": []}
    try:
        import torch
        out["torch"] = torch.__version__
        out["cuda"] = torch.version.cuda
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                p = torch.cuda.get_device_properties(i)
                out["gpus"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sm_count": p.multi_processor_count,
                                    "memory_gb": round(p.total_memory / 2 ** 30, 1)})
    except Exception as e:      # pragma: no cover
        out["torch_error"] = str(e)
    try:
        import pynvml
        pynvml.nvmlInit()
        out["driver"] = pynvml.nvmlSystemGetDriverVersion()
        for g in out["gpus"]:
            h = pynvml.nvmlDeviceGetHandleByIndex(g["index"])
            g["sm_clock_mhz"] = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
            g["sm_clock_max_mhz"] = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            g["power_limit_w"] = pynvml.nvmlDeviceGetPowerManagementLimit(h) / 1000.0
    except Exception:
        pass
    return out
