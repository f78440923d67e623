import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
# guard bands around the kernel library's large buffers (KV pools, scratch areas): scanned after every GPU test
os.environ.setdefault("ATLAS_REDZONES", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch
    have = torch.cuda.is_available()
    ngpu = torch.cuda.device_count() if have else 0
    for item in items:
        if "gpu" in item.keywords and not have:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and ngpu < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(autouse=True)
def _scan_red_zones(request):
    """After every GPU test: no kernel may have written past either end of a guarded buffer.  Buffers of finished
    tests are dropped from the ledger so that the scan stays proportional to what the test allocated."""
    yield
    if "gpu" not in request.keywords:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from atlas_b200.utils import guards
    torch.cuda.synchronize()
    bad = guards.GLOBAL.scan()
    guards.GLOBAL.release("kv.")              # KV pools belong to the test that made them; scratch areas persist
    assert not bad, f"guard band damaged: {bad[:4]}"
