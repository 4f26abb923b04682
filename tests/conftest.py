"""pytest configuration: registers the `gpu` marker and puts the package and the
oracle on sys.path. Tests marked gpu need a CUDA device and call the product only
through its C ABI; everything else runs on CPU."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# The tests run against the test-hook build of the library: the product's objects plus the
# lthn_debug_* entry points that force each kernel variant (go-inference_b200/build.py links
# both). Child processes of the multi-GPU tests inherit the choice through the environment.
_HOOKS = os.path.join(ROOT, "go-inference_b200", "liblthn_cuda_hooks.so")
if "LTHN_CUDA_LIB" not in os.environ and os.path.exists(_HOOKS):
    os.environ["LTHN_CUDA_LIB"] = _HOOKS
for p in (ROOT, os.path.join(ROOT, "go-inference_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _has_gpu() -> bool:
    try:
        import lthn
        return lthn.device_count() > 0
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    o.lib()
    return o


@pytest.fixture(scope="session")
def lthn():
    import lthn as m
    m.lib()
    return m
