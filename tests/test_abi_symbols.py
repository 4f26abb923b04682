"""The C-ABI library loads without a GPU and exports every symbol the public
header declares; the host-side argument validation mirrors the reference's."""
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "lthn_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lthn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import lthn
    lib = lthn.lib()
    names = declared_symbols()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_product_library_has_no_test_hooks():
    """liblthn_cuda.so (what bench.py, smoke() and a cgo shim load) exports every declared symbol
    and none of the lthn_debug_* hooks; those exist only in liblthn_cuda_hooks.so."""
    import ctypes
    prod = ctypes.CDLL(os.path.join(ROOT, "go-inference_b200", "liblthn_cuda.so"))
    missing = [n for n in declared_symbols() if not hasattr(prod, n)]
    assert not missing, missing
    for hook in ("lthn_debug_qmv_force_config", "lthn_debug_qmv_force_kernel", "lthn_debug_qmm_force_tile",
                 "lthn_debug_rmsnorm_gather_local", "lthn_debug_i8_plan"):
        assert not hasattr(prod, hook), hook
    hooks = ctypes.CDLL(os.path.join(ROOT, "go-inference_b200", "liblthn_cuda_hooks.so"))
    assert hasattr(hooks, "lthn_debug_qmv_force_kernel")


def test_binding_covers_every_declared_symbol():
    import lthn
    bound = {n for n in dir(lthn._Sig) if n.startswith("lthn_")}
    unbound = [n for n in declared_symbols() if n not in bound and n != "lthn_last_error"]
    assert not unbound, unbound


def test_available_is_false_not_an_error_without_gpu():
    import lthn
    assert lthn.lib().lthn_cuda_available() in (0, 1)
    assert lthn.lib().lthn_cuda_device_count() >= 0


def test_matvec_validation_matches_reference_surface():
    """enginetest/quant_reference_test.go:43-74: malformed inputs are errors, the
    zero-sized call is a clean empty result. Validation runs before any device work."""
    import lthn
    x = np.zeros(128, dtype=np.uint16)
    p = np.zeros((8, 16), dtype=np.uint32)
    s = np.zeros((8, 2), dtype=np.uint16)
    with pytest.raises(lthn.LthnError):
        lthn.qmv_host(x[:-1], p, s, s, 8, 128, 64, 4)
    with pytest.raises(lthn.LthnError):
        lthn.qmv_host(x, p.reshape(-1)[:-1], s, s, 8, 128, 64, 4)
    with pytest.raises(lthn.LthnError):
        lthn.qmv_host(x, p, s, s, 8, 128, 3, 4)
    with pytest.raises(lthn.LthnError):
        lthn.qmv_host(x, p, s, s, 8, 128, 64, 0)
    with pytest.raises(lthn.LthnError):
        lthn.qmv_host(x, p, s, s, 8, 128, 64, 9)
    e = np.zeros(0, dtype=np.uint8)
    assert lthn.qmv_host(e, e, e, e, 0, 0, 64, 4).size == 0
