"""CPU-side checks of the drop-in boundary: the shared library loads, exports every
symbol the header declares, and its host-only logic agrees with the oracle."""
import ctypes as C
import os
import re

import pytest

import zigneuron_b200 as zn
from oracle import zn_oracle as zo
from zigneuron_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "zn_b200.h")).read()
    return sorted(set(re.findall(r"ZN_API[^;(]*?\b(zn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = header_symbols()
    assert len(names) >= 50
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} declared in zn_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_enums_follow_reference_order():
    # src/activation.zig:14-22 and src/loss.zig:12-22
    assert [a.name for a in zn.Activation] == ["relu", "sigmoid", "tanh", "softmax", "linear", "gelu", "leaky_relu", "elu"]
    assert [l.name for l in zn.Loss] == ["mse", "cross_entropy", "cross_entropy_logits", "binary_cross_entropy", "kl_divergence"]


def test_status_strings():
    assert _lib.lib.zn_status_string(0) == b"ok"
    assert b"shape" in _lib.lib.zn_status_string(7)


def test_distribute_workload_matches_oracle():
    for total, parts in [(10, 4), (65536, 8), (7, 8), (150, 3), (1, 1)]:
        for i in range(parts):
            assert zn.Backend.distributeWorkload(total, parts, i) == zo.distribute_round_robin(total, parts, i)
    s, e = C.c_size_t(), C.c_size_t()
    assert _lib.lib.zn_distribute_workload(10, 0, 0, C.byref(s), C.byref(e)) == 1   # ZN_ERR_INVALID_VALUE
    assert _lib.lib.zn_distribute_workload(10, 2, 2, C.byref(s), C.byref(e)) == 1


def test_no_device_means_error_not_fallback():
    if zn.Backend.device_count() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(zn.ZnError) as ei:
        zn.Backend()
    assert ei.value.status == 4   # ZN_ERR_NO_DEVICE


def test_null_handles_are_rejected():
    assert _lib.lib.zn_matmul(None, None, None, None, 1, 1, 1, 0) == 3   # ZN_ERR_NOT_INITIALIZED
    assert _lib.lib.zn_net_train_step(None, None, None, 1, 0.1, 0, None) == 3
    _lib.lib.zn_ctx_destroy(None)
    _lib.lib.zn_net_destroy(None)


def test_product_package_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "zigneuron_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "zn_oracle" not in text and "import oracle" not in text and "from oracle" not in text, f
