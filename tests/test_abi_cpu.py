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


def _route(elem, m, n, k, sms=148, reserve=0, stageable=1):
    out = (C.c_int32 * 6)()
    assert _lib.lib.zn_debug_tc_route(elem, m, n, k, sms, reserve, stageable, out) == 0
    return dict(zip(("pair", "tile_cols", "staged", "epi_warps", "band", "k_blocks"), out))


@pytest.mark.skipif(any(v in os.environ for v in ("ZN_TC_PAIR", "ZN_TC_NARROW", "ZN_TC_PAIR8", "ZN_TC_STAGED_STORE", "ZN_TC_BAND")),
                    reason="a diagnostic switch overrides the routing")
def test_tensor_core_gemm_routing():
    """Which tcgen05 GEMM form a product gets (host arithmetic, no device): the two-CTA kernel where the main loop is
    long AND its 256 x 256 tiles fill the 74 SM pairs more than once; otherwise the one-CTA kernel, with 128-column
    tiles where N fits one or the 256-column tiles would leave more than half the SMs idle."""
    BF16, TF32 = 0, 1
    # the wide MLP's products at 65,536 rows and at one rank's 8,192 rows of the 8-GPU step: two-CTA, per-thread stores
    for rows in (65536, 8192):
        for (m, n, k) in ((rows, 8192, 4096), (rows, 8192, 8192), (4096, 8192, rows), (8192, 8192, rows), (rows, 4096, 8192)):
            r = _route(BF16, m, n, k)
            assert (r["pair"], r["tile_cols"], r["staged"], r["epi_warps"]) == (1, 256, 0, 4), (m, n, k, r)
    # band height: 16 row tiles while a band's A strips stay within 34 MB (K up to 4096 bf16), else 8
    assert _route(BF16, 65536, 8192, 4096)["band"] == 16 and _route(BF16, 65536, 8192, 8192)["band"] == 8
    assert _route(TF32, 65536, 8192, 2048)["band"] == 16 and _route(TF32, 65536, 8192, 4096)["band"] == 8
    # a data-parallel step leaves 32 SMs free during its last GEMM's first rows: still two-CTA
    assert _route(BF16, 8192, 4096, 8192, reserve=32)["pair"] == 1
    # short main loop (at most 16 k-blocks: 1024 bf16 / 512 tf32 values): one-CTA, staged stores, 8 epilogue warps
    r = _route(BF16, 65536, 512, 512)
    assert (r["pair"], r["tile_cols"], r["staged"], r["epi_warps"], r["k_blocks"]) == (0, 256, 1, 8, 8)
    assert _route(BF16, 4096, 4096, 1024)["pair"] == 0 and _route(BF16, 4096, 4096, 1088)["pair"] == 1
    assert _route(TF32, 4096, 4096, 512)["pair"] == 0 and _route(TF32, 4096, 4096, 544)["pair"] == 1
    # a single wave of 256 x 256 tiles (2048^3: 64 tiles for 74 SM pairs) stays on the one-CTA kernel, two waves do not
    assert _route(BF16, 2048, 2048, 2048)["pair"] == 0 and _route(BF16, 4096, 4096, 4096)["pair"] == 1
    assert _route(BF16, 2048, 2048, 2048)["tile_cols"] == 256          # 128 wide tiles: enough for 148 SMs
    # few tiles: 128-column tiles double them (1024^3: 32 -> 64; the 784-512-256-10 network's layers)
    for shape in ((1024, 1024, 1024), (1024, 512, 784), (784, 512, 1024), (1024, 256, 512), (1024, 10, 256), (130, 10, 256)):
        for elem in (BF16, TF32):
            r = _route(elem, *shape)
            assert (r["pair"], r["tile_cols"]) == (0, 128), (shape, elem, r)
    # one row tile never pairs, whatever K
    assert _route(BF16, 128, 8192, 8192)["pair"] == 0 and _route(BF16, 64, 2048, 1500)["pair"] == 0
    # C += ..., two outputs or an odd pitch: per-thread stores in whichever kernel
    assert _route(BF16, 65536, 512, 512, stageable=0)["staged"] == 0 and _route(BF16, 1024, 1024, 1024, stageable=0)["staged"] == 0
    # bad arguments are refused
    out = (C.c_int32 * 6)()
    assert _lib.lib.zn_debug_tc_route(2, 128, 128, 128, 148, 0, 1, out) != 0
    assert _lib.lib.zn_debug_tc_route(0, 0, 128, 128, 148, 0, 1, out) != 0
    assert _lib.lib.zn_debug_tc_route(0, 128, 128, 128, 148, 0, 1, None) != 0
