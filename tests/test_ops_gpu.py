"""GPU parity of every Backend op on the Dense path against the CPU oracle, through
the C ABI.  Tolerances: bit-exact for FP32_EXACT GEMMs and element-wise ops; 1e-5
relative (L2 and max norm) for the fp32 FMA path; 2e-2 for TF32/BF16 tensor-core
GEMMs on raw inputs, and 1e-5 again when the inputs are pre-rounded to the operand
type (which isolates the kernel from the input rounding)."""
import numpy as np
import pytest

import zigneuron_b200 as zn
from oracle import zn_oracle as zo
from util import assert_close, rel_l2, round_bf16, trunc_tf32

pytestmark = pytest.mark.gpu

P = zn.Precision


@pytest.fixture(scope="module")
def be():
    b = zn.Backend(0)
    yield b
    b.deinit()


def _operands(rng, orient, m, n, k):
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    return a, b


def _store(orient, a, b):
    """Memory layout each entry point expects."""
    if orient == "NN":
        return np.ascontiguousarray(a), np.ascontiguousarray(b)
    if orient == "TN":
        return np.ascontiguousarray(a.T), np.ascontiguousarray(b)      # A stored [k][m]
    return np.ascontiguousarray(a), np.ascontiguousarray(b.T)          # B stored [n][k]


def _oracle(orient, sa, sb, m, n, k, c=None, acc=False):
    f = {"NN": zo.matmul, "TN": zo.matmul_transpose_a, "NT": zo.matmul_transpose_b}[orient]
    return f(sa, sb, m, n, k, c=c, accumulate=acc)


def _reference(orient, sa, sb, m, n, k):
    """The oracle's product; for the few shapes of more than 10^9 multiply-adds, which its plain loops would take
    minutes over, the same product in float64 (the tensor-core tolerances below are far wider than the 1e-6 by
    which the oracle's fp32 sums and float64 differ)."""
    if m * n * k <= 1_000_000_000:
        return _oracle(orient, sa, sb, m, n, k)
    a = sa.astype(np.float64).reshape((k, m) if orient == "TN" else (m, k))
    b = sb.astype(np.float64).reshape((n, k) if orient == "NT" else (k, n))
    return ((a.T if orient == "TN" else a) @ (b.T if orient == "NT" else b)).astype(np.float32)


def _gpu(be, orient, sa, sb, m, n, k, c=None, acc=False):
    out = np.zeros((m, n), np.float32) if c is None else c.copy()
    f = {"NN": be.matMul, "TN": be.matMulTransposeA, "NT": be.matMulTransposeB}[orient]
    f(sa, sb, out, m, n, k, acc)
    return out


SHAPES = [(2, 2, 3), (64, 64, 64), (150, 20, 4), (1, 10, 256), (129, 257, 65), (1024, 512, 784), (300, 130, 1000)]


@pytest.mark.parametrize("orient", ["NN", "NT", "TN"])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemm_fp32(be, orient, shape):
    m, n, k = shape
    rng = np.random.default_rng(4)
    sa, sb = _store(orient, *_operands(rng, orient, m, n, k))
    want = _oracle(orient, sa, sb, m, n, k)
    be.set_precision(P.FP32_EXACT)
    got = _gpu(be, orient, sa, sb, m, n, k)
    assert np.array_equal(got, want), f"exact path differs: {rel_l2(got, want):.3e}"
    be.set_precision(P.FP32_SIMT)
    assert_close(_gpu(be, orient, sa, sb, m, n, k), want, 1e-5, f"simt {orient} {shape}")


def test_gemm_golden_vectors(be):
    """The reference's own known answers (src/test/unit/backend.zig:196-250)."""
    be.set_precision(P.FP32_SIMT)
    a = np.array([1, 2, 3, 4, 5, 6], np.float32)
    b = np.array([7, 8, 9, 10, 11, 12], np.float32)
    c = np.zeros(4, np.float32)
    be.matMul(a, b, c, 2, 2, 3)
    assert np.allclose(c, [58, 64, 139, 154], atol=1e-4)
    ones = np.ones(64 * 64, np.float32)
    c = np.zeros(64 * 64, np.float32)
    for prec in (P.FP32_SIMT, P.TF32_TC, P.BF16_TC):
        be.set_precision(prec)
        be.matMul(ones, ones, c, 64, 64, 64)
        assert np.allclose(c, 64.0, atol=1e-4), prec


@pytest.mark.parametrize("orient", ["NN", "NT", "TN"])
def test_gemm_accumulate(be, orient):
    m, n, k = 70, 40, 33
    rng = np.random.default_rng(5)
    sa, sb = _store(orient, *_operands(rng, orient, m, n, k))
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    want = _oracle(orient, sa, sb, m, n, k, c=c0, acc=True)
    be.set_precision(P.FP32_EXACT)
    assert np.array_equal(_gpu(be, orient, sa, sb, m, n, k, c=c0, acc=True), want)
    be.set_precision(P.BF16_TC)
    assert_close(_gpu(be, orient, sa, sb, m, n, k, c=c0, acc=True), want, 2e-2)


# Routing.  The two-CTA kernel takes products with more than one row tile, a long K (more than 1024 bf16 / 512 tf32
# values) AND more 256 x 256 tiles than the GPU has SM pairs (74): the last row.  Everything else runs the one-CTA
# kernel, with 128-column tiles where N fits one or the 256-column tiles would fill at most half the SMs (rows one
# to three), with 256-column tiles otherwise (row four).
TC_SHAPES = [(128, 256, 64), (256, 512, 256), (300, 200, 100), (130, 10, 256), (1024, 512, 784), (64, 2048, 1500),
             (2048, 1024, 512), (384, 320, 2304), (300, 520, 1100), (513, 260, 4100),
             (1024, 1024, 1024), (200, 136, 96), (256, 384, 512),
             (4096, 1200, 256), (2500, 2304, 200),
             (2048, 2560, 1100), (1300, 3900, 2304)]


@pytest.mark.parametrize("prec", [P.BF16_TC, P.TF32_TC])
@pytest.mark.parametrize("orient", ["NN", "NT", "TN"])
@pytest.mark.parametrize("shape", TC_SHAPES)
def test_gemm_tensor_core(be, prec, orient, shape):
    m, n, k = shape
    rng = np.random.default_rng(4)
    a, b = _operands(rng, orient, m, n, k)
    be.set_precision(prec)
    # (1) raw fp32 inputs: the bar for the tensor-core path is 2e-2
    sa, sb = _store(orient, a, b)
    want = _reference(orient, sa, sb, m, n, k)
    assert_close(_gpu(be, orient, sa, sb, m, n, k), want, 2e-2, f"{prec.name} {orient} {shape}")
    # (2) inputs already representable in the operand type: only accumulation order differs
    rnd = round_bf16 if prec == P.BF16_TC else trunc_tf32
    sa, sb = _store(orient, rnd(a), rnd(b))
    want = _reference(orient, sa, sb, m, n, k)
    # The tensor cores add their products into fp32 without rounding every partial sum to nearest, so what is left
    # grows with the length of the sum: measured 1.08e-5 (tf32) at K = 4100, below 5e-6 up to K = 2304.
    tol = 1e-5 * max(1.0, (k / 1024.0) ** 0.5)
    assert_close(_gpu(be, orient, sa, sb, m, n, k), want, tol, f"{prec.name} {orient} {shape} pre-rounded")


@pytest.mark.parametrize("prec", [P.FP32_EXACT, P.FP32_SIMT, P.TF32_TC, P.BF16_TC])
@pytest.mark.parametrize("act", ["linear", "relu", "sigmoid", "tanh"])
def test_matmul_bias_act(be, prec, act):
    batch, n, k = 200, 96, 72
    rng = np.random.default_rng(4)
    a = rng.standard_normal((batch, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)     # pre-activations of order 1
    bias = rng.uniform(-0.1, 0.1, n).astype(np.float32)
    want = zo.activation_forward(getattr(zo, act.upper()), zo.add_bias(zo.matmul(a, w, batch, n, k), bias))
    be.set_precision(prec)
    got = np.zeros((batch, n), np.float32)
    be._mm_bias(a, w, bias, got, batch, n, k, zn.Activation[act])
    if prec == P.FP32_EXACT and act in ("linear", "relu"):
        assert np.array_equal(got, want)
    else:
        assert_close(got, want, 1e-5 if prec in (P.FP32_EXACT, P.FP32_SIMT) else 2e-2, f"{prec.name} {act}")


def test_bias_ops(be):
    rng = np.random.default_rng(6)
    for rows, cols in [(1, 1), (150, 3), (1024, 10), (4097, 513), (64, 8192)]:
        out = rng.standard_normal((rows, cols)).astype(np.float32)
        bias = rng.standard_normal(cols).astype(np.float32)
        want = zo.add_bias(out, bias)
        got = out.copy()
        be.addBias(got, bias)
        assert np.array_equal(got, want)
        gb0 = rng.standard_normal(cols).astype(np.float32)
        want = zo.accumulate_bias(gb0, out)
        be.set_precision(P.FP32_EXACT)
        got = gb0.copy()
        be.accumulateBias(got, out)
        assert np.array_equal(got, want), (rows, cols)
        be.set_precision(P.FP32_SIMT)
        got = gb0.copy()
        be.accumulateBias(got, out)
        # a blocked sum of `rows` terms: bound the error against the size of the terms
        assert np.max(np.abs(got - want)) <= 1e-5 * max(1.0, np.sqrt(rows)) * np.max(np.abs(out)), (rows, cols)


def test_activations(be):
    # reference vectors: src/test/cuda/operations.zig:201-258
    x = np.array([-1.0, -0.5, 0.0, 0.5, 1.0, 2.0], np.float32)
    y = np.empty_like(x)
    be.activationForward(zn.Activation.relu, x, y)
    assert np.array_equal(y, [0, 0, 0, 0.5, 1, 2])
    gi = np.empty_like(x)
    be.activationBackward(zn.Activation.relu, y, np.ones(6, np.float32), gi)
    assert np.array_equal(gi, [0, 0, 0, 1, 1, 1])
    rng = np.random.default_rng(7)
    x = rng.standard_normal(10007).astype(np.float32) * 3
    g = rng.standard_normal(10007).astype(np.float32)
    for name in ("relu", "linear", "sigmoid", "tanh", "gelu", "leaky_relu", "elu"):
        act, oact = zn.Activation[name], getattr(zo, name.upper())
        y = np.empty_like(x)
        be.activationForward(act, x, y)
        want = zo.activation_forward(oact, x)
        if name in ("relu", "linear", "leaky_relu"):
            assert np.array_equal(y, want)
        else:
            assert_close(y, want, 1e-6, name)
        gi = np.empty_like(x)
        be.activationBackward(act, want, g, gi)
        if name == "gelu":       # its derivative calls tanhf, which differs from the host's in the last place
            assert_close(gi, zo.activation_backward(oact, want, g), 1e-6, name)
        else:
            assert np.array_equal(gi, zo.activation_backward(oact, want, g)), name
    x2 = x.copy()
    be.activationForward(zn.Activation.relu, x2, x2)      # in place, as Dense.forward does
    assert np.array_equal(x2, np.maximum(x, 0))
    # leaky_relu / elu / gelu known answers (src/activation.zig:128-185 by hand)
    pts = np.array([-2.0, -1.0, 0.0, 1.0, 3.0], np.float32)
    out = np.empty_like(pts)
    be.activationForward(zn.Activation.leaky_relu, pts, out)
    assert np.allclose(out, [-0.02, -0.01, 0.0, 1.0, 3.0], atol=1e-7)
    be.activationForward(zn.Activation.elu, pts, out)
    assert np.allclose(out, [np.expm1(-2.0), np.expm1(-1.0), 0.0, 1.0, 3.0], atol=1e-6)
    be.activationForward(zn.Activation.gelu, pts, out)
    assert abs(out[3] - 0.84119199) < 1e-6 and abs(out[1] + 0.15880801) < 1e-6 and out[2] == 0.0


def test_softmax_activation(be):
    """Backend.activationForward / activationBackward with softmax take the whole slice as ONE vector
    (src/backend.zig:377-379, :2650-2652; src/activation.zig:51-95)."""
    # reference test vectors: src/test/unit/activation.zig:55-76, :149-159
    y = np.empty(3, np.float32)
    be.activationForward(zn.Activation.softmax, np.array([1.0, 2.0, 3.0], np.float32), y)
    assert abs(float(y.sum()) - 1.0) < 1e-3 and y[2] > y[1] > y[0]
    assert np.allclose(y, [0.09003057, 0.24472847, 0.66524096], atol=1e-6)
    gi = np.empty(2, np.float32)
    be.activationBackward(zn.Activation.softmax, np.array([0.0, 1.0], np.float32), np.ones(2, np.float32), gi)
    assert abs(float(gi.sum())) < 1e-4
    rng = np.random.default_rng(17)
    for n in (1, 7, 32, 33, 1000, 10007):
        x = (rng.standard_normal(n) * 3).astype(np.float32)
        g = rng.standard_normal(n).astype(np.float32)
        y = np.empty_like(x)
        be.activationForward(zn.Activation.softmax, x, y)
        want = zo.activation_forward(zo.SOFTMAX, x)
        # the oracle adds the exponentials into one running f32 sum; over 1e4 terms that sum is itself off by
        # a few 1e-6 (FP32_EXACT, below, reproduces the order)
        assert_close(y, want, 1e-5, f"softmax {n}")
        gi = np.empty_like(x)
        be.activationBackward(zn.Activation.softmax, want, g, gi)
        wgi = zo.activation_backward(zo.SOFTMAX, want, g)
        assert np.abs(gi - wgi).max() <= 1e-5 * max(np.abs(wgi).max(), 1e-6), n
    x = (rng.standard_normal(50) * 2).astype(np.float32)
    x2 = x.copy()
    be.activationForward(zn.Activation.softmax, x2, x2)     # in place
    assert_close(x2, zo.activation_forward(zo.SOFTMAX, x), 2e-6, "in place")
    # all -inf: the sum of exponentials is not > 0, the reference answers with the uniform vector
    y = np.empty(4, np.float32)
    be.activationForward(zn.Activation.softmax, np.full(4, -np.inf, np.float32), y)
    assert np.allclose(y, 0.25)
    # reference order under FP32_EXACT: the only differences left are expf's last place
    bx = zn.Backend(precision=zn.Precision.FP32_EXACT)
    x = (rng.standard_normal(4099) * 3).astype(np.float32)
    y = np.empty_like(x)
    bx.activationForward(zn.Activation.softmax, x, y)
    assert_close(y, zo.activation_forward(zo.SOFTMAX, x), 1e-6, "exact order")
    bx.deinit()


def test_matmul_bias_softmax_rows(be):
    """The fused Dense forward with softmax normalises every row (src/layer.zig:398-406)."""
    rng = np.random.default_rng(18)
    m, n, k = 37, 10, 64
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((k, n)) / 8).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    c = np.empty((m, n), np.float32)
    be.matMulBiasAct(a, b, bias, c, m, n, k, zn.Activation.softmax)
    z = zo.add_bias(zo.matmul(a, b, m, n, k), bias).reshape(m, n)
    want = np.stack([zo.activation_forward(zo.SOFTMAX, z[r]) for r in range(m)])
    assert_close(c, want, 1e-5, "softmax rows")
    assert np.allclose(c.sum(axis=1), 1.0, atol=1e-5)


def test_losses(be):
    # golden: src/test/unit/loss.zig:14-42, :75-87
    assert abs(be.lossForward(zn.Loss.mse, np.array([1, 2, 3], np.float32), np.array([0, 1, 2], np.float32)) - 1.0) < 1e-6
    g = np.empty(2, np.float32)
    be.lossBackward(zn.Loss.mse, np.array([1, 2], np.float32), np.array([0, 1], np.float32), g)
    assert np.allclose(g, [1, 1], atol=1e-6)
    be.lossBackward(zn.Loss.cross_entropy_logits, np.zeros(2, np.float32), np.array([1, 0], np.float32), g)
    assert np.allclose(g, [-0.5, 0.5], atol=1e-6)
    rng = np.random.default_rng(8)
    for rows, cols in [(1, 3), (150, 3), (1024, 10), (33, 1000), (513, 4096)]:
        o = rng.standard_normal((rows, cols)).astype(np.float32) * 2
        t = np.eye(cols, dtype=np.float32)[rng.integers(0, cols, rows)]
        tm = rng.standard_normal((rows, cols)).astype(np.float32)
        g = np.empty((rows, cols), np.float32)
        be.lossBackward(zn.Loss.mse, o, tm, g, rows)
        assert np.array_equal(g, zo.loss_backward(zo.MSE, o, tm, rows, cols))
        got = be.lossForward(zn.Loss.mse, o, tm, rows)
        exact = float(np.mean((o.astype(np.float64) - tm) ** 2))
        assert abs(got - exact) <= 1e-6 * exact
        # the oracle's single running f32 sum loses digits on long inputs; allow for ITS error there
        assert abs(got - zo.loss_forward(zo.MSE, o, tm, rows, cols)) <= (1e-5 if rows * cols <= 50000 else 5e-3) * exact
        be.lossBackward(zn.Loss.cross_entropy_logits, o, t, g, rows)
        assert_close(g, zo.loss_backward(zo.CE_LOGITS, o, t, rows, cols), 1e-5, f"ce grad {rows}x{cols}")
        got = be.lossForward(zn.Loss.cross_entropy_logits, o, t, rows)
        want = zo.loss_forward(zo.CE_LOGITS, o, t, rows, cols)
        assert abs(got - want) <= 1e-5 * max(1.0, abs(want)), (rows, cols)
    with pytest.raises(zn.ZnError):
        be.lossForward(zn.Loss.kl_divergence, o, t, rows)


def test_cross_entropy_and_bce_losses(be):
    """Loss.cross_entropy (src/loss.zig:110-196) and Loss.binary_cross_entropy (:255-302)."""
    # golden: src/test/unit/loss.zig:63-113
    got = be.lossForward(zn.Loss.cross_entropy, np.array([1, 0], np.float32), np.array([1, 0], np.float32))
    assert abs(got - 0.31326169) < 1e-6
    g = np.empty(2, np.float32)
    be.lossBackward(zn.Loss.cross_entropy, np.zeros(2, np.float32), np.array([1, 0], np.float32), g)
    assert np.allclose(g, [-0.5, 0.5], atol=1e-6)
    got = be.lossForward(zn.Loss.binary_cross_entropy, np.array([0.01, 0.99], np.float32), np.array([0, 1], np.float32))
    assert abs(got - 0.01005034) < 1e-6
    be.lossBackward(zn.Loss.binary_cross_entropy, np.array([0.7, 0.3], np.float32), np.array([1, 0], np.float32), g)
    assert np.allclose(g, [-0.15, 0.15], atol=1e-6)
    rng = np.random.default_rng(28)
    bx = zn.Backend(precision=zn.Precision.FP32_EXACT)
    for rows, cols in [(1, 3), (150, 3), (1024, 10), (33, 1000)]:
        o = (rng.standard_normal((rows, cols)) * 2).astype(np.float32)
        t = np.eye(cols, dtype=np.float32)[rng.integers(0, cols, rows)]
        t[rng.integers(0, rows, rows // 8), rng.integers(0, cols, rows // 8)] = 1.0        # some multi-hot rows
        t[rng.integers(0, rows, max(rows // 16, 1))] = 0.0                                   # some rows without a target
        g = np.empty((rows, cols), np.float32)
        be.lossBackward(zn.Loss.cross_entropy, o, t, g, rows)
        assert_close(g, zo.loss_backward(zo.CE, o, t, rows, cols), 1e-5, f"ce grad {rows}x{cols}")
        want = zo.loss_forward(zo.CE, o, t, rows, cols)
        for b_, tol in ((be, 2e-6), (bx, 1e-6)):
            got = b_.lossForward(zn.Loss.cross_entropy, o, t, rows)
            assert abs(got - want) <= tol * max(1.0, abs(want)), (rows, cols, got, want)
        p = rng.uniform(0, 1, (rows, cols)).astype(np.float32)
        p[rng.integers(0, rows, max(rows // 10, 1)), rng.integers(0, cols, max(rows // 10, 1))] = 0.0       # clamped
        p[rng.integers(0, rows, max(rows // 10, 1)), rng.integers(0, cols, max(rows // 10, 1))] = 1.0
        tb = (rng.uniform(0, 1, (rows, cols)) > 0.5).astype(np.float32)
        be.lossBackward(zn.Loss.binary_cross_entropy, p, tb, g, rows)
        assert np.array_equal(g, zo.loss_backward(zo.BCE, p, tb, rows, cols))
        want = zo.loss_forward(zo.BCE, p, tb, rows, cols)
        exact64 = float(np.mean(-(tb * np.log(np.clip(p, np.float32(1e-7), np.float32(1) - np.float32(1e-7)).astype(np.float64))
                                  + (1 - tb) * np.log(np.clip(np.float32(1) - np.clip(p, np.float32(1e-7), np.float32(1) - np.float32(1e-7)),
                                                              np.float32(1e-7), np.float32(1) - np.float32(1e-7)).astype(np.float64)))))
        got = be.lossForward(zn.Loss.binary_cross_entropy, p, tb, rows)
        assert abs(got - exact64) <= 2e-6 * exact64, (rows, cols, got, exact64)
        got = bx.lossForward(zn.Loss.binary_cross_entropy, p, tb, rows)          # the reference's running f32 sum
        assert abs(got - want) <= 2e-6 * want, (rows, cols, got, want)
    bx.deinit()
    # degenerate rows of cross_entropy give 0
    assert be.lossForward(zn.Loss.cross_entropy, np.array([1, 2, 3], np.float32), np.zeros(3, np.float32)) == 0.0
    assert be.lossForward(zn.Loss.cross_entropy, np.full(3, -np.inf, np.float32), np.array([1, 0, 0], np.float32)) == 0.0


def test_optimizers(be):
    rng = np.random.default_rng(9)
    n = 100003
    w = rng.standard_normal(n).astype(np.float32) * 40
    g = rng.standard_normal(n).astype(np.float32) * 4
    g[::97] = np.nan
    g[5::101] = 77.0
    for lr, wd in [(0.01, 0.0), (0.5, 0.01)]:
        got = w.copy()
        be.sgdUpdate(got, g, lr, wd)
        assert np.array_equal(got, zo.sgd_update(w, g, lr, wd))
    got = w.copy()
    be.sgdUpdateBias(got, g, 2.0)
    assert np.array_equal(got, zo.sgd_update_bias(w, g, 2.0))
    m = rng.standard_normal(n).astype(np.float32) * 0.1
    v = np.abs(rng.standard_normal(n)).astype(np.float32) * 0.01
    for t in (1, 2, 100):
        bc1, bc2 = zo.adam_bias_corrections(0.9, 0.999, t)
        ww, mm, vv = zo.adam_update(w, g, m, v, 1e-3, 0.9, 0.999, 1e-8, bc1, bc2)
        gw, gm, gv = w.copy(), m.copy(), v.copy()
        be.adamUpdate(gw, g, gm, gv, 1e-3, 0.9, 0.999, 1e-8, bc1, bc2)
        assert np.array_equal(gm, mm) and np.array_equal(gv, vv)
        assert np.array_equal(gw, ww)
    # golden: w 0.5, g 0.1, lr 1e-3, t = 1 -> 0.499 (src/test/unit/optimizer.zig:66-88, src/backend.zig:2760-2772)
    w1, m1, v1 = np.array([0.5], np.float32), np.zeros(1, np.float32), np.zeros(1, np.float32)
    bc1, bc2 = zo.adam_bias_corrections(0.9, 0.999, 1)
    be.adamUpdate(w1, np.array([0.1], np.float32), m1, v1, 1e-3, 0.9, 0.999, 1e-8, bc1, bc2)
    assert abs(w1[0] - 0.499) < 1e-6


def test_rmsprop_update(be):
    """Backend.rmspropUpdate (src/backend.zig:446-456, :2774-2783): bit-exact, NaN and clamp cases included,
    on a length that takes the scalar kernel and one that takes the 16-byte kernel."""
    rng = np.random.default_rng(19)
    for n in (100003, 1 << 16):
        w = rng.standard_normal(n).astype(np.float32) * 40
        g = rng.standard_normal(n).astype(np.float32) * 4
        g[::97] = np.nan
        g[5::101] = 77.0
        ga = np.abs(rng.standard_normal(n)).astype(np.float32) * 0.01
        for lr, rho, eps in [(1e-3, 0.9, 1e-8), (0.5, 0.5, 1e-3)]:
            ww, gg = zo.rmsprop_update(w, g, ga, lr, rho, eps)
            gw, gga = w.copy(), ga.copy()
            be.rmspropUpdate(gw, g, gga, lr, rho, eps)
            assert np.array_equal(gga, gg) and np.array_equal(gw, ww)
    # known answer from the formula: w 1, g 0.1, lr 1e-3 -> 1 - 1e-4/(sqrt(1e-3)+1e-8)
    w1, s1 = np.array([1.0], np.float32), np.zeros(1, np.float32)
    be.rmspropUpdate(w1, np.array([0.1], np.float32), s1, 1e-3, 0.9, 1e-8)
    assert abs(w1[0] - 0.99683772) < 1e-6 and abs(s1[0] - 1e-3) < 1e-9


def test_evaluate_classification(be):
    """metrics.evaluateClassification (src/metrics.zig:85-163, :213-264): the confusion matrix is integer work
    and must be identical; the four ratios are f32 expressions of it, formed in the same order."""
    o = np.array([[0.9, 0.05, 0.05], [0.1, 0.8, 0.1], [0.3, 0.3, 0.4], [0.6, 0.3, 0.1], [0.2, 0.2, 0.6], [0.5, 0.5, 0.0]], np.float32)
    t = np.eye(3, dtype=np.float32)[[0, 1, 2, 1, 2, 1]]
    cm, m = be.evaluateClassification(o, t, 3)
    assert np.array_equal(cm, [[1, 0, 0], [2, 1, 0], [0, 0, 2]])
    assert abs(m["accuracy"] - 2 / 3) < 1e-6 and abs(m["precision"] - 7 / 9) < 1e-6 and abs(m["f1_score"] - 7 / 9) < 1e-6
    rng = np.random.default_rng(23)
    for rows, cols, classes in [(1, 2, 2), (150, 3, 3), (4099, 10, 10), (2048, 100, 100), (5000, 40, 64), (777, 1000, 1000)]:
        o = rng.standard_normal((rows, cols)).astype(np.float32)
        o[rng.integers(0, rows, rows // 5), rng.integers(0, cols, rows // 5)] = 3.0     # ties between maxima
        o[rng.integers(0, rows, rows // 7), rng.integers(0, cols, rows // 7)] = 3.0
        o[rng.integers(0, rows, max(rows // 50, 1)), rng.integers(0, cols, max(rows // 50, 1))] = np.nan
        o[rng.integers(0, rows, max(rows // 60, 1)), 0] = np.nan
        t = np.eye(cols, dtype=np.float32)[rng.integers(0, cols, rows)]
        t[rng.integers(0, rows, max(rows // 40, 1))] = 0.25                             # no entry above 0.5 -> class 0
        rc, wcm, wm = zo.evaluate_classification(o, t, classes)
        assert rc == 0
        cm, m = be.evaluateClassification(o, t, classes)
        assert np.array_equal(cm, wcm), (rows, cols)
        got = np.array([m["accuracy"], m["precision"], m["recall"], m["f1_score"]], np.float32)
        assert np.array_equal(got, wm), (rows, cols, got, wm)
        assert int(cm.sum()) == rows
    # device-resident operands
    do, dt = be.tensor(o), be.tensor(t)
    cm2, _ = be.evaluateClassification(do, dt, classes, rows=rows)
    assert np.array_equal(cm2, wcm)
    do.free(), dt.free()
    with pytest.raises(zn.ZnError) as ei:                      # error.InvalidClass
        be.evaluateClassification(np.array([[0.1, 0.2, 0.9]], np.float32), np.array([[1, 0, 0]], np.float32), 2)
    assert ei.value.status == 1          # ZN_ERR_INVALID_VALUE
    with pytest.raises(zn.ZnError) as ei:                      # error.EmptyInput
        be.evaluateClassification(np.zeros((0, 3), np.float32), np.zeros((0, 3), np.float32), 3)
    assert ei.value.status == 7


def test_clip_grad_norm(be):
    rng = np.random.default_rng(10)
    grads = [rng.standard_normal(s).astype(np.float32) for s in (20 * 4, 20, 200 * 100 + 3, 1)]
    want = [g.copy() for g in grads]
    wn, wf = zo.clip_grad_norm(want)
    norm, fac = be.clipGradNorm(grads)
    assert abs(norm - wn) <= 1e-5 * wn and abs(fac - wf) <= 1e-5 * wf
    for a, b in zip(grads, want):
        assert_close(a, b, 1e-5)
    small = [np.full(4, 0.1, np.float32)]
    norm, fac = be.clipGradNorm(small)
    assert fac == 1.0 and np.array_equal(small[0], np.full(4, 0.1, np.float32))


def test_device_resident_operands(be):
    """Device handles in place of host slices: nothing is copied per op."""
    be.set_precision(P.FP32_EXACT)
    rng = np.random.default_rng(12)
    m, n, k = 96, 48, 40
    a, b = rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    da, db, dbias, dc = be.tensor(a), be.tensor(b), be.tensor(bias), be.tensor(m * n)
    be.beginCommandBatch()
    be.matMul(da, db, dc, m, n, k)
    be.addBias(dc, dbias)
    be.activationForward(zn.Activation.relu, dc, dc)
    be.endCommandBatch()
    want = zo.activation_forward(zo.RELU, zo.add_bias(zo.matmul(a, b, m, n, k), bias))
    assert np.array_equal(dc.numpy((m, n)), want)
    for t in (da, db, dbias, dc):
        t.free()


def test_argument_errors(be):
    a = np.zeros(4, np.float32)
    with pytest.raises(zn.ZnError) as ei:
        be.matMul(a, a, a, 0, 2, 2)
    assert ei.value.status == 7          # ZN_ERR_SHAPE
    with pytest.raises(zn.ZnError):
        be.addBias(np.zeros(5, np.float32), np.zeros(2, np.float32))
    with pytest.raises(zn.ZnError):
        be.matMul(None, a, a, 2, 2, 1)


_FORCED_KERNEL_SNIPPET = r"""
import sys
import numpy as np
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
import zigneuron_b200 as zn
from util import assert_close, round_bf16, trunc_tf32
be = zn.Backend(0)
rng = np.random.default_rng(11)
for prec, rnd in ((zn.Precision.BF16_TC, round_bf16), (zn.Precision.TF32_TC, trunc_tf32)):
    be.set_precision(prec)
    for m, n, k in [(256, 512, 256), (300, 200, 100), (1024, 512, 784), (2048, 1024, 512), (300, 520, 1100), (513, 260, 96)]:
        a, b = rnd(rng.standard_normal((m, k)).astype(np.float32)), rnd(rng.standard_normal((k, n)).astype(np.float32))
        bias = rng.uniform(-0.1, 0.1, n).astype(np.float32)
        want = a.astype(np.float64) @ b.astype(np.float64)
        c = np.zeros((m, n), np.float32)
        be.matMul(a, b, c, m, n, k)
        assert_close(c, want, 1e-5, f"NN {{prec.name}} {{(m, n, k)}}")
        be.matMulTransposeB(a, np.ascontiguousarray(b.T), c, m, n, k)
        assert_close(c, want, 1e-5, f"NT {{prec.name}} {{(m, n, k)}}")
        be.matMulTransposeA(np.ascontiguousarray(a.T), b, c, m, n, k)
        assert_close(c, want, 1e-5, f"TN {{prec.name}} {{(m, n, k)}}")
        be.matMulBiasRelu(a, b, bias, c, m, n, k)
        assert_close(c, np.maximum(want + bias, 0), 1e-5, f"bias+relu {{prec.name}} {{(m, n, k)}}")
        c[:] = 1.0
        be.matMul(a, b, c, m, n, k, accumulate=True)
        assert_close(c, want + 1.0, 1e-5, f"accumulate {{prec.name}} {{(m, n, k)}}")
print("forced-kernel checks ok")
"""


@pytest.mark.parametrize("env", [{"ZN_TC_PAIR": "2"}, {"ZN_TC_PAIR": "2", "ZN_TC_STAGED_STORE": "1"}, {"ZN_TC_PAIR": "0"},
                                 {"ZN_TC_PAIR": "0", "ZN_TC_NARROW": "0"}, {"ZN_TC_PAIR": "0", "ZN_TC_NARROW": "2"},
                                 {"ZN_TC_PAIR": "0", "ZN_TC_NARROW": "2", "ZN_TC_STAGED_STORE": "0"},
                                 {"ZN_TC_PAIR": "2", "ZN_TC_PAIR8": "2"}],
                         ids=["two-CTA everywhere", "two-CTA with staged TMA stores", "one-CTA everywhere",
                              "one-CTA, 256-column tiles only", "one-CTA, 128-column tiles only",
                              "one-CTA, 128-column tiles, per-thread stores", "two-CTA with 8 epilogue warps"])
def test_each_tensor_core_kernel_on_shapes_the_default_routes_elsewhere(env):
    """The library picks the one-CTA or the two-CTA kernel and the one-CTA kernel's tile width by shape, and the
    two-CTA kernel's shared-memory-staged bulk-store epilogue is an option.  The choices are read once per process, so each forced combination runs in a
    process of its own, over shapes (ragged edges included) that the default routing would send to the other kernel."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = _FORCED_KERNEL_SNIPPET.format(root=root, tests=os.path.join(root, "tests"))
    r = subprocess.run([sys.executable, "-c", code], env={**os.environ, **env}, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "forced-kernel checks ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]

