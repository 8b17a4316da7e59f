"""Checks at the full sizes of the benchmark configurations, where the CPU oracle would take hours.  They rest on
properties that do not depend on the size:

* a product of small-integer matrices is exact in every precision mode (bf16 and tf32 hold the integers, fp32
  accumulation holds the sums), so its row and column sums must EQUAL what two matrix-vector products in int64 give:
  1^T (A B) = (1^T A) B and (A B) 1 = A (B 1) -- a checksum of checksums over all 67 M outputs;
* the training step is deterministic: two runs from the same weights end bit for bit alike, although tiles are
  handed to CTAs dynamically and four streams overlap;
* the bias gradient of a linear MSE output layer is the column sum of 2 (o - t) / n of the step's own forward
  output; a saved and reloaded network computes the same outputs to the bit; the loss goes down."""
import numpy as np
import pytest

import zigneuron_b200 as zn

pytestmark = pytest.mark.gpu

P = zn.Precision
WIDE = [(4096, 8192), (8192, 8192), (8192, 8192), (8192, 4096)]
WIDE_ACTS = ["relu", "relu", "relu", "linear"]


@pytest.fixture(scope="module")
def be():
    b = zn.Backend(0)
    yield b
    b.deinit()


@pytest.mark.parametrize("prec", [P.BF16_TC, P.TF32_TC, P.FP32_SIMT])
@pytest.mark.parametrize("orient", ["NN", "NT", "TN"])
def test_integer_gemm_checksums_at_layer_size(be, prec, orient):
    """8192 x 8192 x 4096: the forward product of the wide MLP's first layer at batch 8192 and, as TN / NT, the
    shapes of its gradient products."""
    m, n, k = 8192, 8192, 4096
    rng = np.random.default_rng(40)
    a = rng.integers(-4, 5, (m, k)).astype(np.float32)        # |sum| <= 4096 * 16 = 2^16: exact in fp32
    b = rng.integers(-4, 5, (k, n)).astype(np.float32)
    be.set_precision(prec)
    c = np.empty((m, n), np.float32)
    if orient == "NN":
        be.matMul(a, b, c, m, n, k)
    elif orient == "NT":
        be.matMulTransposeB(a, np.ascontiguousarray(b.T), c, m, n, k)      # B stored [n][k]
    else:
        be.matMulTransposeA(np.ascontiguousarray(a.T), b, c, m, n, k)      # A stored [k][m]
    ai, bi = a.astype(np.int64), b.astype(np.int64)
    ci = c.astype(np.int64)
    assert np.array_equal(ci.astype(np.float32), c)                        # every output is an integer
    assert np.array_equal(ci.sum(axis=1), ai @ bi.sum(axis=1))
    assert np.array_equal(ci.sum(axis=0), ai.sum(axis=0) @ bi)
    # and a few hundred outputs directly
    rows, cols = rng.integers(0, m, 256), rng.integers(0, n, 256)
    assert np.array_equal(ci[rows, cols], np.einsum("ik,ki->i", ai[rows], bi[:, cols]))


def _wide_net(be, prec, seed_weights=None):
    net = zn.Network(be, prec)
    for (i, o), act in zip(WIDE, WIDE_ACTS):
        net.addDense(i, o, act)
    if seed_weights is not None:
        for li, (w, b) in enumerate(seed_weights):
            net.setWeights(li, w, b)
    return net


def test_wide_mlp_step_properties_at_full_width(be, tmp_path):
    """The 4096-8192-8192-8192-4096 network at batch 2048 in bf16 (201 M parameters)."""
    B = 2048
    rng = np.random.default_rng(41)
    x = rng.standard_normal((B, 4096)).astype(np.float32)
    t = rng.standard_normal((B, 4096)).astype(np.float32)
    first = _wide_net(be, P.BF16_TC)
    weights = [first.getWeights(i) for i in range(4)]
    out0 = first.forward(x)
    losses = [first.trainStep(x, t, 1e-2, zn.Loss.mse) for _ in range(3)]
    # the loss reported by a step is that of the forward output before the update
    assert abs(losses[0] - float(np.mean((out0.astype(np.float64) - t) ** 2))) <= 1e-3 * losses[0]
    assert losses[2] < losses[1] < losses[0]
    # bias gradient of the linear output layer = column sums of the loss gradient of the LAST step's output
    again = _wide_net(be, P.BF16_TC, weights)
    for _ in range(2):
        again.trainStep(x, t, 1e-2, zn.Loss.mse)
    out2 = again.forward(x)
    again.trainStep(x, t, 1e-2, zn.Loss.mse)
    gb = again.getGrads(3)[1]
    factor = again.lastClip()[1]
    want = (2.0 * (out2.astype(np.float64) - t) / (B * 4096)).sum(axis=0) * factor
    assert np.abs(gb - want).max() <= 2e-2 * np.abs(want).max()       # the gradient block is held in bf16
    # determinism: the second network went through the same three steps from the same weights
    for i in range(4):
        (w1, b1), (w2, b2) = first.getWeights(i), again.getWeights(i)
        assert np.array_equal(w1, w2) and np.array_equal(b1, b2), i
    # save / load: the same outputs to the bit
    path = tmp_path / "wide.znn"
    first.save(path)
    loaded = zn.Network.load(be, path, P.BF16_TC)
    assert np.array_equal(loaded.forward(x), first.forward(x))
    for n_ in (first, again, loaded):
        n_.deinit()
