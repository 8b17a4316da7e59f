"""Pins the CPU oracle against the known-answer values of the reference's own
unit tests (tests/golden/reference_kat.json) and against closed-form checks of
the parts no reference test pins."""
import json
import os

import numpy as np

from oracle import zn_oracle as zo

KAT = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kat.json")))
ACT = {"relu": zo.RELU, "linear": zo.LINEAR, "sigmoid": zo.SIGMOID, "tanh": zo.TANH}


def f32(x):
    return np.asarray(x, dtype=np.float32)


def test_matmul_nn_golden():
    for case in KAT["matmul_nn"]:
        m, n, k = case["m"], case["n"], case["k"]
        if "a" in case:
            a, b = f32(case["a"]), f32(case["b"])
        elif "a_fill" in case:
            a, b = np.full(m * k, case["a_fill"], np.float32), np.full(k * n, case["b_fill"], np.float32)
        else:
            a = f32([(i % 10) / 10.0 for i in range(m * k)])
            b = f32([((i + 1) % 10) / 10.0 for i in range(k * n)])
        c = zo.matmul(a, b, m, n, k).reshape(-1)
        if "expected" in case:
            assert np.allclose(c, f32(case["expected"]), atol=case["tol"], rtol=0)
        elif "expected_fill" in case:
            assert np.allclose(c, case["expected_fill"], atol=case["tol"], rtol=0)
        else:
            want = sum(a[p] * b[p * n] for p in range(k))
            assert abs(c[0] - want) < case["tol"]
            assert abs(c[0] - case["expected_first"]) < case["tol"]


def test_dense_forward_backward_golden():
    for case in KAT["dense_forward"]:
        net = zo.Net()
        net.add_dense(case["in"], case["out"], ACT[case["act"]])
        net.set_params(0, f32(case["W"]), f32(case["b"]))
        y = net.forward(f32(case["x"]), 1).reshape(-1)
        assert np.allclose(y, f32(case["expected"]), atol=case["tol"], rtol=0), case["cite"]
    for case in KAT["dense_backward"]:
        # Dense.backward: G = dY * act'(y); dX = G . W^T
        g = zo.activation_backward(ACT[case["act"]], f32(case["y"]), f32(case["grad_out"]))
        dx = zo.matmul_transpose_b(g, f32(case["W"]), 1, case["in"], case["out"]).reshape(-1)
        assert np.allclose(dx, f32(case["expected_dx"]), atol=case["tol"], rtol=0)


def test_relu_golden():
    for case in KAT["relu_forward"]:
        x = f32(case["x"]) if "x" in case else f32([i / 2.0 - 2.5 for i in range(case["n"])])
        want = f32(case["expected"]) if "expected" in case else np.where(x > 0, x, 0)
        assert np.allclose(zo.activation_forward(zo.RELU, x), want, atol=case["tol"], rtol=0)
    for case in KAT["relu_backward"]:
        got = zo.activation_backward(zo.RELU, f32(case["y"]), f32(case["grad_out"]))
        assert np.allclose(got, f32(case["expected"]), atol=case["tol"], rtol=0)


def test_loss_golden():
    for case in KAT["mse_forward"]:
        got = zo.loss_forward(zo.MSE, f32(case["o"]), f32(case["t"]), 1, len(case["o"]))
        assert abs(got - case["expected"]) < case["tol"]
    for case in KAT["mse_backward"]:
        if "o" in case:
            o, t = f32(case["o"]), f32(case["t"])
        else:
            o = f32([i / 2.0 for i in range(case["n"])])
            t = f32([(i + 5) / 2.0 for i in range(case["n"])])
        got = zo.loss_backward(zo.MSE, o, t, 1, o.size).reshape(-1)
        assert np.allclose(got, f32(case["expected"]), atol=case["tol"], rtol=0)
    for case in KAT["ce_backward"]:
        got = zo.loss_backward(zo.CE_LOGITS, f32(case["logits"]), f32(case["t"]), 1, 2).reshape(-1)
        assert np.allclose(got, f32(case["expected"]), atol=case["tol"], rtol=0)


def test_remaining_losses_golden():
    kat = KAT["losses_n2"]
    for case in kat["ce_forward"]:
        got = zo.loss_forward(zo.CE, f32(case["o"]), f32(case["t"]), 1, len(case["o"]))
        assert abs(got - case["expected"]) < case["tol"] and 0 <= got < 1.0
    for case in kat["ce_backward"]:
        got = zo.loss_backward(zo.CE, f32(case["o"]), f32(case["t"]), 1, len(case["o"])).reshape(-1)
        assert np.allclose(got, f32(case["expected"]), atol=case["tol"], rtol=0)
    for case in kat["bce_forward"]:
        got = zo.loss_forward(zo.BCE, f32(case["o"]), f32(case["t"]), 1, len(case["o"]))
        assert abs(got - case["expected"]) < case["tol"] and 0 <= got < 0.1
    for case in kat["bce_backward"]:
        got = zo.loss_backward(zo.BCE, f32(case["o"]), f32(case["t"]), 1, len(case["o"])).reshape(-1)
        assert np.allclose(got, f32(case["expected"]), atol=case["tol"], rtol=0)
    # degenerate inputs of crossEntropyForward give 0 (src/loss.zig:126-129, :144-146, :166-167)
    assert zo.loss_forward(zo.CE, np.full(3, -np.inf, np.float32), f32([1, 0, 0]), 1, 3) == 0.0
    assert zo.loss_forward(zo.CE, f32([1, 2, 3]), f32([0, 0, 0]), 1, 3) == 0.0
    # two entries above 0.5: the mean of their losses
    o = f32([0.5, -1.0, 2.0])
    lse = np.log(np.exp(o - 2.0).sum()) + 2.0
    got = zo.loss_forward(zo.CE, o, f32([1, 0, 1]), 1, 3)
    assert abs(got - ((lse - 0.5) + (lse - 2.0)) / 2) < 1e-6
    # BCE clamps probabilities to [1e-7, 1 - 1e-7]
    got = zo.loss_forward(zo.BCE, f32([0.0, 1.0]), f32([1.0, 0.0]), 1, 2)
    one_minus = np.float32(1.0) - (np.float32(1.0) - np.float32(1e-7))      # 1.19e-7 in f32, not 1e-7
    assert abs(got - (-np.log(np.float32(1e-7)) - np.log(one_minus)) / 2) < 1e-5


def test_optimizer_golden():
    for case in KAT["sgd"]:
        got = zo.sgd_update(f32(case["w"]), f32(case["g"]), case["lr"])
        assert np.allclose(got, f32(case["expected"]), atol=case["tol"], rtol=0), case["cite"]
    for case in KAT["adam"]:
        bc1, bc2 = zo.adam_bias_corrections(case["beta1"], case["beta2"], case["t"])
        w, m, v = zo.adam_update(f32(case["w"]), f32(case["g"]), np.zeros(1, np.float32), np.zeros(1, np.float32),
                                 case["lr"], case["beta1"], case["beta2"], case["eps"], bc1, bc2)
        assert np.allclose(w, f32(case["expected"]), atol=case["tol"], rtol=0)
        assert w[0] < case["w"][0]
    for case in KAT["sgd_momentum"]:
        w, vel = f32(case["w"]), np.zeros(len(case["w"]), np.float32)
        for step in case["steps"]:
            w, vel = zo.sgd_momentum_update(w, f32(step["g"]), vel, case["lr"], case["momentum"])
            assert np.allclose(w, f32(step["expected"]), atol=step["tol"], rtol=0), case["cite"]
    for case in KAT["rmsprop"]:
        w, ga = zo.rmsprop_update(f32(case["w"]), f32(case["g"]), np.zeros(1, np.float32),
                                  case["lr"], case["rho"], case["eps"])
        assert np.allclose(w, f32(case["expected"]), atol=case["tol"], rtol=0), case["cite"]
        assert np.allclose(ga, f32(case["expected_g_avg"]), rtol=1e-6)


def test_adamw_is_adam_then_decoupled_decay():
    """AdamW.step (src/optimizer.zig:273-297): Adam's update without the L2 term, then w *= 1 - lr*wd on
    weights and bias alike."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((8, 5)).astype(np.float32)
    t = rng.standard_normal((8, 3)).astype(np.float32)
    w0 = (rng.standard_normal((5, 3)) * 0.3).astype(np.float32)
    b0 = (rng.standard_normal(3) * 0.1).astype(np.float32)
    lr, wd = 0.01, 0.1
    nets = []
    for kind in ("adam", "adamw"):
        net = zo.Net()
        net.add_dense(5, 3, zo.TANH)
        net.set_params(0, w0, b0)
        (net.set_adam(0, 0.9, 0.999, 1e-8, 0.0) if kind == "adam" else net.set_adamw(0, 0.9, 0.999, 1e-8, wd))
        net.train_step(x, t, 8, lr, zo.MSE)
        nets.append(net.get_params(0))
    (wa, ba), (ww, bw) = nets
    mul = np.float32(1.0) - np.float32(lr) * np.float32(wd)
    assert np.array_equal(ww, wa * mul) and np.array_equal(bw, ba * mul)


def test_remaining_activations_golden():
    kat = KAT["activations_n2"]
    for case in kat["softmax"]:
        y = zo.activation_forward(zo.SOFTMAX, f32(case["x"]))
        assert np.allclose(y, f32(case["expected"]), atol=case["tol"], rtol=0)
        assert abs(float(y.sum()) - 1.0) < 1e-3 and y[2] > y[1] > y[0]
    for case in kat["softmax_backward"]:
        gi = zo.activation_backward(zo.SOFTMAX, f32(case["s"]), f32(case["g"]))
        assert np.allclose(gi, f32(case["expected"]), atol=case["tol"], rtol=0) and abs(float(gi.sum())) < 1e-4
    ids = {"leaky_relu": zo.LEAKY_RELU, "elu": zo.ELU, "gelu": zo.GELU}
    for case in kat["pointwise"]:
        y = zo.activation_forward(ids[case["act"]], f32(case["x"]))
        assert np.allclose(y, f32(case["forward"]), atol=case["tol"], rtol=0), case["cite"]
        if "backward_at_y_g1" in case:
            gi = zo.activation_backward(ids[case["act"]], y, np.ones_like(y))
            assert np.allclose(gi, f32(case["backward_at_y_g1"]), atol=case["tol"], rtol=0), case["cite"]
    # gelu's derivative is the analytic one evaluated at y (src/activation.zig:139-150): check it against
    # a float64 evaluation of the same formula
    y = np.linspace(-3, 3, 41).astype(np.float32)
    c, k = 0.7978845608, 0.044715
    yd = y.astype(np.float64)
    th = np.tanh(c * (yd + k * yd ** 3))
    want = 0.5 * (1 + th) + 0.5 * yd * (1 - th * th) * c * (1 + 3 * k * yd * yd)
    got = zo.activation_backward(zo.GELU, y, np.full_like(y, 2.0))
    assert np.allclose(got, 2.0 * want, atol=2e-6, rtol=0)
    # all inputs -inf: x - max is NaN, the sum is not > 0, the result is uniform (src/activation.zig:69-77)
    y = zo.activation_forward(zo.SOFTMAX, np.full(4, -np.inf, np.float32))
    assert np.allclose(y, 0.25)


def test_classification_metrics_golden():
    for case in KAT["classification_metrics"]:
        o = f32(case["outputs"])
        t = np.eye(case["classes"], dtype=np.float32)[case["true"]]
        rc, cm, m = zo.evaluate_classification(o, t, case["classes"])
        assert rc == 0 and np.array_equal(cm, np.array(case["confusion"], np.uint64))
        want = [case[k] for k in ("accuracy", "precision", "recall", "f1_score")]
        assert np.allclose(m, want, atol=case["tol"], rtol=0)
    # error.EmptyInput and error.InvalidClass (src/metrics.zig:92, :105-110)
    assert zo.evaluate_classification(np.zeros((0, 3), np.float32), np.zeros((0, 3), np.float32), 3)[0] == 1
    o = np.array([[0.1, 0.2, 0.9]], np.float32)
    assert zo.evaluate_classification(o, np.array([[1, 0, 0]], np.float32), 2)[0] == 2
    # no target above 0.5 counts as class 0; a NaN in front pins the prediction to class 0
    rc, cm, _ = zo.evaluate_classification(np.array([[np.nan, 5.0], [1.0, np.nan]], np.float32),
                                           np.array([[0.2, 0.3], [0.0, 1.0]], np.float32), 2)
    assert rc == 0 and np.array_equal(cm, [[1, 0], [1, 0]])


def test_three_gemm_orientations_agree():
    rng = np.random.default_rng(7)
    m, n, k = 13, 9, 21
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    nn = zo.matmul(a, b, m, n, k)
    nt = zo.matmul_transpose_b(a, np.ascontiguousarray(b.T), m, n, k)
    tn = zo.matmul_transpose_a(np.ascontiguousarray(a.T), b, m, n, k)
    for got in (nn, nt, tn):
        assert np.allclose(got, ref, atol=1e-4)
    # NT and TN walk k in the same order with the same multiply-then-add, so they agree exactly.
    assert np.array_equal(nt, tn)
    acc = zo.matmul(a, b, m, n, k, c=np.ones((m, n), np.float32), accumulate=True)
    assert np.allclose(acc, ref + 1, atol=1e-4)


def test_clamps_and_nan():
    w = zo.sgd_update(f32([0.0, 0.0, 99.99, 0.0]), f32([100.0, -100.0, -5.0, np.nan]), 1.0)
    assert np.allclose(w, f32([-5.0, 5.0, 100.0, 0.0]))
    b = zo.sgd_update_bias(f32([49.0, -49.0]), f32([-5.0, 5.0]), 1.0)
    assert np.allclose(b, f32([50.0, -50.0]))
    w, m, v = zo.adam_update(f32([1.0]), f32([np.nan]), f32([0.0]), f32([0.0]), 0.1, 0.9, 0.999, 1e-8, 0.1, 0.001)
    assert w[0] == 1.0 and m[0] == 0.0 and v[0] == 0.0


def test_grad_clip():
    g1, g2 = f32([3.0, 0.0]), f32([4.0])
    norm, fac = zo.clip_grad_norm([g1, g2])
    assert abs(norm - 5.0) < 1e-6 and abs(fac - 1.0 / (5.0 + 1e-6)) < 1e-7
    assert np.allclose(np.concatenate([g1, g2]), f32([0.6, 0.0, 0.8]), atol=1e-6)
    g = f32([0.5, 0.5])
    norm, fac = zo.clip_grad_norm([g])
    assert fac == 1.0 and np.array_equal(g, f32([0.5, 0.5]))


def test_ce_rows_and_loss_value():
    logits = f32([[0.0, 0.0], [2.0, 0.0]])
    t = f32([[1.0, 0.0], [0.0, 1.0]])
    want = (np.log(2.0) + (np.log(np.exp(2.0) + 1.0) - 0.0)) / 2.0
    assert abs(zo.loss_forward(zo.CE_LOGITS, logits, t, 2, 2) - want) < 1e-6
    g = zo.loss_backward(zo.CE_LOGITS, logits, t, 2, 2)
    p = np.exp(2.0) / (np.exp(2.0) + 1.0)
    assert np.allclose(g, f32([[-0.5, 0.5], [p, (1 - p) - 1.0]]), atol=1e-6)


def test_distribute_round_robin():
    spans = [zo.distribute_round_robin(10, 4, i) for i in range(4)]
    assert spans == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [zo.distribute_round_robin(65536, 8, i) for i in (0, 7)] == [(0, 8192), (57344, 65536)]


def test_train_step_matches_numpy_float64():
    """One batched step of a 5-7-3 net against a float64 numpy derivation."""
    rng = np.random.default_rng(3)
    B, I, H, O = 6, 5, 7, 3
    x = rng.standard_normal((B, I)).astype(np.float32)
    t = np.eye(O, dtype=np.float32)[rng.integers(0, O, B)]
    W1 = (rng.uniform(-1, 1, (I, H)) * np.sqrt(2 / I)).astype(np.float32)
    W2 = (rng.uniform(-1, 1, (H, O)) * np.sqrt(1 / H)).astype(np.float32)
    b1, b2 = f32(rng.uniform(-0.1, 0.1, H)), f32(rng.uniform(-0.1, 0.1, O))
    net = zo.Net()
    net.add_dense(I, H, zo.RELU)
    net.add_dense(H, O, zo.LINEAR)
    net.set_params(0, W1, b1)
    net.set_params(1, W2, b2)
    lr = 0.05
    loss = net.train_step(x, t, B, lr, zo.CE_LOGITS)

    X, T = x.astype(np.float64), t.astype(np.float64)
    h = np.maximum(X @ W1 + b1, 0)
    z = h @ W2 + b2
    p = np.exp(z - z.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    want_loss = -np.log((p * T).sum(1)).mean()
    g2 = p - T
    gW2, gb2 = h.T @ g2, g2.sum(0)
    g1 = (g2 @ W2.T) * (h > 0)
    gW1, gb1 = X.T @ g1, g1.sum(0)
    norm = np.sqrt(sum((a ** 2).sum() for a in (gW1, gb1, gW2, gb2)))
    fac = 1.0 / (norm + 1e-6) if norm > 1 else 1.0
    assert abs(loss - want_loss) < 1e-5
    got_norm, got_fac = net.last_clip()
    assert abs(got_norm - norm) < 1e-4 and abs(got_fac - fac) < 1e-5
    W1n, b1n = net.get_params(0)
    W2n, b2n = net.get_params(1)
    assert np.allclose(W1n, W1 - lr * np.clip(gW1 * fac, -5, 5), atol=1e-5)
    assert np.allclose(b2n, b2 - lr * np.clip(gb2 * fac, -5, 5), atol=1e-5)
    assert np.allclose(W2n, W2 - lr * np.clip(gW2 * fac, -5, 5), atol=1e-5)
    assert np.allclose(b1n, b1 - lr * np.clip(gb1 * fac, -5, 5), atol=1e-5)


def test_per_sample_train_is_sequence_of_single_steps():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 3)).astype(np.float32)
    t = rng.standard_normal((4, 2)).astype(np.float32)
    W = rng.uniform(-0.5, 0.5, (3, 2)).astype(np.float32)
    a, b = zo.Net(), zo.Net()
    for n in (a, b):
        n.add_dense(3, 2, zo.LINEAR)
        n.set_params(0, W, np.zeros(2, np.float32))
        n.set_adam(0)
    ep = a.train(x, t, 2, 0.01, zo.MSE)
    losses = [[b.train_step(x[s], t[s], 1, 0.01, zo.MSE) for s in range(4)] for _ in range(2)]
    assert np.allclose(ep, [np.float32(sum(np.float32(v) for v in l)) / 4 for l in losses], rtol=1e-6)
    assert np.array_equal(a.get_params(0)[0], b.get_params(0)[0])


# ---- the oracle's curves on configurations 1 and 2 (tests/golden/config_curves.json) ---------------------------

def _curves():
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import configs as cfg
    return cfg, json.load(open(os.path.join(os.path.dirname(__file__), "golden", "config_curves.json")))


def _oracle_net(dims, acts, Ws, bs, adam):
    net = zo.Net()
    for i, ((a, b), act) in enumerate(zip(dims, acts)):
        net.add_dense(a, b, zo.RELU if act == "relu" else zo.LINEAR)
        net.set_params(i, Ws[i], bs[i])
        if adam:
            net.set_adam(i)
    return net


def test_config1_curves_are_the_oracles():
    """The committed 1000-step and 20-epoch curves of configuration 1 are what the oracle computes today, bit for bit."""
    cfg, curves = _curves()
    x, t, Ws, bs = cfg.iris_config()
    net = _oracle_net(cfg.IRIS_DIMS, cfg.IRIS_ACTS, Ws, bs, False)
    losses = [net.train_step(x, t, 150, 0.005, zo.CE_LOGITS) for _ in range(1000)]
    want = curves["config1"]["full_batch"]
    assert np.array_equal(np.array(losses, np.float32), np.array(want["loss"], np.float32))
    for i in range(3):
        assert np.array_equal(net.get_params(i)[0].ravel(), np.array(want["weights"][i]["w"], np.float32))
    assert losses[-1] < 0.05 * losses[0]
    net = _oracle_net(cfg.IRIS_DIMS, cfg.IRIS_ACTS, Ws, bs, False)
    epoch = net.train(x, t, 20, 0.005, zo.CE_LOGITS)
    assert np.array_equal(np.asarray(epoch, np.float32), np.array(curves["config1"]["per_sample"]["epoch_loss"], np.float32))


def test_config2_curve_starts_as_the_oracle_does():
    """Configuration 2 at its stated batch of 1024 costs the oracle seconds per step, so only the first two of the
    100 committed steps are recomputed here: loss, gradient norm, clip factor and the weight samples, bit for bit."""
    cfg, curves = _curves()
    x, t, Ws, bs = cfg.mlp784_config()
    net = _oracle_net(cfg.MLP784_DIMS, cfg.MLP784_ACTS, Ws, bs, True)
    want = curves["config2"]
    assert len(want["loss"]) == 100 and want["loss"][-1] < 0.2 * want["loss"][0]
    for step in (1, 2):
        loss = net.train_step(x, t, 1024, 1e-3, zo.CE_LOGITS)
        norm, factor = net.last_clip()
        assert np.float32(loss) == np.float32(want["loss"][step - 1])
        assert np.float32(norm) == np.float32(want["norm"][step - 1]) and np.float32(factor) == np.float32(want["factor"][step - 1])
        for i in range(3):
            W, b = net.get_params(i)
            snap = want["snapshots"][str(step)][i]
            assert np.array_equal(W.ravel()[cfg.snapshot_indices(W.size)], np.array(snap["w"], np.float32))
            assert np.array_equal(b[:10], np.array(snap["b"], np.float32))
