"""Shared helpers for the parity tests: seeded inputs, error norms, precision rounding."""
import numpy as np


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def rel_max(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def assert_close(got, want, tol, what=""):
    e2, em = rel_l2(got, want), rel_max(got, want)
    assert e2 <= tol and em <= tol, f"{what}: rel_l2={e2:.3e} rel_max={em:.3e} > {tol:.1e}"


def round_bf16(x):
    """Round-to-nearest-even to bfloat16, returned as float32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def trunc_tf32(x):
    """Drop the 13 low mantissa bits (values exactly representable in tf32)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return u.view(np.float32).reshape(np.shape(x))


def reference_init(rng, n_in, n_out, act):
    """Weights in the reference's distribution: U(-1,1) * scale(act) (src/layer.zig:330-338)."""
    if act in ("relu", "leaky_relu"):
        scale = np.sqrt(2.0 / n_in)
    elif act == "linear":
        scale = np.sqrt(1.0 / n_in)
    else:
        scale = np.sqrt(2.0 / (n_in + n_out))
    return (rng.uniform(-1, 1, (n_in, n_out)) * scale).astype(np.float32)


def iris_style(seed=0):
    """150 samples, 3 Gaussian clusters in R^4 (means U[-2,2], sigma 0.5, 50 per class), one-hot targets."""
    rng = np.random.default_rng(seed)
    means = rng.uniform(-2, 2, (3, 4))
    x = np.concatenate([means[c] + 0.5 * rng.standard_normal((50, 4)) for c in range(3)]).astype(np.float32)
    t = np.zeros((150, 3), np.float32)
    for c in range(3):
        t[50 * c:50 * (c + 1), c] = 1.0
    return x, t


def emulate_bf16_mse_step(x, t, Ws, bs, acts):
    """What a CORRECT bf16-operand / fp32-accumulate implementation of one MSE training step computes:
    float64 arithmetic with a bfloat16 rounding at every point where the GPU path stores an operand
    (input, weight copies, hidden activations, every gradient block).  Separates the kernel's own error
    from the rounding the precision mode implies.  Returns (loss, [gW], [gb])."""
    rb = round_bf16
    L = len(Ws)
    h = [rb(x)]
    for i in range(L):
        z = h[-1].astype(np.float64) @ rb(Ws[i]).astype(np.float64) + bs[i]
        if acts[i] == "relu":
            z = np.maximum(z, 0)
        z = z.astype(np.float32)
        h.append(rb(z) if i + 1 < L else z)          # the last output stays fp32
    n = h[-1].size
    d = h[-1].astype(np.float64) - t
    loss = float((d ** 2).sum() / n)
    g = rb((2 * (h[-1] - t) / np.float32(n)).astype(np.float32))
    gWs, gbs = [None] * L, [None] * L
    for i in range(L - 1, -1, -1):
        gWs[i] = (h[i].astype(np.float64).T @ g.astype(np.float64)).astype(np.float32)
        gbs[i] = g.astype(np.float64).sum(0).astype(np.float32)
        if i > 0:
            dx = g.astype(np.float64) @ rb(Ws[i]).astype(np.float64).T
            if acts[i - 1] == "relu":
                dx = dx * (h[i] > 0)
            g = rb(dx.astype(np.float32))
    return loss, gWs, gbs
