"""Seeded inputs and weights of the benchmark configurations at the sizes they state, shared by the script that
writes the oracle's curves (make_config_curves.py) and by the tests that read them.  Everything comes from
numpy's Generator(PCG64), whose streams do not change between numpy releases.

Synthetic data stands in for the datasets the configurations are shaped after: Gaussian clusters of the Iris
table's shape (150 x 4, 3 classes x 50) and U[0,1) rows of MNIST's width (784)."""
import numpy as np

IRIS_DIMS, IRIS_ACTS = [(4, 20), (20, 10), (10, 3)], ["relu", "relu", "linear"]
MLP784_DIMS, MLP784_ACTS = [(784, 512), (512, 256), (256, 10)], ["relu", "relu", "linear"]
WIDE_DIMS, WIDE_ACTS = [(4096, 8192), (8192, 8192), (8192, 8192), (8192, 4096)], ["relu", "relu", "relu", "linear"]
SNAP_STEPS = (1, 2, 5, 10, 20, 50, 100)   # steps after which a sample of every layer's weights is kept
SNAP_VALUES = 64


def iris_config():
    """Config 1: 150 samples in 3 Gaussian clusters in R^4 (means U[-2,2], sigma 0.5, 50 per class, class-major),
    one-hot targets; weights U(-1,1)*scale(act) as Dense.init draws them (src/layer.zig:326-339), bias 0; seed 0."""
    rng = np.random.default_rng(0)
    means = rng.uniform(-2, 2, (3, 4))
    x = np.concatenate([means[c] + 0.5 * rng.standard_normal((50, 4)) for c in range(3)]).astype(np.float32)
    t = np.zeros((150, 3), np.float32)
    for c in range(3):
        t[50 * c:50 * (c + 1), c] = 1.0
    Ws, bs = [], []
    for (a, b), act in zip(IRIS_DIMS, IRIS_ACTS):
        scale = np.sqrt(2.0 / a) if act == "relu" else np.sqrt(1.0 / a)
        Ws.append((rng.uniform(-1, 1, (a, b)) * scale).astype(np.float32))
        bs.append(np.zeros(b, np.float32))
    return x, t, Ws, bs


def mlp784_config(batch=1024):
    """Config 2: X batch x 784 ~ U[0,1), labels uniform over 10 classes as one-hot rows, weights
    U(-1,1)*sqrt(2/(in+out)) (the Xavier-style branch of Dense.init, src/layer.zig:333-335), bias 0; seed 1."""
    rng = np.random.default_rng(1)
    x = rng.random((batch, 784), dtype=np.float32)
    t = np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)]
    Ws, bs = [], []
    for a, b in MLP784_DIMS:
        Ws.append(((rng.random((a, b), dtype=np.float32) * 2 - 1) * np.float32(np.sqrt(2.0 / (a + b)))).astype(np.float32))
        bs.append(np.zeros(b, np.float32))
    return x, t, Ws, bs


def wide_layer_weights(layer, seed=2):
    """Configs 3 and 4: fp32 master weights U(-1,1)*sqrt(2/in) (relu) or sqrt(1/in) (linear output layer)."""
    (a, b), act = WIDE_DIMS[layer], WIDE_ACTS[layer]
    rng = np.random.default_rng([seed, 100 + layer])
    w = rng.random((a, b), dtype=np.float32)
    w *= np.float32(2.0)
    w -= np.float32(1.0)
    w *= np.float32(np.sqrt((2.0 if act == "relu" else 1.0) / a))
    return w


def wide_rows(rows, seed=2):
    """Configs 3 and 4: inputs and targets ~ N(0,1), `rows` rows of each."""
    rng = np.random.default_rng([seed, 7])
    x = rng.standard_normal((rows, WIDE_DIMS[0][0]), dtype=np.float32)
    t = rng.standard_normal((rows, WIDE_DIMS[-1][1]), dtype=np.float32)
    return x, t


def snapshot_indices(count):
    return (np.arange(SNAP_VALUES, dtype=np.int64) * 7919) % count
