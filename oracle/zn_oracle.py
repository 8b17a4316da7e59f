"""ctypes front end of the CPU oracle (oracle/zn_oracle.c).

TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the CPU-baseline leg
of the benchmark import this module as the checker.  The product package
(zigneuron_b200) never does.

`build()` compiles oracle/zn_oracle.c with the Makefile beside it;
`load()` returns the shared object (building it first if it is missing).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libzn_oracle.so")

RELU, SIGMOID, TANH, SOFTMAX, LINEAR, GELU, LEAKY_RELU, ELU = range(8)
MSE, CE, CE_LOGITS, BCE, KL = range(5)

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_lib = None


def build(force=False):
    src = os.path.join(_HERE, "zn_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libzn_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_SO):
        build()
    lib = C.CDLL(_SO)
    sz, f, i, vp = C.c_size_t, C.c_float, C.c_int, C.c_void_p
    sig = {
        "zo_matmul": (None, [_f32p, _f32p, _f32p, sz, sz, sz, i]),
        "zo_matmul_transpose_a": (None, [_f32p, _f32p, _f32p, sz, sz, sz, i]),
        "zo_matmul_transpose_a_rows": (None, [_f32p, _f32p, _f32p, sz, sz, sz, sz, sz]),
        "zo_matmul_transpose_b": (None, [_f32p, _f32p, _f32p, sz, sz, sz, i]),
        "zo_add_bias": (None, [_f32p, sz, _f32p, sz]),
        "zo_accumulate_bias": (None, [_f32p, sz, _f32p, sz]),
        "zo_activation_forward": (None, [i, _f32p, _f32p, sz]),
        "zo_activation_backward": (None, [i, _f32p, _f32p, _f32p, sz]),
        "zo_mse_forward": (f, [_f32p, _f32p, sz]),
        "zo_mse_backward": (None, [_f32p, _f32p, _f32p, sz]),
        "zo_ce_logits_forward": (f, [_f32p, _f32p, sz]),
        "zo_ce_logits_backward": (None, [_f32p, _f32p, _f32p, sz]),
        "zo_loss_forward": (f, [i, _f32p, _f32p, sz, sz]),
        "zo_loss_backward": (None, [i, _f32p, _f32p, _f32p, sz, sz]),
        "zo_sgd_update": (None, [_f32p, _f32p, sz, f, f]),
        "zo_sgd_update_bias": (None, [_f32p, _f32p, sz, f]),
        "zo_adam_update": (None, [_f32p, _f32p, _f32p, _f32p, sz, f, f, f, f, f, f]),
        "zo_adam_bias_corrections": (None, [f, f, sz, C.POINTER(f), C.POINTER(f)]),
        "zo_clip_grad_norm": (f, [C.POINTER(vp), C.POINTER(sz), sz, C.POINTER(f)]),
        "zo_distribute_round_robin": (None, [sz, sz, sz, C.POINTER(sz), C.POINTER(sz)]),
        "zo_evaluate_classification": (i, [_f32p, _f32p, sz, sz, sz, np.ctypeslib.ndpointer(dtype=np.uint64, flags="C_CONTIGUOUS"), _f32p]),
        "zo_net_create": (vp, []),
        "zo_net_destroy": (None, [vp]),
        "zo_net_add_dense": (i, [vp, sz, sz, i]),
        "zo_net_layer_count": (sz, [vp]),
        "zo_net_set_params": (None, [vp, sz, _f32p, _f32p]),
        "zo_net_get_params": (None, [vp, sz, _f32p, _f32p]),
        "zo_net_get_grads": (None, [vp, sz, _f32p, _f32p]),
        "zo_net_set_grads": (None, [vp, sz, _f32p, _f32p]),
        "zo_net_set_sgd": (None, [vp, sz, f]),
        "zo_net_set_adam": (None, [vp, sz, f, f, f, f]),
        "zo_net_set_adamw": (None, [vp, sz, f, f, f, f]),
        "zo_net_set_sgd_momentum": (None, [vp, sz, f]),
        "zo_net_set_rmsprop": (None, [vp, sz, f, f, f]),
        "zo_rmsprop_update": (None, [_f32p, _f32p, _f32p, sz, f, f, f]),
        "zo_sgd_momentum_update": (None, [_f32p, _f32p, _f32p, sz, f, f]),
        "zo_net_forward": (None, [vp, _f32p, sz, _f32p]),
        "zo_net_train_step": (f, [vp, _f32p, _f32p, sz, f, i]),
        "zo_net_shard_gradients": (f, [vp, _f32p, _f32p, sz, sz, i]),
        "zo_net_clip_and_update": (None, [vp, f]),
        "zo_net_last_clip": (None, [vp, C.POINTER(f), C.POINTER(f)]),
        "zo_net_train": (None, [vp, _f32p, _f32p, sz, sz, f, i, _f32p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def matmul(a, b, m, n, k, c=None, accumulate=False):
    out = np.zeros((m, n), np.float32) if c is None else _c(c).copy()
    load().zo_matmul(_c(a), _c(b), out, m, n, k, int(accumulate))
    return out


def matmul_transpose_a(a, b, m, n, k, c=None, accumulate=False):
    out = np.zeros((m, n), np.float32) if c is None else _c(c).copy()
    load().zo_matmul_transpose_a(_c(a), _c(b), out, m, n, k, int(accumulate))
    return out


def matmul_transpose_b(a, b, m, n, k, c=None, accumulate=False):
    out = np.zeros((m, n), np.float32) if c is None else _c(c).copy()
    load().zo_matmul_transpose_b(_c(a), _c(b), out, m, n, k, int(accumulate))
    return out


def add_bias(out, bias):
    o = _c(out).copy()
    load().zo_add_bias(o, o.size, _c(bias), bias.size)
    return o


def accumulate_bias(grad_bias, g):
    gb = _c(grad_bias).copy()
    load().zo_accumulate_bias(gb, gb.size, _c(g), g.size)
    return gb


def activation_forward(act, x):
    x = _c(x)
    y = np.empty_like(x)
    load().zo_activation_forward(act, x, y, x.size)
    return y


def activation_backward(act, y, grad_out):
    y, g = _c(y), _c(grad_out)
    gi = np.empty_like(y)
    load().zo_activation_backward(act, y, g, gi, y.size)
    return gi


def loss_forward(loss, o, t, rows, cols):
    return float(load().zo_loss_forward(loss, _c(o), _c(t), rows, cols))


def loss_backward(loss, o, t, rows, cols):
    g = np.empty(rows * cols, np.float32)
    load().zo_loss_backward(loss, _c(o), _c(t), g, rows, cols)
    return g.reshape(rows, cols)


def sgd_update(w, g, lr, wd=0.0):
    w = _c(w).copy()
    load().zo_sgd_update(w.reshape(-1), _c(g).reshape(-1), w.size, lr, wd)
    return w


def sgd_update_bias(b, g, lr):
    b = _c(b).copy()
    load().zo_sgd_update_bias(b, _c(g), b.size, lr)
    return b


def adam_bias_corrections(beta1, beta2, t):
    a, b = C.c_float(), C.c_float()
    load().zo_adam_bias_corrections(beta1, beta2, t, C.byref(a), C.byref(b))
    return a.value, b.value


def adam_update(w, g, m, v, lr, beta1, beta2, eps, bc1, bc2):
    w, m, v = _c(w).copy(), _c(m).copy(), _c(v).copy()
    load().zo_adam_update(w.reshape(-1), _c(g).reshape(-1), m.reshape(-1), v.reshape(-1), w.size,
                          lr, beta1, beta2, eps, bc1, bc2)
    return w, m, v


def rmsprop_update(w, g, g_avg, lr, rho, eps):
    w, ga = _c(w).copy(), _c(g_avg).copy()
    load().zo_rmsprop_update(w.reshape(-1), _c(g).reshape(-1), ga.reshape(-1), w.size, lr, rho, eps)
    return w, ga


def sgd_momentum_update(w, g, vel, lr, momentum):
    w, v = _c(w).copy(), _c(vel).copy()
    load().zo_sgd_momentum_update(w.reshape(-1), _c(g).reshape(-1), v.reshape(-1), w.size, lr, momentum)
    return w, v


def evaluate_classification(outputs, targets, classes):
    """metrics.evaluateClassification: returns (status, confusion[classes, classes], [accuracy, precision, recall, f1])."""
    o, t = _c(outputs), _c(targets)
    rows = o.shape[0] if o.ndim == 2 else 0
    cols = o.shape[1] if o.ndim == 2 else 1
    cm = np.zeros((classes, classes), np.uint64)
    out = np.zeros(4, np.float32)
    rc = load().zo_evaluate_classification(o.reshape(-1) if rows else np.zeros(1, np.float32),
                                           t.reshape(-1) if rows else np.zeros(1, np.float32), rows, cols, classes, cm, out)
    return rc, cm, out


def clip_grad_norm(grads):
    """grads: list of float32 arrays, scaled IN PLACE; returns (norm, factor)."""
    lib = load()
    n = len(grads)
    ptrs = (C.c_void_p * n)(*[g.ctypes.data for g in grads])
    lens = (C.c_size_t * n)(*[g.size for g in grads])
    fac = C.c_float()
    norm = lib.zo_clip_grad_norm(ptrs, lens, n, C.byref(fac))
    return float(norm), fac.value


def distribute_round_robin(total, n, i):
    s, e = C.c_size_t(), C.c_size_t()
    load().zo_distribute_round_robin(total, n, i, C.byref(s), C.byref(e))
    return s.value, e.value


class Net:
    """Oracle network: the reference's Network restricted to Dense layers."""

    def __init__(self):
        self._lib = load()
        self._h = self._lib.zo_net_create()
        self.shapes = []

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.zo_net_destroy(self._h)
            self._h = None

    def add_dense(self, n_in, n_out, act):
        r = self._lib.zo_net_add_dense(self._h, n_in, n_out, act)
        if r < 0:
            raise ValueError("invalid layer size")
        self.shapes.append((n_in, n_out))
        return r

    def set_params(self, layer, W, b):
        self._lib.zo_net_set_params(self._h, layer, _c(W).reshape(-1), _c(b).reshape(-1))

    def get_params(self, layer):
        i, o = self.shapes[layer]
        W, b = np.empty(i * o, np.float32), np.empty(o, np.float32)
        self._lib.zo_net_get_params(self._h, layer, W, b)
        return W.reshape(i, o), b

    def get_grads(self, layer):
        i, o = self.shapes[layer]
        W, b = np.empty(i * o, np.float32), np.empty(o, np.float32)
        self._lib.zo_net_get_grads(self._h, layer, W, b)
        return W.reshape(i, o), b

    def set_grads(self, layer, gW, gb):
        self._lib.zo_net_set_grads(self._h, layer, _c(gW).reshape(-1), _c(gb).reshape(-1))

    def set_sgd(self, layer, weight_decay=0.0):
        self._lib.zo_net_set_sgd(self._h, layer, weight_decay)

    def set_adam(self, layer, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        self._lib.zo_net_set_adam(self._h, layer, beta1, beta2, eps, weight_decay)

    def set_adamw(self, layer, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        self._lib.zo_net_set_adamw(self._h, layer, beta1, beta2, eps, weight_decay)

    def set_sgd_momentum(self, layer, momentum):
        self._lib.zo_net_set_sgd_momentum(self._h, layer, momentum)

    def set_rmsprop(self, layer, rho=0.9, eps=1e-8, weight_decay=0.0):
        self._lib.zo_net_set_rmsprop(self._h, layer, rho, eps, weight_decay)

    def forward(self, x, rows):
        out = np.empty(rows * self.shapes[-1][1], np.float32)
        self._lib.zo_net_forward(self._h, _c(x).reshape(-1), rows, out)
        return out.reshape(rows, -1)

    def train_step(self, x, t, rows, lr, loss):
        return float(self._lib.zo_net_train_step(self._h, _c(x).reshape(-1), _c(t).reshape(-1), rows, lr, loss))

    def shard_gradients(self, x, t, rows, global_rows, loss):
        return float(self._lib.zo_net_shard_gradients(self._h, _c(x).reshape(-1), _c(t).reshape(-1),
                                                      rows, global_rows, loss))

    def clip_and_update(self, lr):
        self._lib.zo_net_clip_and_update(self._h, lr)

    def last_clip(self):
        a, b = C.c_float(), C.c_float()
        self._lib.zo_net_last_clip(self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def train(self, inputs, targets, epochs, lr, loss):
        samples = inputs.shape[0]
        out = np.zeros(epochs, np.float32)
        self._lib.zo_net_train(self._h, _c(inputs).reshape(-1), _c(targets).reshape(-1), samples, epochs, lr, loss, out)
        return out
