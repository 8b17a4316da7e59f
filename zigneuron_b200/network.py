"""Network: the reference's `Network` (src/network.zig) restricted to Dense
layers, resident on the GPU.  Names follow the reference: addDense, forward,
trainStep, train; per-layer optimizers as in `Network.optimizers`."""
import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from ._lib import check, lib, ptr
from .backend import Activation, Backend, Loss, Precision


@dataclass
class Sgd:                      # src/optimizer.zig:81-85; momentum > 0 ignores weight_decay, as Sgd.step does
    momentum: float = 0.0
    weight_decay: float = 0.0


@dataclass
class Adam:                     # src/optimizer.zig:169-184
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0


@dataclass
class AdamW:                    # src/optimizer.zig:236-250
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01


@dataclass
class Rmsprop:                  # src/optimizer.zig:311-320
    rho: float = 0.9
    eps: float = 1e-8
    weight_decay: float = 0.0


class Network:
    def __init__(self, backend: Backend, precision=None):
        self.backend = backend
        self.precision = Precision(precision if precision is not None else backend.precision)
        h = C.c_void_p()
        check(lib.zn_net_create(backend.handle, int(self.precision), C.byref(h)), backend.handle)
        self.handle = h.value
        self.shapes = []

    def deinit(self):
        if getattr(self, "handle", None) and self.backend.handle:
            lib.zn_net_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.deinit()
        except Exception:
            pass

    def _ck(self, status):
        check(status, self.backend.handle)

    # Network.addDense, src/network.zig:104-122
    def addDense(self, input_size, output_size, act):
        idx = C.c_int32()
        self._ck(lib.zn_net_add_dense(self.handle, input_size, output_size, int(Activation[act] if isinstance(act, str) else act),
                                      C.byref(idx)))
        self.shapes.append((input_size, output_size))
        return idx.value

    def setOptimizer(self, opt, layer=-1):
        if isinstance(opt, Adam):
            self._ck(lib.zn_net_set_adam(self.handle, layer, opt.beta1, opt.beta2, opt.eps, opt.weight_decay))
        elif isinstance(opt, AdamW):
            self._ck(lib.zn_net_set_adamw(self.handle, layer, opt.beta1, opt.beta2, opt.eps, opt.weight_decay))
        elif isinstance(opt, Rmsprop):
            self._ck(lib.zn_net_set_rmsprop(self.handle, layer, opt.rho, opt.eps, opt.weight_decay))
        elif isinstance(opt, Sgd):
            if opt.momentum > 0.0:
                self._ck(lib.zn_net_set_sgd_momentum(self.handle, layer, opt.momentum))
            else:
                self._ck(lib.zn_net_set_sgd(self.handle, layer, opt.weight_decay))
        else:
            raise TypeError(opt)

    def setWeights(self, layer, weights=None, bias=None):
        w = None if weights is None else np.ascontiguousarray(weights, np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, np.float32)
        self._ck(lib.zn_net_set_weights(self.handle, layer, ptr(w), ptr(b)))

    def getWeights(self, layer):
        i, o = self.shapes[layer]
        w, b = np.empty((i, o), np.float32), np.empty(o, np.float32)
        self._ck(lib.zn_net_get_weights(self.handle, layer, ptr(w), ptr(b)))
        return w, b

    def getGrads(self, layer):
        i, o = self.shapes[layer]
        w, b = np.empty((i, o), np.float32), np.empty(o, np.float32)
        self._ck(lib.zn_net_get_grads(self.handle, layer, ptr(w), ptr(b)))
        return w, b

    def getInputGrad(self, rows):
        g = np.empty((rows, self.shapes[0][0]), np.float32)
        self._ck(lib.zn_net_get_input_grad(self.handle, ptr(g), g.size))
        return g

    # Network.forward, src/network.zig:309
    def forward(self, input, rows=None):
        x = np.ascontiguousarray(input, np.float32)
        rows = rows if rows is not None else x.size // self.shapes[0][0]
        out = np.empty((rows, self.shapes[-1][1]), np.float32)
        self._ck(lib.zn_net_forward(self.handle, ptr(x), rows, ptr(out)))
        return out

    def evaluateClassification(self, input, target, num_classes, rows=None):
        """Network.forward on the block, then metrics.evaluateClassification (src/metrics.zig:239-264), on the device."""
        if isinstance(input, np.ndarray):
            input = np.ascontiguousarray(input, np.float32)
        if isinstance(target, np.ndarray):
            target = np.ascontiguousarray(target, np.float32)
        if rows is None:
            rows = input.size // self.shapes[0][0]
        cm = np.zeros((num_classes, num_classes), np.uint64)
        m = np.zeros(4, np.float32)
        self._ck(lib.zn_net_evaluate_classification(self.handle, ptr(input), ptr(target), rows, num_classes,
                                                    cm.ctypes.data, m.ctypes.data))
        return cm, dict(zip(("accuracy", "precision", "recall", "f1_score"), (float(v) for v in m)))

    # Network.trainStep, src/network.zig:481
    def trainStep(self, input, target, learning_rate, loss_fn, rows=None):
        if rows is None:
            rows = input.size // self.shapes[0][0]
        if isinstance(input, np.ndarray):
            input = np.ascontiguousarray(input, np.float32)
        if isinstance(target, np.ndarray):
            target = np.ascontiguousarray(target, np.float32)
        out = C.c_float()
        self._ck(lib.zn_net_train_step(self.handle, ptr(input), ptr(target), rows, learning_rate, int(loss_fn), C.byref(out)))
        return out.value

    def submitStep(self, host_input, host_target, rows, learning_rate, loss_fn):
        self._ck(lib.zn_net_submit_step(self.handle, ptr(host_input), ptr(host_target), rows, learning_rate, int(loss_fn)))

    def waitStep(self):
        out = C.c_float()
        self._ck(lib.zn_net_wait_step(self.handle, C.byref(out)))
        return out.value

    # Network.train, src/network.zig:596 (constant scheduler, no early stopping)
    def train(self, inputs, targets, epochs, learning_rate, loss_fn):
        x = np.ascontiguousarray(inputs, np.float32)
        t = np.ascontiguousarray(targets, np.float32)
        samples = x.shape[0]
        losses = np.zeros(epochs, np.float32)
        self._ck(lib.zn_net_train(self.handle, ptr(x), ptr(t), samples, epochs, learning_rate, int(loss_fn), ptr(losses)))
        return losses

    # Network.save / Network.load, src/network.zig:692-745 (the reference's .znn format)
    def save(self, path):
        self._ck(lib.zn_net_save(self.handle, os.fsencode(path)))

    def saveOptimizer(self, path):
        """Optimizer kind, hyper-parameters, step count and state tensors of every layer (not part of .znn)."""
        self._ck(lib.zn_net_save_optimizer(self.handle, os.fsencode(path)))

    def loadOptimizer(self, path):
        self._ck(lib.zn_net_load_optimizer(self.handle, os.fsencode(path)))

    @classmethod
    def load(cls, backend, path, precision=None):
        net = cls.__new__(cls)
        net.backend = backend
        net.precision = Precision(precision if precision is not None else backend.precision)
        h = C.c_void_p()
        check(lib.zn_net_load(backend.handle, int(net.precision), os.fsencode(path), C.byref(h)), backend.handle)
        net.handle = h.value
        net.shapes = []
        with open(path, "rb") as f:
            f.seek(8)
            count = int.from_bytes(f.read(4), "little")
            for _ in range(count):
                _type, n_in, n_out, _act = (int.from_bytes(f.read(4), "little") for _ in range(4))
                net.shapes.append((n_in, n_out))
                f.seek(4 * (n_in * n_out + n_out), 1)
        return net

    def lastClip(self):
        a, b = C.c_float(), C.c_float()
        self._ck(lib.zn_net_last_clip(self.handle, C.byref(a), C.byref(b)))
        return a.value, b.value

    def setDataParallel(self, global_rows):
        self._ck(lib.zn_net_set_data_parallel(self.handle, global_rows))

    def setUpdateSharding(self, on=True):
        """After setDataParallel: reduce-scatter / update 1/world of the parameters / all-gather instead of
        all-reduce + full update on every rank."""
        self._ck(lib.zn_net_set_update_sharding(self.handle, int(on)))


__all__ = ["Network", "Sgd", "Adam", "Loss", "Activation"]
