"""Backend: the reference's `Backend` struct (src/backend.zig:26-125) for the
methods on the Dense path, each forwarding to the C-ABI entry point that stands
in for its CUDA arm.  Method names and argument order follow the reference;
slices become numpy float32 arrays (host operands) or DeviceTensor handles (the
role of the reference's `?*const metal.MTLBuffer` slot).  Results land in the
output argument, as in the reference."""
import ctypes as C
import enum

import numpy as np

from ._lib import ZnError, check, lib, ptr


class Precision(enum.IntEnum):
    FP32_SIMT = 0
    FP32_EXACT = 1
    TF32_TC = 2
    BF16_TC = 3


class Activation(enum.IntEnum):      # order of src/activation.zig:14-22
    relu = 0
    sigmoid = 1
    tanh = 2
    softmax = 3
    linear = 4
    gelu = 5
    leaky_relu = 6
    elu = 7


class Loss(enum.IntEnum):            # order of src/loss.zig:12-22
    mse = 0
    cross_entropy = 1
    cross_entropy_logits = 2
    binary_cross_entropy = 3
    kl_divergence = 4


class DeviceTensor:
    """A float32 block resident on the GPU (Tensor.init + its device handle, src/tensor.zig:17-118)."""

    def __init__(self, backend, count):
        self.backend, self.count = backend, int(count)
        out = C.c_void_p()
        check(lib.zn_tensor_alloc(backend.handle, self.count, C.byref(out)), backend.handle)
        self.address = out.value

    @classmethod
    def from_numpy(cls, backend, array):
        a = np.ascontiguousarray(array, dtype=np.float32)
        t = cls(backend, a.size)
        check(lib.zn_tensor_upload(backend.handle, t.address, a.ctypes.data, a.size), backend.handle)
        return t

    def numpy(self, shape=None):
        out = np.empty(self.count, np.float32)
        check(lib.zn_tensor_download(self.backend.handle, out.ctypes.data, self.address, self.count), self.backend.handle)
        return out.reshape(shape) if shape is not None else out

    def free(self):
        if self.address and self.backend.handle:
            lib.zn_tensor_free(self.backend.handle, self.address)
        self.address = None


class Backend:
    """`Backend.init(allocator)` of the reference picks CUDA when a device exists
    (src/backend.zig:43-94); here construction fails with ZN_ERR_NO_DEVICE instead
    of falling back to CPU code."""

    def __init__(self, device=0, precision=Precision.FP32_SIMT):
        h = C.c_void_p()
        check(lib.zn_ctx_create(int(device), C.byref(h)))
        self.handle = h.value
        self.device = int(device)
        self.set_precision(precision)

    @staticmethod
    def device_count():
        return int(lib.zn_device_count())

    def deinit(self):
        if getattr(self, "handle", None):
            lib.zn_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.deinit()
        except Exception:
            pass

    def _ck(self, status):
        check(status, self.handle)

    def set_precision(self, precision):
        self.precision = Precision(precision)
        self._ck(lib.zn_ctx_set_precision(self.handle, int(precision)))

    def tensor(self, array_or_count):
        if isinstance(array_or_count, (int, np.integer)):
            return DeviceTensor(self, array_or_count)
        return DeviceTensor.from_numpy(self, array_or_count)

    # ---- src/backend.zig:105-136
    def beginCommandBatch(self):
        self._ck(lib.zn_begin_command_batch(self.handle))

    def endCommandBatch(self):
        self._ck(lib.zn_end_command_batch(self.handle))

    def copyData(self, src, dst, count=None):
        n = count if count is not None else (src.size if isinstance(src, np.ndarray) else src.count)
        self._ck(lib.zn_copy_data(self.handle, ptr(src), ptr(dst), n))

    # ---- GEMMs, src/backend.zig:169-325
    def matMul(self, a, b, c, m, n, k, accumulate=False):
        self._ck(lib.zn_matmul(self.handle, ptr(a), ptr(b), ptr(c), m, n, k, int(accumulate)))

    def matMulBatch(self, a, b, c, batch_size, n, k, accumulate=False):
        self.matMul(a, b, c, batch_size, n, k, accumulate)

    def matMulTransposeA(self, a, b, c, m, n, k, accumulate=False):
        self._ck(lib.zn_matmul_transpose_a(self.handle, ptr(a), ptr(b), ptr(c), m, n, k, int(accumulate)))

    def matMulTransposeB(self, a, b, c, m, n, k, accumulate=False):
        self._ck(lib.zn_matmul_transpose_b(self.handle, ptr(a), ptr(b), ptr(c), m, n, k, int(accumulate)))

    def _mm_bias(self, a, b, bias, c, batch_size, n, k, act):
        self._ck(lib.zn_matmul_bias_act(self.handle, ptr(a), ptr(b), ptr(bias), ptr(c), batch_size, n, k, int(act)))

    def matMulBiasAct(self, a, b, bias, c, batch_size, n, k, act):
        """The fused Dense forward with any activation (softmax is applied row by row)."""
        self._mm_bias(a, b, bias, c, batch_size, n, k, Activation(act))

    def matMulBias(self, a, b, bias, c, batch_size, n, k):
        self._mm_bias(a, b, bias, c, batch_size, n, k, Activation.linear)

    def matMulBiasRelu(self, a, b, bias, c, batch_size, n, k):
        self._mm_bias(a, b, bias, c, batch_size, n, k, Activation.relu)

    def matMulBiasSigmoid(self, a, b, bias, c, batch_size, n, k):
        self._mm_bias(a, b, bias, c, batch_size, n, k, Activation.sigmoid)

    def matMulBiasTanh(self, a, b, bias, c, batch_size, n, k):
        self._mm_bias(a, b, bias, c, batch_size, n, k, Activation.tanh)

    # ---- bias / activations, src/backend.zig:367-399, :649-671
    @staticmethod
    def _len(x):
        return x.size if isinstance(x, np.ndarray) else x.count

    def addBias(self, output, bias):
        self._ck(lib.zn_add_bias(self.handle, ptr(output), self._len(output), ptr(bias), self._len(bias)))

    def accumulateBias(self, grad_bias, grad_after_act):
        self._ck(lib.zn_accumulate_bias(self.handle, ptr(grad_bias), self._len(grad_bias), ptr(grad_after_act),
                                        self._len(grad_after_act)))

    def accumulateBiasNoAlloc(self, grad_bias, grad_after_act):
        """accumulateBias for callers that must not allocate device memory (device tensors only; the partial
        sums live in a fixed block inside the library instead of the context's growable scratch)."""
        self._ck(lib.zn_accumulate_bias_noalloc(self.handle, ptr(grad_bias), self._len(grad_bias), ptr(grad_after_act),
                                                self._len(grad_after_act)))

    def activationForward(self, act, input, output):
        self._ck(lib.zn_activation_forward(self.handle, int(act), ptr(input), ptr(output), self._len(input)))

    def activationBackward(self, act, input, grad_output, grad_input):
        self._ck(lib.zn_activation_backward(self.handle, int(act), ptr(input), ptr(grad_output), ptr(grad_input),
                                            self._len(input)))

    # ---- loss, src/backend.zig:403-417 and Loss.forward src/loss.zig:34-46
    def lossBackward(self, loss_fn, output, target, grad_output, rows=1):
        n = self._len(output)
        self._ck(lib.zn_loss_backward(self.handle, int(loss_fn), ptr(output), ptr(target), ptr(grad_output), rows, n // rows))

    def lossForward(self, loss_fn, output, target, rows=1):
        n = self._len(output)
        out = C.c_float()
        self._ck(lib.zn_loss_forward(self.handle, int(loss_fn), ptr(output), ptr(target), rows, n // rows, C.byref(out)))
        return out.value

    # ---- metrics.evaluateClassification, src/metrics.zig:239-264
    def evaluateClassification(self, outputs, targets, num_classes, rows=None):
        """Returns (confusion[num_classes, num_classes] uint64 indexed [true][predicted],
        dict(accuracy, precision, recall, f1_score))."""
        if rows is None:
            rows = outputs.shape[0] if isinstance(outputs, np.ndarray) and outputs.ndim == 2 else 0
        cols = self._len(outputs) // rows if rows else 1
        cm = np.zeros((num_classes, num_classes), np.uint64)
        m = np.zeros(4, np.float32)
        self._ck(lib.zn_evaluate_classification(self.handle, ptr(outputs), ptr(targets), rows, cols, num_classes,
                                                cm.ctypes.data, m.ctypes.data))
        return cm, dict(zip(("accuracy", "precision", "recall", "f1_score"), (float(v) for v in m)))

    # ---- optimizers, src/backend.zig:420-443, :640-646
    def sgdUpdate(self, weights, gradients, learning_rate, weight_decay):
        self._ck(lib.zn_sgd_update(self.handle, ptr(weights), ptr(gradients), self._len(weights), learning_rate, weight_decay))

    def sgdUpdateBias(self, bias, gradients, learning_rate):
        self._ck(lib.zn_sgd_update_bias(self.handle, ptr(bias), ptr(gradients), self._len(bias), learning_rate))

    def adamUpdate(self, weights, gradients, m, v, lr, beta1, beta2, eps, bias_corr1, bias_corr2):
        self._ck(lib.zn_adam_update(self.handle, ptr(weights), ptr(gradients), ptr(m), ptr(v), self._len(weights),
                                    lr, beta1, beta2, eps, bias_corr1, bias_corr2))

    def rmspropUpdate(self, weights, gradients, g_avg, lr, rho, eps):
        self._ck(lib.zn_rmsprop_update(self.handle, ptr(weights), ptr(gradients), ptr(g_avg), self._len(weights),
                                       lr, rho, eps))

    def clipGradNorm(self, grads):
        """The clip inside Network.trainStep (src/network.zig:513-535); scales in place, returns (norm, factor)."""
        n = len(grads)
        ptrs = (C.c_void_p * n)(*[ptr(g) for g in grads])
        lens = (C.c_size_t * n)(*[self._len(g) for g in grads])
        norm, fac = C.c_float(), C.c_float()
        self._ck(lib.zn_clip_grad_norm(self.handle, ptrs, lens, n, C.byref(norm), C.byref(fac)))
        return norm.value, fac.value

    # ---- measurement
    def profile(self, on=True):
        self._ck(lib.zn_profile_enable(self.handle, int(on)))

    def profile_reset(self):
        self._ck(lib.zn_profile_reset(self.handle))

    def profile_get(self, family):
        ms, fl, by, n = C.c_double(), C.c_double(), C.c_double(), C.c_uint64()
        self._ck(lib.zn_profile_get(self.handle, int(family), C.byref(ms), C.byref(n), C.byref(fl), C.byref(by)))
        return {"ms": ms.value, "launches": n.value, "flops": fl.value, "bytes": by.value}

    def timer_start(self):
        self._ck(lib.zn_timer_start(self.handle))

    def timer_stop(self):
        ms = C.c_float()
        self._ck(lib.zn_timer_stop(self.handle, C.byref(ms)))
        return ms.value

    def host_alloc(self, shape):
        """Pinned host memory as a float32 numpy array (for the pipelined step's inputs)."""
        count = int(np.prod(shape))
        p = C.c_void_p()
        self._ck(lib.zn_host_alloc(self.handle, count, C.byref(p)))
        buf = (C.c_float * count).from_address(p.value)
        arr = np.frombuffer(buf, dtype=np.float32).reshape(shape)
        return arr

    def launch_count(self):
        n = C.c_uint64()
        self._ck(lib.zn_launch_count(self.handle, C.byref(n)))
        return n.value

    # ---- data parallel
    @staticmethod
    def dp_unique_id():
        buf = C.create_string_buffer(128)
        check(lib.zn_dp_unique_id(buf))
        return buf.raw

    def dp_init(self, rank, world, unique_id):
        self._ck(lib.zn_dp_init(self.handle, rank, world, unique_id))

    def dp_set_timeout_ms(self, ms):
        """Deadline of every host wait that may sit behind a collective; past it the communicator is aborted
        and the call fails with ZN_ERR_NCCL."""
        self._ck(lib.zn_dp_set_timeout_ms(self.handle, int(ms)))

    def dp_destroy(self):
        self._ck(lib.zn_dp_destroy(self.handle))

    # ---- failure-path probes
    def debug_bounded_wait_probe(self, limit_cycles):
        self._ck(lib.zn_debug_bounded_wait_probe(self.handle, int(limit_cycles)))

    def debug_set_device_status(self, code):
        self._ck(lib.zn_debug_set_device_status(self.handle, int(code)))

    @staticmethod
    def distributeWorkload(total, parts, index):
        """MultiCudaContext.distributeWorkload(.round_robin), src/cuda_multi_gpu.zig:247-265."""
        s, e = C.c_size_t(), C.c_size_t()
        check(lib.zn_distribute_workload(total, parts, index, C.byref(s), C.byref(e)))
        return s.value, e.value


__all__ = ["Backend", "DeviceTensor", "Activation", "Loss", "Precision", "ZnError"]
