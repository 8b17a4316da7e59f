"""ctypes binding of libzn_b200.so (the C ABI in include/zn_b200.h).

There is no fallback: if the shared library has not been built the import of
this package fails, and every compute call fails when no CUDA device is present.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libzn_b200.so")

OK = 0
STATUS_NAMES = {
    0: "ZN_OK", 1: "ZN_ERR_INVALID_VALUE", 2: "ZN_ERR_OUT_OF_MEMORY", 3: "ZN_ERR_NOT_INITIALIZED",
    4: "ZN_ERR_NO_DEVICE", 5: "ZN_ERR_INVALID_DEVICE", 6: "ZN_ERR_CUDA", 7: "ZN_ERR_SHAPE",
    8: "ZN_ERR_UNSUPPORTED", 9: "ZN_ERR_TIMEOUT", 10: "ZN_ERR_NCCL", 11: "ZN_ERR_NOT_AVAILABLE",
}


class ZnError(RuntimeError):
    def __init__(self, status, detail=""):
        self.status = status
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {detail}")


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python zigneuron_b200/build.py` "
        "(there is no CPU implementation to fall back to)")

lib = C.CDLL(LIB_PATH)

vp, sz, f32, i32, u64 = C.c_void_p, C.c_size_t, C.c_float, C.c_int32, C.c_uint64
pf, pvp, psz = C.POINTER(C.c_float), C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)

# Every symbol the header declares: name -> (restype, argtypes).  Float pointers are void* here so
# that numpy buffers (host) and integer device addresses can both be passed.
SIGNATURES = {
    "zn_device_count": (i32, []),
    "zn_ctx_create": (i32, [i32, pvp]),
    "zn_ctx_destroy": (None, [vp]),
    "zn_last_error_string": (C.c_char_p, [vp]),
    "zn_status_string": (C.c_char_p, [i32]),
    "zn_ctx_set_precision": (i32, [vp, i32]),
    "zn_begin_command_batch": (i32, [vp]),
    "zn_end_command_batch": (i32, [vp]),
    "zn_tensor_alloc": (i32, [vp, sz, pvp]),
    "zn_tensor_free": (i32, [vp, vp]),
    "zn_tensor_upload": (i32, [vp, vp, vp, sz]),
    "zn_tensor_download": (i32, [vp, vp, vp, sz]),
    "zn_copy_data": (i32, [vp, vp, vp, sz]),
    "zn_matmul": (i32, [vp, vp, vp, vp, sz, sz, sz, i32]),
    "zn_matmul_transpose_a": (i32, [vp, vp, vp, vp, sz, sz, sz, i32]),
    "zn_matmul_transpose_b": (i32, [vp, vp, vp, vp, sz, sz, sz, i32]),
    "zn_matmul_bias_act": (i32, [vp, vp, vp, vp, vp, sz, sz, sz, i32]),
    "zn_add_bias": (i32, [vp, vp, sz, vp, sz]),
    "zn_accumulate_bias": (i32, [vp, vp, sz, vp, sz]),
    "zn_accumulate_bias_noalloc": (i32, [vp, vp, sz, vp, sz]),
    "zn_activation_forward": (i32, [vp, i32, vp, vp, sz]),
    "zn_activation_backward": (i32, [vp, i32, vp, vp, vp, sz]),
    "zn_loss_forward": (i32, [vp, i32, vp, vp, sz, sz, pf]),
    "zn_loss_backward": (i32, [vp, i32, vp, vp, vp, sz, sz]),
    "zn_sgd_update": (i32, [vp, vp, vp, sz, f32, f32]),
    "zn_sgd_update_bias": (i32, [vp, vp, vp, sz, f32]),
    "zn_adam_update": (i32, [vp, vp, vp, vp, vp, sz, f32, f32, f32, f32, f32, f32]),
    "zn_evaluate_classification": (i32, [vp, vp, vp, sz, sz, sz, vp, vp]),
    "zn_rmsprop_update": (i32, [vp, vp, vp, vp, sz, f32, f32, f32]),
    "zn_clip_grad_norm": (i32, [vp, pvp, psz, sz, pf, pf]),
    "zn_net_create": (i32, [vp, i32, pvp]),
    "zn_net_destroy": (None, [vp]),
    "zn_net_add_dense": (i32, [vp, sz, sz, i32, C.POINTER(i32)]),
    "zn_net_layer_count": (i32, [vp, psz]),
    "zn_net_set_weights": (i32, [vp, sz, vp, vp]),
    "zn_net_get_weights": (i32, [vp, sz, vp, vp]),
    "zn_net_get_grads": (i32, [vp, sz, vp, vp]),
    "zn_net_get_input_grad": (i32, [vp, vp, sz]),
    "zn_net_set_sgd": (i32, [vp, i32, f32]),
    "zn_net_set_adam": (i32, [vp, i32, f32, f32, f32, f32]),
    "zn_net_set_sgd_momentum": (i32, [vp, i32, f32]),
    "zn_net_set_adamw": (i32, [vp, i32, f32, f32, f32, f32]),
    "zn_net_set_rmsprop": (i32, [vp, i32, f32, f32, f32]),
    "zn_net_forward": (i32, [vp, vp, sz, vp]),
    "zn_net_evaluate_classification": (i32, [vp, vp, vp, sz, sz, vp, vp]),
    "zn_net_train_step": (i32, [vp, vp, vp, sz, f32, i32, pf]),
    "zn_net_submit_step": (i32, [vp, vp, vp, sz, f32, i32]),
    "zn_net_wait_step": (i32, [vp, pf]),
    "zn_net_train": (i32, [vp, vp, vp, sz, sz, f32, i32, vp]),
    "zn_net_last_clip": (i32, [vp, pf, pf]),
    "zn_net_save": (i32, [vp, C.c_char_p]),
    "zn_net_load": (i32, [vp, i32, C.c_char_p, pvp]),
    "zn_net_save_optimizer": (i32, [vp, C.c_char_p]),
    "zn_net_load_optimizer": (i32, [vp, C.c_char_p]),
    "zn_host_alloc": (i32, [vp, sz, pvp]),
    "zn_host_free": (i32, [vp, vp]),
    "zn_distribute_workload": (i32, [sz, sz, sz, psz, psz]),
    "zn_dp_unique_id": (i32, [C.c_char_p]),
    "zn_dp_init": (i32, [vp, i32, i32, C.c_char_p]),
    "zn_dp_destroy": (i32, [vp]),
    "zn_net_set_data_parallel": (i32, [vp, sz]),
    "zn_net_set_update_sharding": (i32, [vp, i32]),
    "zn_dp_set_timeout_ms": (i32, [vp, C.c_int64]),
    "zn_wait_poll": (i32, [vp, vp, vp, C.c_int64, C.POINTER(i32)]),
    "zn_debug_bounded_wait_probe": (i32, [vp, C.c_int64]),
    "zn_debug_set_device_status": (i32, [vp, i32]),
    "zn_debug_tc_route": (i32, [i32, C.c_int64, C.c_int64, C.c_int64, i32, i32, i32, C.POINTER(i32)]),
    "zn_profile_enable": (i32, [vp, i32]),
    "zn_profile_reset": (i32, [vp]),
    "zn_profile_get": (i32, [vp, i32, C.POINTER(C.c_double), C.POINTER(u64), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "zn_timer_start": (i32, [vp]),
    "zn_timer_stop": (i32, [vp, pf]),
    "zn_launch_count": (i32, [vp, C.POINTER(u64)]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = header and library disagree
    _fn.restype, _fn.argtypes = _res, _args


def ptr(x):
    """void* for a numpy array (host), a DeviceTensor, an int device address, or None."""
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        if x.dtype != np.float32 or not x.flags["C_CONTIGUOUS"]:
            raise TypeError("operands must be C-contiguous float32 arrays")
        return x.ctypes.data
    if hasattr(x, "address"):
        return x.address
    return int(x)


def check(status, ctx_handle=None):
    if status != OK:
        detail = ""
        if ctx_handle:
            detail = (lib.zn_last_error_string(ctx_handle) or b"").decode()
        if not detail:
            detail = (lib.zn_status_string(status) or b"").decode()
        raise ZnError(status, detail)
