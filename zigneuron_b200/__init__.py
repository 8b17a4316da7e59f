"""zigneuron_b200: ZigNeuron's Dense-layer training path on NVIDIA B200.

Host-side mirror of the reference's Backend / Network / Loss / optimizer
interface for that path, over the C ABI of libzn_b200.so (include/zn_b200.h).
Importing the package loads the shared library and fails if it has not been
built; there is no CPU implementation behind these classes.
"""
from ._lib import LIB_PATH, ZnError, lib  # noqa: F401  (import = load the .so, or fail)
from .backend import Activation, Backend, DeviceTensor, Loss, Precision  # noqa: F401
from .network import Adam, AdamW, Network, Rmsprop, Sgd  # noqa: F401

__all__ = ["Backend", "Network", "Activation", "Loss", "Precision", "DeviceTensor", "Sgd", "Adam", "AdamW", "Rmsprop", "ZnError"]
