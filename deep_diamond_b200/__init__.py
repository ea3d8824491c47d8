"""deep_diamond_b200 -- a B200-native (sm_100a) backend for Deep Diamond's data-parallel tensor hot
path: layout reorder with data type conversion, eltwise activation forward/backward, broadcast
op-tensor and reduce-tensor, behind the reference's tensor / dnn API as a new factory.

    from deep_diamond_b200 import b200_factory, tensor, dnn

Layers, bottom up (same split as the reference's cuDNN backend):
  libdd_b200.so (csrc/, C ABI in include/dd_b200.h)  hand-written CUDA kernels
  _lib        raw ctypes binding + status check          (cudnn/impl.clj)
  constants   keyword tables                             (cudnn/constants.clj)
  core        functional wrappers                        (cudnn/core.clj)
  factory     factory, tensor, transformer, batcher ...  (cudnn/factory.clj, cudnn/tensor.clj)
  tensor, dnn the public API                             (base/tensor.clj, base/dnn.clj)
  sharded     batch-dim sharding over several GPUs       (no counterpart in the reference)
"""
from ._lib import DiamondError, LIB_PATH  # noqa: F401  (import fails loudly without the library)
from .factory import B200Factory, b200_factory  # noqa: F401
from . import constants, core, dnn, tensor  # noqa: F401
