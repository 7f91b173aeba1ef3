"""adrastea_b200: the matmul hot path of eiz/adrastea, hand-written for B200 (sm_100a).

Public surface (mirrors adrastea_models/src/kernels.rs and tensor.rs for this path):
``GpuKernels``, ``MatmulTracer``, ``MatmulOptions``, ``MatmulStore``, ``MatmulLoad``,
``MatmulMask``, ``TensorLayout``, ``TensorView``.
"""
from .tensor import TensorLayout, TensorView, TensorViewMut  # noqa: F401
from .kernels import (  # noqa: F401
    AdrError, BinaryOp, GpuKernels, Kernel, MatmulLoad, MatmulLoadOp, MatmulMask, MatmulOptions,
    MatmulStore, MatmulStoreOp, MatmulTracer, lower_matmul,
)
