"""fastnn_b200: a B200 (sm_100a) CUDA backend for fastnn's quantized-weight MatMul path.

The product is ``libfastnn_cuda.so`` (C ABI in ``include/fastnn_cuda.h``, kernels in
``fastnn_b200/csrc``).  The Python modules mirror the reference's host-side interface for this
path -- ``Backend`` trait, plan instructions, ``GraphBuilder``, ``GraphExecutor``,
``AotExecutor``, ``Runtime`` -- over that C ABI.  There is no CPU fallback.
"""
from . import _lib
from .backend import (BackendError, BufferSlice, CallKernel, CudaBackend, CudaBuffer,
                      ExecutablePlan, Fill, MemCopy, ProfileEntry, QuantizedWeightMeta,
                      QWeightHandle, ShapeEnv, WriteConst)
from .compiler import (AotExecutor, ComputeGraph, GraphBuilder, GraphExecutor, GraphTensor, IrDType,
                       MemoryPlan, Opcode, TensorType, WeightDtype, fuse_operators, lower_to_plan,
                       plan_memory, quantize_weight_constant, quantize_weights)
from .runtime import Runtime, plan_from_bytes, plan_to_bytes

__all__ = [n for n in dir() if not n.startswith("_")]
