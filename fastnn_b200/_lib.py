"""ctypes binding of ``libfastnn_cuda.so`` (the C ABI declared in ``include/fastnn_cuda.h``).

The library is the product; this module only loads it and declares signatures.  There is no
fallback: if the shared library is missing or a CUDA device is absent, the call raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfastnn_cuda.so")

FNN_OK = 0
ERR_NAMES = {1: "Compilation", 2: "Dispatch", 3: "Memory", 4: "UnsupportedOp"}

FMT_I8, FMT_I4, FMT_F8, FMT_F4, FMT_I4CB = 0, 1, 2, 3, 4
EPI_NONE, EPI_RELU, EPI_GELU, EPI_SILU = 0, 1, 2, 3
PATH_AUTO, PATH_ROWS, PATH_MMA, PATH_TC = 0, 1, 2, 3
EW_ADD, EW_MUL, EW_SUB, EW_RELU, EW_GELU, EW_SILU = 0, 1, 2, 10, 11, 12

_c = ctypes
_vp, _sz, _int, _i64, _f = _c.c_void_p, _c.c_size_t, _c.c_int, _c.c_int64, _c.c_float

# name -> (restype, argtypes); every symbol include/fastnn_cuda.h declares.
SIGNATURES = {
    "fnn_cuda_ctx_create": (_int, [_int, _c.POINTER(_vp)]),
    "fnn_cuda_ctx_create_on_stream": (_int, [_int, _vp, _c.POINTER(_vp)]),
    "fnn_cuda_ctx_stream": (_vp, [_vp]),
    "fnn_cuda_ctx_set_overlap": (_int, [_vp, _int]),
    "fnn_cuda_ctx_destroy": (_int, [_vp]),
    "fnn_cuda_sync": (_int, [_vp]),
    "fnn_cuda_last_error": (_c.c_char_p, []),
    "fnn_cuda_launch_count": (_int, [_vp, _c.POINTER(_c.c_uint64)]),
    "fnn_cuda_device_info": (_int, [_vp, _c.POINTER(_int), _c.POINTER(_int), _c.POINTER(_int),
                                    _c.POINTER(_sz)]),
    "fnn_cuda_arena_alloc": (_int, [_vp, _sz, _c.POINTER(_vp)]),
    "fnn_cuda_arena_wrap": (_int, [_vp, _vp, _sz, _c.POINTER(_vp)]),
    "fnn_cuda_arena_free": (_int, [_vp]),
    "fnn_cuda_arena_write": (_int, [_vp, _sz, _vp, _sz]),
    "fnn_cuda_arena_read": (_int, [_vp, _sz, _vp, _sz]),
    "fnn_cuda_arena_write_async": (_int, [_vp, _sz, _vp, _sz]),
    "fnn_cuda_arena_read_async": (_int, [_vp, _sz, _vp, _sz]),
    "fnn_cuda_arena_device_ptr": (_vp, [_vp]),
    "fnn_cuda_arena_size": (_sz, [_vp]),
    "fnn_cuda_host_alloc": (_int, [_sz, _c.POINTER(_vp)]),
    "fnn_cuda_host_free": (_int, [_vp]),
    "fnn_cuda_qweight_upload": (_int, [_vp, _int, _vp, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _sz, _vp,
                                       _c.POINTER(_vp)]),
    "fnn_cuda_qweight_from_arena": (_int, [_vp, _int, _vp, _sz, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _sz, _vp,
                                           _c.POINTER(_vp)]),
    "fnn_cuda_qweight_prepare": (_int, [_vp, _vp, _int]),
    "fnn_cuda_qweight_free": (_int, [_vp]),
    "fnn_cuda_qweight_packed_bytes": (_sz, [_vp]),
    "fnn_cuda_qweight_unrepack": (_int, [_vp, _vp, _sz]),
    "fnn_cuda_qweight_dequant": (_int, [_vp, _vp, _sz]),
    "fnn_cuda_qmatmul": (_int, [_vp, _vp, _vp, _sz, _sz, _i64, _sz, _int, _int]),
    "fnn_cuda_qmatmul_ptr": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _int, _int]),
    "fnn_cuda_qmatmul_noalloc": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _int]),
    "fnn_cuda_last_path": (_c.c_char_p, [_vp]),
    "fnn_cuda_ipc_export": (_int, [_vp, _vp]),
    "fnn_cuda_ipc_open": (_int, [_vp, _vp, _c.POINTER(_vp)]),
    "fnn_cuda_ipc_close": (_int, [_vp, _vp]),
    "fnn_cuda_gather_wait": (_int, [_vp, _vp, _sz, _sz, _int, _sz, _vp]),
    "fnn_cuda_qmatmul_gather": (_int, [_vp, _vp, _vp, _vp, _sz, _int, _int, _int, _c.POINTER(_vp), _sz, _sz,
                                       _sz]),
    "fnn_cuda_qmatmul_allgather": (_int, [_vp, _vp, _vp, _vp, _sz, _int, _int, _int, _c.POINTER(_vp), _sz, _sz,
                                          _sz, _sz]),
    "fnn_cuda_elementwise": (_int, [_vp, _int, _vp, _sz, _sz, _sz, _sz, _sz, _sz]),
    "fnn_cuda_rms_norm": (_int, [_vp, _vp, _sz, _sz, _c.c_longlong, _sz, _sz, _c.c_float, _sz]),
    "fnn_cuda_row_norm": (_int, [_vp, _vp, _int, _sz, _sz, _c.c_longlong, _c.c_longlong, _sz, _c.c_longlong, _sz,
                                 _sz, _c.c_float, _sz]),
    "fnn_cuda_softmax": (_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz]),
    "fnn_cuda_memcpy": (_int, [_vp, _vp, _sz, _sz, _sz]),
    "fnn_cuda_fill": (_int, [_vp, _vp, _sz, _sz, _f]),
    "fnn_cuda_memcpy2d": (_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz]),
    "fnn_cuda_graph_begin": (_int, [_vp]),
    "fnn_cuda_graph_end": (_int, [_vp, _c.POINTER(_vp)]),
    "fnn_cuda_graph_launch": (_int, [_vp, _vp]),
    "fnn_cuda_graph_free": (_int, [_vp]),
    "fnn_cuda_timer_start": (_int, [_vp, _int]),
    "fnn_cuda_timer_stop": (_int, [_vp, _int]),
    "fnn_cuda_timer_elapsed_ms": (_int, [_vp, _int, _c.POINTER(_f)]),
    "fnn_cuda_flush_l2": (_int, [_vp]),
    "fnn_quant_packed_bytes": (_sz, [_int, _sz, _sz]),
    "fnn_quant_num_scales": (_sz, [_int, _sz, _sz]),
    "fnn_quantize_weights": (_int, [_int, _vp, _sz, _sz, _vp, _vp, _vp, _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (built in-tree by ``fastnn_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m fastnn_b200.build` "
            "(there is no CPU fallback for the CUDA backend)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().fnn_cuda_last_error().decode("utf-8", "replace")
