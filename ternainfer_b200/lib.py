"""ctypes binding of ``libternaspmm.so`` (built in-tree under ``csrc/``).

The reference binds its library with ``ctypes.CDLL('./kernels/libternaspmm.so')``
and passes every pointer as ``c_void_p`` (model.py:21, :76-89 of
Gu-J/TernaInfer); this module does the same against the B200 library and
declares argument types so that mistakes fail in Python rather than on the GPU.
There is no fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
_LIB = None

_P = ctypes.c_void_p
_I = ctypes.c_int
_SPMM_ARGS = [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]


class ListItem(ctypes.Structure):
    """``ternaspmm_list_item`` of include/ternaspmm.h."""
    _fields_ = [(n, _P) for n in ("x", "bitmap", "tile_offsets", "quarter_offsets", "sign_words", "out", "s", "ws",
                                  "residual")] + \
               [(n, _I) for n in ("ws_num", "M", "N", "K", "seg1", "seg2", "seg3", "prefill_form")]


def library_path() -> str:
    return os.path.join(_CSRC, "libternaspmm.so")


def build_library(verbose: bool = False) -> str:
    """Compile the library for sm_100a with nvcc (``make -C csrc``)."""
    subprocess.run(["make", "-C", _CSRC] + (["verbose"] if verbose else []), check=True)
    return library_path()


def load_library() -> ctypes.CDLL:
    """Load the shared library; raises ``OSError`` if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise OSError(f"{path} not found: build it with `make -C {_CSRC}` (or __graft_entry__.build())")
    lib = ctypes.CDLL(path)
    for name in ("bitlinear_TernaSpMM", "bitlinear_TernaSpMM_decode", "bitlinear_TernaSpMM_prefill"):
        fn = getattr(lib, name)
        fn.argtypes = _SPMM_ARGS
        fn.restype = None
    lib.bitlinear_TernaSpMM_benchmark.argtypes = [_I, _I, _I] + _SPMM_ARGS
    lib.bitlinear_TernaSpMM_benchmark.restype = None
    lib.checkLastCudaError.argtypes = [_I]
    lib.checkLastCudaError.restype = None
    lib.reorder_WT_h.argtypes = [_P, _P, _I, _I]
    lib.reorder_WT_h.restype = None
    lib.convert_reorderd.argtypes = [_P, _I, _I, _I, _I, _I, _I, _I, _I,
                                     ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P),
                                     ctypes.POINTER(_P), ctypes.POINTER(_I)]
    lib.convert_reorderd.restype = _I
    lib.gpu_sleep.argtypes = [ctypes.c_double, _P]
    lib.gpu_sleep.restype = None
    lib.ternaspmm_last_status.argtypes = []
    lib.ternaspmm_last_status.restype = _I
    lib.ternaspmm_set_wait_limit_ms.argtypes = [_I]
    lib.ternaspmm_set_wait_limit_ms.restype = None
    lib.ternaspmm_last_launch_shape.argtypes = [_P]
    lib.ternaspmm_last_launch_shape.restype = None
    lib.ternaspmm_debug_inject_host_failure.argtypes = [_I]
    lib.ternaspmm_debug_inject_host_failure.restype = None
    lib.ternaspmm_list_plan.argtypes = [_P, _I, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong)]
    lib.ternaspmm_list_plan.restype = _I
    lib.ternaspmm_list_create.argtypes = [_P, _I, _P, _P, _P]
    lib.ternaspmm_list_create.restype = _P
    lib.ternaspmm_list_run.argtypes = [_P, _P]
    lib.ternaspmm_list_run.restype = None
    lib.ternaspmm_list_destroy.argtypes = [_P]
    lib.ternaspmm_list_destroy.restype = None
    lib.ternaspmm_lm_head_argmax.argtypes = [_P, _P, _I, _I, _I, _P, _P, _I, _P, _P]
    lib.ternaspmm_lm_head_argmax.restype = None
    lib.ternaspmm_lm_head_argmax_noalloc.argtypes = [_P, _P, _I, _I, _I, _P, _P, _I, _P]
    lib.ternaspmm_lm_head_argmax_noalloc.restype = None
    lib.ternaspmm_lm_head_scratch_bytes.argtypes = []
    lib.ternaspmm_lm_head_scratch_bytes.restype = ctypes.c_longlong
    lib.ternaspmm_accumulate_i32.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P]
    lib.ternaspmm_accumulate_i32.restype = None
    lib.ternaspmm_linear_segments.argtypes = [_P] * 8 + [_I] * 8 + [_P]
    lib.ternaspmm_linear_segments.restype = None
    for name in ("ternaspmm_rmsnorm_quant", "ternaspmm_relu2_gate_rmsnorm_quant"):
        fn = getattr(lib, name)
        fn.argtypes = [_P, _P, ctypes.c_float, _I, _I, _P, _P, _P]
        fn.restype = None
    lib.ternaspmm_rmsnorm.argtypes = [_P, _P, ctypes.c_float, _I, _I, _P, _P]
    lib.ternaspmm_debug_int8_mma_rate.argtypes = [_I, _P]
    lib.ternaspmm_debug_int8_mma_rate.restype = ctypes.c_double
    lib.ternaspmm_rmsnorm.restype = None
    lib.ternaspmm_quant.argtypes = [_P, _I, _I, _P, _P, _P]
    lib.ternaspmm_quant.restype = None
    lib.ternaspmm_scale_quant_sumsq.argtypes = [_P, _P, _I, _I, _I, _P, _P, _P, _P]
    lib.ternaspmm_scale_quant_sumsq.restype = None
    lib.ternaspmm_partial_f32.argtypes = [_P] * 7 + [_I, _I, _I, _P]
    lib.ternaspmm_partial_f32.restype = None
    lib.ternaspmm_tp_finish.argtypes = [_P, _P, ctypes.c_float, _I, _I, _I, _P, _P, _P]
    lib.ternaspmm_tp_finish.restype = None
    lib.ternaspmm_tp_allreduce_finish.argtypes = [_P, _P, _P, _I, _I, _P, _P, ctypes.c_float, _I, _I, _I, _P, _P]
    lib.ternaspmm_tp_allreduce_finish.restype = None
    lib.bitlinear_TernaSpMM_ws.argtypes = [_P] * 8 + [_I] * 4 + [_P, _P, ctypes.c_longlong, _I, _P]
    lib.bitlinear_TernaSpMM_ws.restype = None
    lib.bitlinear_TernaSpMM_residual.argtypes = [_P] * 8 + [_I] * 4 + [_P, _P]
    lib.bitlinear_TernaSpMM_residual.restype = None
    lib.ternaspmm_pack_i8.argtypes = [_P, _I, _I, _P, _P, _P, _P]
    lib.ternaspmm_pack_i8.restype = ctypes.c_longlong
    lib.ternaspmm_unpack_i8.argtypes = [_P, _P, _P, _I, _I, _P]
    lib.ternaspmm_unpack_i8.restype = _I
    lib.ternaspmm_transcode_reference_layout.argtypes = [_P, _P, _P, _I, _I, _P, _P, _P]
    lib.ternaspmm_transcode_reference_layout.restype = _I
    _LIB = lib
    return lib


EXPORTED_SYMBOLS = (
    "bitlinear_TernaSpMM", "bitlinear_TernaSpMM_decode", "bitlinear_TernaSpMM_prefill",
    "bitlinear_TernaSpMM_benchmark", "checkLastCudaError", "reorder_WT_h", "convert_reorderd",
    "gpu_sleep", "ternaspmm_last_status", "ternaspmm_set_wait_limit_ms", "ternaspmm_last_launch_shape",
    "ternaspmm_debug_inject_host_failure", "ternaspmm_debug_int8_mma_rate", "ternaspmm_lm_head_argmax", "ternaspmm_lm_head_scratch_bytes",
    "ternaspmm_lm_head_argmax_noalloc",
    "ternaspmm_list_plan", "ternaspmm_list_create", "ternaspmm_list_run", "ternaspmm_list_destroy",
    "ternaspmm_accumulate_i32", "ternaspmm_linear_segments", "bitlinear_TernaSpMM_residual", "bitlinear_TernaSpMM_ws", "ternaspmm_quant",
    "ternaspmm_scale_quant_sumsq", "ternaspmm_partial_f32", "ternaspmm_tp_finish", "ternaspmm_tp_allreduce_finish", "ternaspmm_rmsnorm_quant", "ternaspmm_relu2_gate_rmsnorm_quant", "ternaspmm_rmsnorm", "ternaspmm_pack_i8",
    "ternaspmm_unpack_i8", "ternaspmm_transcode_reference_layout",
)
