"""ctypes binding of the C oracle (oracle/ternaspmm_oracle.c).  Test
infrastructure only: used by the tests, the smoke check and the CPU-baseline
leg of the benchmark; never by the product package."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    subprocess.run(["make", "-C", _HERE, "libternaspmm_oracle.so"], check=True)


def load():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libternaspmm_oracle.so")
        if not os.path.exists(path):
            build()
        lib = ctypes.CDLL(path)
        P, I = ctypes.c_void_p, ctypes.c_int
        lib.oracle_num_threads.restype = I
        lib.oracle_set_num_threads.argtypes = [I]
        lib.oracle_gemm_i32.argtypes = [P, P, I, I, I, P]
        lib.oracle_epilogue.argtypes = [P, P, P, I, I, I, I, P]
        lib.oracle_ternaspmm.argtypes = [P, P, P, P, I, I, I, I, I, P, P]
        _LIB = lib
    return _LIB


def ternaspmm(xq, W, s_bits, ws_bits, ws_num, mode=-1):
    """Dense ternary W[N][K] int8, xq[M][K] int8, bf16 bit patterns for the
    scales -> (acc int32 [M][N], out bf16 bits [M][N])."""
    lib = load()
    M, K = xq.shape
    N = W.shape[0]
    xq, W = np.ascontiguousarray(xq), np.ascontiguousarray(W)
    s_bits = np.ascontiguousarray(s_bits, dtype=np.uint16)
    ws_bits = np.ascontiguousarray(ws_bits, dtype=np.uint16)
    acc = np.empty((M, N), np.int32)
    out = np.empty((M, N), np.uint16)
    lib.oracle_ternaspmm(xq.ctypes.data, W.ctypes.data, s_bits.ctypes.data, ws_bits.ctypes.data, ws_num, M, N, K, mode,
                         acc.ctypes.data, out.ctypes.data)
    return acc, out
