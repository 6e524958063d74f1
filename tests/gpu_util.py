"""Helpers for the GPU parity tests: device buffers (torch is only plumbing)
and calls through the C ABI with raw pointers."""
import ctypes

import numpy as np
import torch

import ternaspmm_oracle as o
from ternainfer_b200.convert import compress_weight


def dev(a: np.ndarray) -> torch.Tensor:
    """numpy array of any integer width -> CUDA tensor with the same bytes."""
    a = np.ascontiguousarray(a)
    return torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda()


class Packed:
    def __init__(self, w: np.ndarray, arrays=None):
        self.N, self.K = w.shape
        self.w = w
        if arrays is None:
            arrays = [t.numpy() for t in compress_weight(torch.from_numpy(w))]
        self.host = arrays
        self.cv, self.tg, self.tm, self.bm = (dev(a) for a in arrays)


def call(lib, entry, xq, pk: Packed, s_bits, ws_bits, ws_num, stream=None, out=None, pad=0):
    """bf16 bits [M][N] from one of the three bitlinear_* entry points.  With
    ``pad`` > 0 the output sits between canary regions that are checked."""
    M, K = xq.shape
    x_d, s_d, ws_d = dev(xq), dev(np.asarray(s_bits, np.uint16)), dev(np.asarray(ws_bits, np.uint16))
    total = M * pk.N + 2 * pad
    buf = torch.full((total,), 0x7B7B, dtype=torch.int16, device="cuda") if out is None else out
    optr = buf.data_ptr() + 2 * pad
    st = torch.cuda.current_stream().cuda_stream if stream is None else stream
    getattr(lib, entry)(x_d.data_ptr(), pk.bm.data_ptr(), pk.tg.data_ptr(), pk.tm.data_ptr(), pk.cv.data_ptr(),
                        optr, s_d.data_ptr(), ws_d.data_ptr(), ws_num, M, pk.N, K, 7, 0, st)
    torch.cuda.synchronize()
    h = buf.cpu().numpy().view(np.uint16)
    if pad:
        assert (h[:pad] == 0x7B7B).all() and (h[pad + M * pk.N:] == 0x7B7B).all(), "canary overwritten"
    return h[pad:pad + M * pk.N].reshape(M, pk.N).copy()


def accumulate(lib, xq, pk: Packed):
    M, K = xq.shape
    x_d = dev(xq)
    out = torch.full((M * pk.N,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    lib.ternaspmm_accumulate_i32(x_d.data_ptr(), pk.bm.data_ptr(), pk.tg.data_ptr(), pk.tm.data_ptr(),
                                 pk.cv.data_ptr(), out.data_ptr(), M, pk.N, K,
                                 torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out.cpu().numpy().reshape(M, pk.N)


def inputs(M, N, K, ws_num, p_zero=0.45, seed=100):
    w = o.make_ternary(N, K, p_zero, seed)
    xq, s = o.make_activations(M, K, seed + 1)
    ws = o.make_ws(ws_num, seed + 2)
    return w, xq, s, ws


def max_rel_err(got_bits, want_bits):
    a, b = o.bf16_bits_to_f32(got_bits).astype(np.float64), o.bf16_bits_to_f32(want_bits).astype(np.float64)
    d = np.abs(a - b)
    return float(np.max(np.where(d == 0, 0.0, d / np.maximum(np.abs(b), 1e-30))))
