"""Call site of the TernaSpMM operator: the PyTorch side of the boundary.

Mirrors ``TernaInfer_linear`` / ``SpBitLinear`` / ``get_global_workspace`` of
the reference's ``model.py`` (:37-133 in Gu-J/TernaInfer): same names, same
argument meaning, same checkpoint keys.  Differences, all on this side of the
C ABI: the activation quantiser runs as plain torch ops (no ``torch.compile``,
hence no Triton); rows are not padded to a power of two because the B200
library accepts any token count >= 1; the workspace is accepted and ignored
(the library reduces its K split on chip).

PyTorch is only plumbing here (device memory, the current stream); all
arithmetic of the linear layer happens in ``libternaspmm.so``.  There is no
CPU path: calling with CPU tensors raises.
"""
from __future__ import annotations

import ctypes

import torch
from torch import nn

from .lib import load_library

_GLOBAL_WORKSPACE = {}
_WORKSPACE_BYTES = 13824 * 2560      # the largest BitNet-2B layer as dense int8, as model.py:34 of the reference sizes it


def reserve_workspace(nbytes: int):
    """Raise the size the shared workspace is created with (call before the first forward; a layer
    whose dense int8 copy does not fit simply keeps the on-chip decode at every token count)."""
    global _WORKSPACE_BYTES
    _WORKSPACE_BYTES = max(_WORKSPACE_BYTES, int(nbytes))


def get_global_workspace(device="cuda"):
    """One workspace shared by all layers of a device (model.py:37-42 of the reference).  The
    reference needs it for its split-K partial sums and, at more than 64 tokens, for the dense int8
    copy of the weight its prefill GEMM reads.  Here only large-batch calls use it, the same way:
    the weight is decoded once per call into it and both operands reach the tensor cores by TMA."""
    dev = torch.device(device)
    if dev.index is None and dev.type == "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    ws = _GLOBAL_WORKSPACE.get(dev)
    if ws is None or ws.numel() < _WORKSPACE_BYTES:
        ws = _GLOBAL_WORKSPACE[dev] = torch.empty(_WORKSPACE_BYTES, dtype=torch.int8, device=dev)
    return ws


def quant_input(input: torch.Tensor):
    """Per-token absmax int8 quantisation (model.py:120-123):
    s = 127 / clamp(max|x|, 1e-5); x_q = clamp(round(x*s), -128, 127)."""
    s = 127 / input.abs().max(dim=-1, keepdim=True).values.clamp_(min=1e-5)
    return (input * s).round().clamp(-128, 127).to(torch.int8), s


def _builtin_segments(segments, out_features, ws_num):
    """Whether explicit scale-segment lengths say the same as the reference's built-in rule (equal
    widths, or 2560/640/640 for 3840 outputs with three scales), which is what the entry points
    without segment arguments apply."""
    if segments is None or len(segments) <= 1:
        return True
    if ws_num == 3 and out_features == 3840:
        return list(segments) == [2560, 640, 640]
    return out_features % ws_num == 0 and all(v == out_features // ws_num for v in segments)


_ENTRY = {"auto": "bitlinear_TernaSpMM", "decode": "bitlinear_TernaSpMM_decode",
          "prefill": "bitlinear_TernaSpMM_prefill"}


def rmsnorm_quant(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, gated: bool = False):
    """One fused kernel for RMSNorm(x) * weight followed by ``quant_input``
    (``gated``: x holds [x1 | x3] and the normalised value is relu(x1)^2 * x3).
    bf16 [..., K or 2K] -> (int8 [..., K], bf16 scale [..., 1])."""
    if not x.is_cuda:
        raise RuntimeError("rmsnorm_quant needs CUDA tensors: the B200 library has no CPU path")
    lib = load_library()
    K = norm_weight.shape[0]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    M = x2.shape[0]
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M, 1), dtype=torch.bfloat16, device=x.device)
    fn = lib.ternaspmm_relu2_gate_rmsnorm_quant if gated else lib.ternaspmm_rmsnorm_quant
    fn(x2.data_ptr(), norm_weight.data_ptr(), float(eps), M, K, q.data_ptr(), s.data_ptr(),
       torch.cuda.current_stream().cuda_stream)
    return q.reshape(*x.shape[:-1], K), s.reshape(*x.shape[:-1], 1)


def rmsnorm(x: torch.Tensor, norm_weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm(x) * weight in one kernel, in the summation order of ``rmsnorm_quant``; bf16 in, bf16 out."""
    if not x.is_cuda:
        raise RuntimeError("rmsnorm needs CUDA tensors: the B200 library has no CPU path")
    lib = load_library()
    K = norm_weight.shape[0]
    x2 = x.reshape(-1, K).contiguous()
    y = torch.empty_like(x2)
    lib.ternaspmm_rmsnorm(x2.data_ptr(), norm_weight.data_ptr(), float(eps), x2.shape[0], K, y.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
    return y.reshape(x.shape)


_HEAD_SCRATCH = {}


def lm_head_argmax(h: torch.Tensor, embedding: torch.Tensor, want_logits: bool = True, want_argmax: bool = True):
    """Output head for up to 8 rows: (fp32 logits [M, V] or None, int64 greedy tokens [M] or None).
    One kernel that reads the embedding once; the logits carry the bf16 rounding of the reference's
    bf16 linear and the arg-max is taken over them (smallest index on ties)."""
    if not h.is_cuda:
        raise RuntimeError("lm_head_argmax needs CUDA tensors: the B200 library has no CPU path")
    lib = load_library()
    V, K = embedding.shape
    h2 = h.reshape(-1, K).contiguous()
    M = h2.shape[0]
    assert 1 <= M <= 8 and h2.dtype == torch.bfloat16 and embedding.dtype == torch.bfloat16 and embedding.is_contiguous()
    dev = h.device
    scratch = _HEAD_SCRATCH.get(dev)
    if scratch is None:   # one zero-initialised scratch area per device (calls on one device run in stream order)
        scratch = _HEAD_SCRATCH[dev] = torch.zeros(int(lib.ternaspmm_lm_head_scratch_bytes()), dtype=torch.uint8, device=dev)
    logits = torch.empty((M, V), dtype=torch.float32, device=dev) if want_logits else None
    tokens = torch.empty((M,), dtype=torch.int64, device=dev) if want_argmax else None
    lib.ternaspmm_lm_head_argmax(h2.data_ptr(), embedding.data_ptr(), M, V, K,
                                 logits.data_ptr() if want_logits else None,
                                 tokens.data_ptr() if want_argmax else None, 1, scratch.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    return logits, tokens


def TernaInfer_linear(input, compressed_val, TileOffsets_global, TileOffsets_median, bitmap,
                      workspace, s, ws, ws_num, out_features, mode: str = "auto", residual=None, segments=None):
    """out = TernaSpMM(input_int8, packed weight) as bf16 (model.py:45-92).
    ``input`` is int8 [..., K] on the GPU, ``s`` its per-token bf16 scale,
    ``ws`` the 4-slot bf16 weight scale with ``ws_num`` non-zero slots.
    ``segments`` (optional, not in the reference): lengths of the scale segments;
    without it the reference's built-in rule decides (equal widths, or
    2560/640/640 for 3840 outputs)."""
    if not input.is_cuda:
        raise RuntimeError("TernaInfer_linear needs CUDA tensors: the B200 library has no CPU path")
    lib = load_library()
    out_shape = list(input.shape)
    out_shape[-1] = out_features
    K = input.shape[-1]
    M = input.numel() // K
    x2 = input.reshape(M, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if s.dtype != torch.bfloat16:
        s = s.to(torch.bfloat16)
    s = s.contiguous()
    ret = torch.empty((M, out_features), dtype=torch.bfloat16, device=input.device)
    stream = torch.cuda.current_stream()
    if (workspace is not None and mode == "auto" and M > 64 and _builtin_segments(segments, out_features, ws_num)
            and workspace.numel() * workspace.element_size() >= out_features * K):
        # large batch with the reference-sized workspace: decode once into it, both operands by TMA
        res = None
        if residual is not None:
            res = residual.reshape(M, out_features)
            assert res.is_contiguous() and res.dtype == torch.bfloat16
        lib.bitlinear_TernaSpMM_ws(x2.data_ptr(), bitmap.data_ptr(), TileOffsets_global.data_ptr(),
                                   TileOffsets_median.data_ptr(), compressed_val.data_ptr(), ret.data_ptr(), s.data_ptr(),
                                   ws.data_ptr(), ws_num, M, out_features, K, res.data_ptr() if res is not None else None,
                                   workspace.data_ptr(), workspace.numel() * workspace.element_size(), 0, stream.cuda_stream)
        return ret.reshape(*out_shape)
    if segments is not None and len(segments) > 1 and residual is None:
        bounds = [sum(segments[:i + 1]) for i in range(len(segments) - 1)] + [2 ** 31 - 1] * 3
        form = {"auto": -1, "decode": 0, "prefill": 1}[mode]
        lib.ternaspmm_linear_segments(x2.data_ptr(), bitmap.data_ptr(), TileOffsets_global.data_ptr(),
                                      TileOffsets_median.data_ptr(), compressed_val.data_ptr(), ret.data_ptr(),
                                      s.data_ptr(), ws.data_ptr(), ws_num, M, out_features, K, bounds[0], bounds[1],
                                      bounds[2], form, stream.cuda_stream)
        return ret.reshape(*out_shape)
    if residual is not None:
        res = residual.reshape(M, out_features)
        assert mode == "auto" and res.is_contiguous() and res.dtype == torch.bfloat16
        lib.bitlinear_TernaSpMM_residual(x2.data_ptr(), bitmap.data_ptr(), TileOffsets_global.data_ptr(),
                                         TileOffsets_median.data_ptr(), compressed_val.data_ptr(), ret.data_ptr(),
                                         s.data_ptr(), ws.data_ptr(), ws_num, M, out_features, K, res.data_ptr(),
                                         stream.cuda_stream)
        return ret.reshape(*out_shape)
    getattr(lib, _ENTRY[mode])(
        ctypes.c_void_p(x2.data_ptr()),
        ctypes.c_void_p(bitmap.data_ptr()),
        ctypes.c_void_p(TileOffsets_global.data_ptr()),
        ctypes.c_void_p(TileOffsets_median.data_ptr()),
        ctypes.c_void_p(compressed_val.data_ptr()),
        ctypes.c_void_p(ret.data_ptr()),
        ctypes.c_void_p(s.data_ptr()),
        ctypes.c_void_p(ws.data_ptr()),
        ctypes.c_int(ws_num),
        ctypes.c_int(M), ctypes.c_int(out_features), ctypes.c_int(K),
        ctypes.c_int(1), ctypes.c_void_p(workspace.data_ptr() if workspace is not None else 0),
        ctypes.c_void_p(stream.cuda_stream),
    )
    return ret.reshape(*out_shape)


class SpBitLinear(nn.Module):
    """Ternary linear layer bound to packed checkpoint tensors (model.py:96-133):
    ``<key>.weight_compressed_val`` (uint32), ``_TileOffsets_global`` (int32),
    ``_TileOffsets_median`` (uint16), ``_bitmap`` (uint64), ``.weight_scale``
    (bf16[4])."""

    def __init__(self, in_features: int, out_features: int, dic: dict, key: str, bias: bool = False):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        dev = "cuda"
        self.weight_compressed_val = nn.Parameter(dic[key + ".weight_compressed_val"].to(dev), requires_grad=False)
        self.weight_TileOffsets_global = nn.Parameter(dic[key + ".weight_TileOffsets_global"].to(dev),
                                                      requires_grad=False)
        self.weight_TileOffsets_median = nn.Parameter(dic[key + ".weight_TileOffsets_median"].to(dev),
                                                      requires_grad=False)
        self.weight_bitmap = nn.Parameter(dic[key + ".weight_bitmap"].to(dev), requires_grad=False)
        ws = dic[key + ".weight_scale"]
        self.weight_scale = nn.Parameter(ws.to(dev), requires_grad=False)
        self.ws_num = int((ws != 0).sum().item())
        # explicit scale-segment lengths when the checkpoint carries them (written by this
        # library's converter); absent in checkpoints converted by the reference
        seg = dic.get(key + ".weight_segments")
        self.segments = [int(v) for v in seg] if seg is not None else None
        if self.segments is not None:
            assert sum(self.segments) == out_features and len(self.segments) == self.ws_num

    quant_input = staticmethod(quant_input)

    def forward_quantized(self, input_q, s, residual=None):
        """Already quantised input (int8 + per-token scale), optional fused residual add."""
        return TernaInfer_linear(
            input_q,
            self.weight_compressed_val, self.weight_TileOffsets_global, self.weight_TileOffsets_median,
            self.weight_bitmap, get_global_workspace(input_q.device), s, self.weight_scale, self.ws_num, self.out_features,
            residual=residual, segments=self.segments)

    def forward(self, input):
        input, s = quant_input(input)
        return TernaInfer_linear(
            input,
            self.weight_compressed_val, self.weight_TileOffsets_global, self.weight_TileOffsets_median,
            self.weight_bitmap,
            get_global_workspace(input.device),
            s, self.weight_scale, self.ws_num,
            self.out_features, segments=self.segments,
        )
