"""Tensor-parallel sharding of the ternary linears (one process per GPU).

The reference is single-GPU (``local_rank = 0`` is hard-coded, generate.py:361
of Gu-J/TernaInfer); this is the sharding for models that do not fit or are
too batch-heavy for one chip: the fused QKV and gate-up linears are split by
output rows (column-parallel, no collective, activations replicated), the O
and down linears by input columns (row-parallel, ONE all-reduce each).

Row-parallel detail.  In front of ``wo`` / ``w2`` sit a sub-layer RMSNorm over
the full width and the per-token absmax quantiser, both of which need
cross-rank statistics.  Two modes:

``single`` (default) - one collective per linear.  Each rank quantises its
    un-normalised slice ``x_r * g_r`` with its *local* absmax, multiplies on the
    GPU, divides by its own scale and appends its partial sums of squares; a
    single fp32 all-reduce of M*N + M values carries everything and the RMS
    factor and weight scale are applied after.  On the GPU this is three
    launches around the collective (``ternaspmm_scale_quant_sumsq`` ->
    ``ternaspmm_partial_f32`` -> all-reduce -> ``ternaspmm_tp_finish``, the last
    one also adding the residual stream).  Mathematically identical to the
    unsharded layer, numerically within bf16 rounding of it (each rank rounds
    with its own scale).
``fused`` - the arithmetic of ``single`` with the collective inside the last
    kernel: partials and outputs live in symmetric memory that every rank has
    mapped (``torch.distributed._symmetric_memory``), and
    ``ternaspmm_tp_allreduce_finish`` is a reduce-scatter plus all-gather in one
    launch: it signals the peers, waits for them (bounded), reduces this rank's
    slice of the outputs over all ranks' partials with plain loads over NVLink,
    applies the RMS factor and weight scale, pushes the finished bf16 slice to
    every rank and waits for the peers' slices.  Three launches per linear, no
    NCCL kernel.  Every output element is computed by exactly one rank, so all
    ranks hold identical activations.  Needs ``max_tokens`` at construction
    (buffer size).  The returned tensor is a view of the call site's symmetric
    output buffer: it is overwritten by the next call of the same module.
    After a step, ``check_status()`` raises if a device-side wait ran out.
``exact`` - bit-identical to the unsharded layer: all-reduce the sum of
    squares, normalise, all-reduce (max) the absmax, quantise with the global
    scale, all-reduce the int32 accumulators, then apply the decode epilogue.
    Three collectives, two of them a few hundred bytes.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import torch
import torch.distributed as dist
from torch import nn

from .convert import compress_weight
from .lib import load_library


# ----------------------------------------------------------------- sharding
def shard_rows(w: torch.Tensor, segments: Sequence[int], rank: int, tp: int) -> torch.Tensor:
    """Column-parallel shard: rank r keeps rows [r*len/tp, (r+1)*len/tp) of every
    segment (q, k, v / gate, up), concatenated in segment order."""
    out, start = [], 0
    for seg in segments:
        assert seg % tp == 0, "segment length must divide by the tensor-parallel size"
        step = seg // tp
        out.append(w[start + rank * step: start + (rank + 1) * step])
        start += seg
    return torch.cat(out, dim=0).contiguous()


def shard_cols(w: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """Row-parallel shard: rank r keeps input columns [r*K/tp, (r+1)*K/tp)."""
    K = w.shape[1]
    assert K % (64 * tp) == 0, "K/tp must be a multiple of 64"
    return w[:, rank * (K // tp):(rank + 1) * (K // tp)].contiguous()


def shard_vector(v: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    n = v.shape[0]
    return v[rank * (n // tp):(rank + 1) * (n // tp)].contiguous()


def local_segments(segments: Sequence[int], tp: int) -> List[int]:
    return [s // tp for s in segments]


# ------------------------------------------------------------ kernel calls
def _accumulate_i32(xq: torch.Tensor, packed, N: int) -> torch.Tensor:
    """int8 [M, K] x packed weight -> int32 accumulators [M, N] on the GPU."""
    if not xq.is_cuda:
        raise RuntimeError("the TernaSpMM library has no CPU path")
    lib = load_library()
    cv, tg, tm, bm = packed
    M, K = xq.shape
    out = torch.empty((M, N), dtype=torch.int32, device=xq.device)
    lib.ternaspmm_accumulate_i32(xq.data_ptr(), bm.data_ptr(), tg.data_ptr(), tm.data_ptr(), cv.data_ptr(),
                                 out.data_ptr(), M, N, K, torch.cuda.current_stream().cuda_stream)
    return out


def _linear_segments(xq, s, packed, ws, bounds, N: int) -> torch.Tensor:
    if not xq.is_cuda:
        raise RuntimeError("the TernaSpMM library has no CPU path")
    lib = load_library()
    cv, tg, tm, bm = packed
    M, K = xq.shape
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    b = list(bounds) + [2 ** 31 - 1] * (3 - len(bounds))
    lib.ternaspmm_linear_segments(xq.data_ptr(), bm.data_ptr(), tg.data_ptr(), tm.data_ptr(), cv.data_ptr(),
                                  out.data_ptr(), s.data_ptr(), ws.data_ptr(), len(bounds) + 1, M, N, K,
                                  b[0], b[1], b[2], -1, torch.cuda.current_stream().cuda_stream)
    return out


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _quant_fused(x2: torch.Tensor):
    """Per-token absmax int8 quantiser as one kernel (``ternaspmm_quant``)."""
    lib = load_library()
    M, K = x2.shape
    xq = torch.empty((M, K), dtype=torch.int8, device=x2.device)
    s = torch.empty((M, 1), dtype=torch.bfloat16, device=x2.device)
    lib.ternaspmm_quant(x2.data_ptr(), M, K, xq.data_ptr(), s.data_ptr(), _stream())
    return xq, s


def _quant(x: torch.Tensor, amax: torch.Tensor = None):
    if amax is None:
        amax = x.abs().max(dim=-1, keepdim=True).values
    s = 127 / amax.clamp(min=1e-5)
    return (x * s).round().clamp(-128, 127).to(torch.int8), s


def check_status():
    """Raise if the library recorded an error since the last check - in particular status 4: a
    bounded device-side wait for a peer ran out and the step's outputs were poisoned with NaN.
    Synchronises the device; call it once per step outside any graph capture."""
    st = load_library().ternaspmm_last_status()
    if st != 0:
        raise RuntimeError(f"TernaSpMM library status {st}" + (" (a wait for a peer rank timed out)" if st == 4 else ""))


def announce_leaving(store, rank: int):
    """Tell the other ranks, through the rendezvous store (host side), that this rank leaves the group.
    Call it between steps, with none of this rank's kernels or collectives in flight."""
    store.set(f"tp_rank_left_{rank}", "1")


def check_peers(store, rank: int, world: int):
    """Raise before the next launch if a peer has announced that it left: a step whose collective or
    fused tail waited for that peer would end in a time-out (status 4) or an error from the
    process group instead.  Host side only: one store query per peer."""
    for r in range(world):
        if r != rank and store.check([f"tp_rank_left_{r}"]):
            raise RuntimeError(f"tensor-parallel rank {r} has left the group")


class _PeerBuffers:
    """One call site's symmetric memory: ``numel`` floats of partials, 16 uint32 flags and
    ``out_numel`` bf16 outputs, mapped into every rank of ``group``, plus two local counters.
    Construction is collective (every rank must build its modules in the same order)."""

    def __init__(self, numel: int, out_numel: int, group, device):
        import ctypes as C
        import os
        import torch.distributed._symmetric_memory as symm_mem
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads only
        grp = group if group is not None else dist.group.WORLD
        self.numel = numel
        self.rank, self.world = dist.get_rank(grp), dist.get_world_size(grp)
        nf = (numel + 3) // 4 * 4
        no = (out_numel + 7) // 8 * 4                       # bf16 outputs, in float units, 16-byte granules
        total = nf + 16 + no                                # floats, then the flag words, then the outputs
        self.local = symm_mem.empty(total, dtype=torch.float32, device=device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, grp)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        flag_off, out_off = 4 * nf, 4 * (nf + 16)
        self.buf_ptrs = (C.c_void_p * self.world)(*ptrs)
        self.flag_ptrs = (C.c_void_p * self.world)(*[p + flag_off for p in ptrs])
        self.out_ptrs = (C.c_void_p * self.world)(*[p + out_off for p in ptrs])
        self.out_local = self.local[nf + 16:].view(torch.bfloat16)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize()
        dist.barrier(group=grp)                             # every rank's flags are zero before the first call


# ------------------------------------------------------------------ modules
class ColumnParallelSpBitLinear(nn.Module):
    """Rows of a fused linear owned by this rank.  ``dic[key + '.weight_*']``
    already hold the rank's packed shard; ``dic[key + '.weight_segments']`` the
    local segment lengths (e.g. [q/tp, k/tp, v/tp])."""

    def __init__(self, in_features: int, out_features: int, dic: dict, key: str):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        self.packed = [dic[key + s].to(dev) for s in (".weight_compressed_val", ".weight_TileOffsets_global",
                                                      ".weight_TileOffsets_median", ".weight_bitmap")]
        self.weight_scale = dic[key + ".weight_scale"].to(dev)
        segs = [int(v) for v in dic[key + ".weight_segments"]]
        assert sum(segs) == out_features
        self.bounds = [sum(segs[:i + 1]) for i in range(len(segs) - 1)]

    def forward(self, x):
        shape = list(x.shape[:-1]) + [self.out_features]
        x2 = x.reshape(-1, self.in_features)
        if x2.is_cuda and x2.dtype == torch.bfloat16:
            xq, s = _quant_fused(x2.contiguous())
        else:
            xq, s = _quant(x2)
            s = s.to(torch.bfloat16).contiguous()
        y = _linear_segments(xq, s, self.packed, self.weight_scale, self.bounds, self.out_features)
        return y.reshape(shape)


class RowParallelSpBitLinear(nn.Module):
    """Input-column shard of ``wo`` / ``w2`` with the preceding sub-layer norm
    folded in (see the module docstring).  ``norm_weight`` is this rank's slice
    of the norm weight; ``in_features`` is the local width K/tp.  With
    ``gated=True`` the input is this rank's ``[gate | up]`` block of width
    2*K/tp and relu(gate)^2 * up is formed in the same kernel (``single`` mode
    on the GPU only)."""

    def __init__(self, in_features: int, out_features: int, dic: dict, key: str, group=None,
                 norm_weight: torch.Tensor = None, eps: float = 1e-5, mode: str = "single", gated: bool = False,
                 max_tokens: int = 0):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        self.packed = [dic[key + s].to(dev) for s in (".weight_compressed_val", ".weight_TileOffsets_global",
                                                      ".weight_TileOffsets_median", ".weight_bitmap")]
        self.ws_bf16 = dic[key + ".weight_scale"].to(dev).to(torch.bfloat16).contiguous()
        self.ws = self.ws_bf16.float()[0]
        self.norm_weight_bf16 = norm_weight.to(dev).to(torch.bfloat16).contiguous()
        self.norm_weight = self.norm_weight_bf16.float()
        self.group, self.eps, self.mode, self.gated = group, eps, mode, gated
        self.tp = dist.get_world_size(group) if dist.is_initialized() else 1
        self.fused = True       # False: the torch formulation of the same arithmetic (tests compare the two)
        self._peer = None
        if mode == "fused":
            assert max_tokens > 0, "the fused collective needs max_tokens (size of the symmetric buffer)"
            self._peer = _PeerBuffers(max_tokens * out_features + max_tokens, max_tokens * out_features, group, dev)

    def _forward_fused(self, x2: torch.Tensor, residual):
        """GPU path of the ``single`` mode: three launches around one all-reduce."""
        lib = load_library()
        M, K, N = x2.shape[0], self.in_features, self.out_features
        dev = x2.device
        xq = torch.empty((M, K), dtype=torch.int8, device=dev)
        s = torch.empty((M,), dtype=torch.bfloat16, device=dev)
        buf = torch.empty((M * N + M,), dtype=torch.float32, device=dev)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        cv, tg, tm, bm = self.packed
        st = _stream()
        lib.ternaspmm_scale_quant_sumsq(x2.data_ptr(), self.norm_weight_bf16.data_ptr(), int(self.gated), M, K,
                                        xq.data_ptr(), s.data_ptr(), buf.data_ptr() + 4 * M * N, st)
        lib.ternaspmm_partial_f32(xq.data_ptr(), bm.data_ptr(), tg.data_ptr(), tm.data_ptr(), cv.data_ptr(),
                                  buf.data_ptr(), s.data_ptr(), M, N, K, st)
        if self.tp > 1:
            dist.all_reduce(buf, group=self.group)                 # the one collective of this linear
        lib.ternaspmm_tp_finish(buf.data_ptr(), self.ws_bf16.data_ptr(), self.eps, K * self.tp, M, N,
                                residual.data_ptr() if residual is not None else None, out.data_ptr(), st)
        return out

    def _forward_peer(self, x2: torch.Tensor, residual):
        """``fused`` mode: partials into the symmetric buffer, collective inside the finish kernel."""
        lib = load_library()
        M, K, N = x2.shape[0], self.in_features, self.out_features
        pb = self._peer
        assert M * N + M <= pb.numel, "more tokens than max_tokens"
        dev = x2.device
        xq = torch.empty((M, K), dtype=torch.int8, device=dev)
        s = torch.empty((M,), dtype=torch.bfloat16, device=dev)
        out = pb.out_local[:M * N].view(M, N)              # every rank's kernel writes its slice here
        cv, tg, tm, bm = self.packed
        st = _stream()
        base = pb.local.data_ptr()
        lib.ternaspmm_scale_quant_sumsq(x2.data_ptr(), self.norm_weight_bf16.data_ptr(), int(self.gated), M, K,
                                        xq.data_ptr(), s.data_ptr(), base + 4 * M * N, st)
        lib.ternaspmm_partial_f32(xq.data_ptr(), bm.data_ptr(), tg.data_ptr(), tm.data_ptr(), cv.data_ptr(),
                                  base, s.data_ptr(), M, N, K, st)
        lib.ternaspmm_tp_allreduce_finish(pb.buf_ptrs, pb.flag_ptrs, pb.out_ptrs, pb.rank, pb.world,
                                          pb.counters.data_ptr(), self.ws_bf16.data_ptr(), self.eps, K * self.tp, M, N,
                                          residual.data_ptr() if residual is not None else None, st)
        return out

    def forward(self, x, residual=None):
        shape = list(x.shape[:-1]) + [self.out_features]
        x2 = x.reshape(-1, self.in_features * (2 if self.gated else 1))
        if self.mode == "fused":
            res2 = residual.reshape(-1, self.out_features).contiguous() if residual is not None else None
            return self._forward_peer(x2.contiguous(), res2).reshape(shape)
        if self.fused and self.mode == "single" and x2.is_cuda and x2.dtype == torch.bfloat16:
            res2 = residual.reshape(-1, self.out_features).contiguous() if residual is not None else None
            return self._forward_fused(x2.contiguous(), res2).reshape(shape)
        if self.gated:
            x1, x3 = x2.chunk(2, dim=-1)
            x2 = torch.relu(x1) ** 2 * x3
        full_width = self.in_features * self.tp
        xf = x2.float()
        ss = xf.pow(2).sum(-1, keepdim=True)
        if self.mode == "exact":
            if self.tp > 1:
                dist.all_reduce(ss, group=self.group)
            y = (xf * torch.rsqrt(ss / full_width + self.eps) * self.norm_weight).to(x.dtype)
            amax = y.abs().max(dim=-1, keepdim=True).values
            if self.tp > 1:
                dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
            xq, s = _quant(y, amax)
            acc = _accumulate_i32(xq, self.packed, self.out_features)
            if self.tp > 1:
                dist.all_reduce(acc, group=self.group)
            out = (acc.float() / s.float() * self.ws).to(torch.bfloat16)
        else:
            z = (xf * self.norm_weight).to(x.dtype)               # un-normalised: the RMS factor is applied last
            xq, s = _quant(z)
            acc = _accumulate_i32(xq, self.packed, self.out_features)
            M, N = acc.shape
            buf = torch.cat([(acc.float() / s.float()).reshape(-1), ss.reshape(-1)])  # partial outputs, then sums of squares
            if self.tp > 1:
                dist.all_reduce(buf, group=self.group)             # the one collective of this linear
            rstd = torch.rsqrt(buf[M * N:].reshape(M, 1) / full_width + self.eps)
            out = (buf[:M * N].reshape(M, N) * rstd * self.ws).to(torch.bfloat16)
        if residual is not None:
            out = residual.reshape(-1, self.out_features) + out
        return out.reshape(shape)


# ------------------------------------------------- sharded checkpoint helper
def shard_checkpoint_entry(dic: dict, key: str, w_int8: torch.Tensor, ws: torch.Tensor, segments, kind: str,
                           rank: int, tp: int):
    """Pack this rank's shard of one ternary weight into ``dic`` under ``key``
    (``kind`` = 'column' or 'row')."""
    if kind == "column":
        local = shard_rows(w_int8, segments, rank, tp)
        dic[key + ".weight_segments"] = torch.tensor(local_segments(segments, tp))
    else:
        local = shard_cols(w_int8, rank, tp)
    cv, tg, tm, bm = compress_weight(local)
    dic[key + ".weight_compressed_val"], dic[key + ".weight_TileOffsets_global"] = cv, tg
    dic[key + ".weight_TileOffsets_median"], dic[key + ".weight_bitmap"] = tm, bm
    dic[key + ".weight_scale"] = ws
    return local


def shard_model_checkpoint(dic: dict, n_layers: int, rank: int, tp: int) -> dict:
    """This rank's checkpoint of a whole model from an unsharded one that still holds the ternary
    weights (``<key>.weight_int8``, as ``random_checkpoint(dense=True)`` returns them): QKV and gate-up
    column-parallel by scale segment (whole heads per rank), O and down row-parallel with the matching
    slice of the sub-layer norm weight; norms, embedding and scales are replicated."""
    out = {k: v for k, v in dic.items() if not k.startswith("layers.")}
    kinds = (("attention.wqkv", "column"), ("attention.wo", "row"), ("feed_forward.w13", "column"),
             ("feed_forward.w2", "row"))
    for i in range(n_layers):
        p = f"layers.{i}."
        for name, kind in kinds:
            key = p + name
            w = dic[key + ".weight_int8"]
            segs = dic.get(key + ".weight_segments")
            segs = [int(v) for v in segs.tolist()] if segs is not None else [w.shape[0]]
            shard_checkpoint_entry(out, key, w, dic[key + ".weight_scale"], segs, kind, rank, tp)
        out[p + "attention.attn_sub_norm.weight"] = shard_vector(dic[p + "attention.attn_sub_norm.weight"], rank, tp)
        out[p + "feed_forward.ffn_sub_norm.weight"] = shard_vector(dic[p + "feed_forward.ffn_sub_norm.weight"], rank, tp)
        out[p + "attention_norm.weight"] = dic[p + "attention_norm.weight"]
        out[p + "ffn_norm.weight"] = dic[p + "ffn_norm.weight"]
    return out

