"""CPU oracle for the TernaSpMM path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain numpy, the arithmetic and the compressed-weight
format of the reference (Gu-J/TernaInfer).  It exists to check the CUDA
library; nothing in the product package imports it.  Only the tests, the
smoke check and the CPU-baseline leg of the benchmark may use it.

Parity status: the *format* half (reorder / compress / decode of the
reference layout) is pinned against golden vectors produced by the
reference's own packer (``convert/convert_utils.py``) - see
``tests/golden/make_golden.py``.  The *arithmetic* half follows the kernel
sources cited at each function; the reference ships no CPU GEMM and no stored
known-answer vectors for it, so its only procedural known answer (all-ones
activations, unit scales -> row sums of W, ``tests/test_kernel.cu:81,337-351,
414-429``) is reproduced as a test.  The prefill contraction of the reference
lives in NVIDIA/cutlass v4.3.4 (not vendored); it is an exact int8->int32
GEMM, restated here as an exact integer matrix product.

All citations are paths inside the reference repository.
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------
# bf16 helpers (numpy has no bfloat16): values are carried as float32 that are
# exactly representable in bf16, bits as uint16.
# --------------------------------------------------------------------------


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit pattern (what
    ``__float2bfloat16_rn`` does, kernels/src/SpMM/Reduction_Kernel.cuh:60)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    nan = np.isnan(x)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = rounded.astype(np.uint16)
    out[nan] = 0x7FC0
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# --------------------------------------------------------------------------
# Scales and quantisers
# --------------------------------------------------------------------------


def quant_weight_ternary(w: np.ndarray):
    """Absmean ternarisation of one weight segment
    (convert/convert_TernaInfer.py:159-163): s = 1/clamp(mean|W|,1e-5),
    W_t = clamp(round(W*s),-1,1), stored scale = bf16(1/s)."""
    w = np.asarray(w, dtype=np.float32)
    s = np.float32(1.0) / np.maximum(np.abs(w).mean(dtype=np.float32), np.float32(1e-5))
    wt = np.clip(np.rint(w * s), -1, 1).astype(np.int8)
    scale = bf16_round(np.array([np.float32(1.0) / s], dtype=np.float32))
    return wt, scale


def quant_input(x_bf16: np.ndarray):
    """Per-token absmax int8 quantisation of bf16 activations
    (model.py:120-123), evaluated op by op in bf16 like the eager reference.
    ``127 / t`` on a tensor is ``t.reciprocal() * 127`` in PyTorch, so
    s = bf16(bf16(1/clamp(max|x|,1e-5)) * 127);
    x_q = clamp(round_half_even(bf16(x*s)), -128, 127).
    (Under torch.compile the reference keeps fp32 intermediates; the C
    boundary receives x_q and s, so parity there does not depend on this.)
    ``x_bf16`` is float32 holding bf16-representable values."""
    x = np.asarray(x_bf16, dtype=np.float32)
    amax = bf16_round(np.maximum(np.abs(x).max(axis=-1, keepdims=True), np.float32(1e-5)))
    s = bf16_round(bf16_round(np.float32(1.0) / amax) * np.float32(127.0))
    prod = bf16_round(x * s)
    xq = np.clip(np.rint(prod), -128, 127).astype(np.int8)
    return xq, s


# --------------------------------------------------------------------------
# Contraction and epilogues
# --------------------------------------------------------------------------


def gemm_i32(xq: np.ndarray, wt: np.ndarray) -> np.ndarray:
    """acc[t,n] = sum_k xq[t,k]*W[n,k], exact.  |acc| <= 128*K < 2**53 so a
    float64 BLAS product is exact; this is what the tensor-core int8 MMA of
    kernels/src/SpMM/MatMulUtilities.cuh:180-192 and the CUTLASS int8 GEMM of
    kernels/src/TernaSpMM_API.cuh:166-207 compute."""
    acc = xq.astype(np.float64) @ wt.astype(np.float64).T
    return acc.astype(np.int64).astype(np.int32)


def ws_group_decode(n_idx: np.ndarray, N: int, ws_num: int) -> np.ndarray:
    """Scale-segment index of an output column on the decode path
    (kernels/src/SpMM/Reduction_Kernel.cuh:42-54).  One thread owns 8
    consecutive outputs and takes the group of the first of them."""
    col = (np.asarray(n_idx) // 8) * 8
    if ws_num == 3 and N == 3840:
        return np.where(col < 2560, 0, np.where(col < 3200, 1, 2)).astype(np.int64)
    return (col // (N // ws_num)).astype(np.int64)


def ws_group_prefill(n_idx: np.ndarray, N: int, ws_num: int) -> np.ndarray:
    """Scale-segment index on the prefill path
    (kernels/src/GEMM/epilogue_visitor_scale_ws.h:135-145): chosen once per
    128-column threadblock from the block's first column, clamped to
    ws_num-1; N == 3840 alone triggers the 2560/640/640 split."""
    col = (np.asarray(n_idx) // 128) * 128
    if N == 3840:
        g = np.where(col < 2560, 0, np.where(col < 3200, 1, 2))
    else:
        g = col // (N // ws_num)
    return np.minimum(g, ws_num - 1).astype(np.int64)


def epilogue_decode(acc: np.ndarray, s: np.ndarray, ws: np.ndarray, ws_num: int) -> np.ndarray:
    """out = bf16_rn(float(acc) / s[t] * ws[g(n)])
    (kernels/src/SpMM/Reduction_Kernel.cuh:45-61).  Returns bf16 bits."""
    M, N = acc.shape
    g = ws_group_decode(np.arange(N), N, ws_num)
    s32 = np.asarray(s, dtype=np.float32).reshape(M, 1)
    w32 = np.asarray(ws, dtype=np.float32)[g].reshape(1, N)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        v = (acc.astype(np.float32) / s32).astype(np.float32) * w32
    return f32_to_bf16_bits(v.astype(np.float32))


def epilogue_prefill(acc: np.ndarray, s: np.ndarray, ws: np.ndarray, ws_num: int) -> np.ndarray:
    """out = bf16_rn(float(acc) * (ws[g]/s[t])), 0 when s == 0
    (kernels/src/GEMM/epilogue_visitor_scale_ws.h:183-210)."""
    M, N = acc.shape
    g = ws_group_prefill(np.arange(N), N, ws_num)
    s32 = np.asarray(s, dtype=np.float32).reshape(M, 1)
    w32 = np.asarray(ws, dtype=np.float32)[g].reshape(1, N)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        coeff = np.where(s32 != 0, (w32 / s32).astype(np.float32), np.float32(0))
        v = acc.astype(np.float32) * coeff.astype(np.float32)
    return f32_to_bf16_bits(v.astype(np.float32))


def ternaspmm(xq, wt, s, ws, ws_num, mode="auto"):
    """Whole operator as the dispatcher sees it (kernels/TernaSpMM.cu:25-71):
    tokens <= 64 take the decode epilogue, more take the prefill epilogue."""
    acc = gemm_i32(xq, wt)
    if mode == "auto":
        mode = "decode" if xq.shape[0] <= 64 else "prefill"
    if mode == "decode":
        return epilogue_decode(acc, s, ws, ws_num)
    return epilogue_prefill(acc, s, ws, ws_num)


def bf16_linear_dense(xq, wt_scaled_bf16, s):
    """Dense comparator ``BF16BitLinear.forward`` (model.py:146-153):
    F.linear(x_q.bf16, W_bf16) / s with a bf16 rounding after the GEMM and
    after the division."""
    y = bf16_round((xq.astype(np.float32) @ wt_scaled_bf16.astype(np.float32).T).astype(np.float32))
    return f32_to_bf16_bits((y / np.asarray(s, np.float32).reshape(-1, 1)).astype(np.float32))


# --------------------------------------------------------------------------
# Reference compressed layout (format restatement)
# --------------------------------------------------------------------------


def _reorder_map() -> np.ndarray:
    """dst_flat -> src_flat map of the 16x16 block permutation
    (convert/convert_utils.py:8-35; C twin kernels/TernaSpMM.cu:241-280)."""
    m = np.empty(256, dtype=np.int64)
    for i in range(16):
        for k in range(16):
            ri, rk = i, (k + 1) // 2
            if i < 8:
                if k & 2:
                    ri += 8
                    rk -= 1
            else:
                rk += 8
                if (k & 2) == 0:
                    ri -= 8
                else:
                    rk -= 1
            m[ri * 16 + rk] = i * 16 + k
    return m


_RMAP = _reorder_map()


def reorder_weight_ref(w: np.ndarray) -> np.ndarray:
    """Apply the block permutation to every 16x16 block
    (convert/convert_utils.py:37-49)."""
    N, K = w.shape
    assert N % 16 == 0 and K % 16 == 0
    b = w.reshape(N // 16, 16, K // 16, 16).transpose(0, 2, 1, 3).reshape(N // 16, K // 16, 256)
    b = b[:, :, _RMAP]
    return b.reshape(N // 16, K // 16, 16, 16).transpose(0, 2, 1, 3).reshape(N, K).copy()


def unreorder_weight_ref(a: np.ndarray) -> np.ndarray:
    N, K = a.shape
    inv = np.empty(256, dtype=np.int64)
    inv[_RMAP] = np.arange(256)
    b = a.reshape(N // 16, 16, K // 16, 16).transpose(0, 2, 1, 3).reshape(N // 16, K // 16, 256)
    b = b[:, :, inv]
    return b.reshape(N // 16, K // 16, 16, 16).transpose(0, 2, 1, 3).reshape(N, K).copy()


def _ref_walk(a: np.ndarray) -> np.ndarray:
    """(tiles, 4096) view of a reordered matrix in the packer's walk order:
    64x64 tiles row-major; inside, four 16-row warp tiles; inside, four 16-wide
    K groups; inside, 2x2 8x8 blocks column-major; 8x8 row-major
    (convert/convert_utils.py:96-136)."""
    N, K = a.shape
    gm, gk = N // 64, K // 64
    v = a.reshape(gm, 4, 2, 8, gk, 4, 2, 8)  # gm, med, i, r, gk, lkg, j, c
    v = v.transpose(0, 4, 1, 5, 6, 2, 3, 7)  # gm, gk, med, lkg, j, i, r, c
    return v.reshape(gm * gk, 4096)


def _ref_unwalk(t: np.ndarray, N: int, K: int) -> np.ndarray:
    gm, gk = N // 64, K // 64
    v = t.reshape(gm, gk, 4, 4, 2, 2, 8, 8).transpose(0, 2, 5, 6, 1, 3, 4, 7)
    return v.reshape(N, K).copy()


def _pack_walked(t: np.ndarray, quarter: int = 1024):
    """Common tail of the packer: from tiles in walk order build the four
    arrays (convert/convert_utils.py:138-228): 1 bit/weight bitmaps, sign bits
    of the non-zeros (1 = negative) LSB-first in 32-bit words with every tile
    padded to a multiple of 32 values, per-tile prefix offsets in values, and
    three cumulative non-zero counts per tile (after each quarter)."""
    tiles = t.shape[0]
    nz = t != 0
    bitmap = np.packbits(nz.reshape(tiles, 64, 64), axis=-1, bitorder="little")
    bitmap = bitmap.reshape(tiles, 64, 8).copy().view("<u8").reshape(tiles * 64)
    cnt = nz.sum(axis=1).astype(np.int64)
    padded = (cnt + 31) // 32 * 32
    tile_off = np.zeros(tiles + 1, dtype=np.int64)
    np.cumsum(padded, out=tile_off[1:])
    csum = np.cumsum(nz, axis=1)
    median = np.stack([csum[:, quarter - 1], csum[:, 2 * quarter - 1], csum[:, 3 * quarter - 1]], axis=1)
    rank = csum - 1
    pos = (tile_off[:-1, None] + rank)[nz]
    neg = (t < 0)[nz]
    bits = np.zeros(int(tile_off[-1]), dtype=np.uint8)
    bits[pos] = neg
    words = np.packbits(bits.reshape(-1, 32), axis=-1, bitorder="little").view("<u4").reshape(-1)
    return (words.astype(np.uint32), tile_off.astype(np.int32),
            median.reshape(-1).astype(np.uint16), bitmap.astype(np.uint64))


def _unpack_walked(words, tile_off, bitmap, tiles):
    bm = np.ascontiguousarray(bitmap, dtype="<u8").view(np.uint8).reshape(tiles, 512)
    nz = np.unpackbits(bm, axis=-1, bitorder="little").reshape(tiles, 4096).astype(bool)
    bits = np.unpackbits(np.ascontiguousarray(words, dtype="<u4").view(np.uint8), bitorder="little")
    rank = np.cumsum(nz, axis=1) - 1
    pos = (np.asarray(tile_off[:-1], dtype=np.int64)[:, None] + rank)[nz]
    t = np.zeros((tiles, 4096), dtype=np.int8)
    t[nz] = np.where(bits[pos] == 1, -1, 1)
    return t


def compress_weight_ref(w: np.ndarray):
    """Reference packer, vectorised: returns (compressed_val u32,
    TileOffsets_global i32, TileOffsets_median u16, bitmap u64) exactly as
    ``compress_weight`` does (convert/convert_utils.py:52-228)."""
    assert w.dtype == np.int8 and w.shape[0] % 64 == 0 and w.shape[1] % 64 == 0
    return _pack_walked(_ref_walk(reorder_weight_ref(w)))


def decode_weight_ref(words, tile_off, median, bitmap, N, K) -> np.ndarray:
    """Inverse of the reference packer; equals what the kernel's fragment
    decode (kernels/src/SpMM/MatMulUtilities.cuh:79-114 with the sign
    expansion at :226-259) reconstructs."""
    t = _unpack_walked(words, tile_off, bitmap, (N // 64) * (K // 64))
    return unreorder_weight_ref(_ref_unwalk(t, N, K))


def decode_weight_ref_lanewise(words, tile_off, median, bitmap, N, K) -> np.ndarray:
    """Slow lane-by-lane emulation of the reference kernel's decode, used on
    small matrices to pin ``decode_weight_ref``: warp w of a tile starts at the
    cumulative count ``median[3*tile+w-1]`` (kernels/src/SpMM/SpMM_Kernel.cuh:
    66-68,94), lane l owns bits 2l,2l+1 of each 8x8 bitmap and finds its value
    by popcount of the lower bits (MatMulUtilities.cuh:88-110); register
    a[i][j] is the mma.m16n8k16 A fragment: row l/4+8j, k 16i+4(l%4)+0..3."""
    out = np.zeros((N, K), dtype=np.int8)
    nkb = K // 64
    for y in range(N // 64):
        for kb in range(nkb):
            g = y * nkb + kb
            start, nnz = int(tile_off[g]), int(tile_off[g + 1] - tile_off[g])
            wd = words[start // 32:(start + nnz) // 32]
            vals = np.array([-1 if (int(x) >> j) & 1 else 1 for x in wd for j in range(32)], dtype=np.int8)
            bmt = bitmap[g * 64:(g + 1) * 64]
            for warp in range(4):
                woff = 0 if warp == 0 else int(median[g * 3 + warp - 1])
                sv, sb = vals[woff:], bmt[warp * 16:warp * 16 + 16]
                for lane in range(32):
                    sp = 0
                    for i in range(4):
                        for j in range(2):
                            by = []
                            for t in range(2):
                                b = int(sb[i * 4 + j * 2 + t])
                                lo = lane * 2
                                nb = bin(b & ((1 << lo) - 1)).count("1")
                                x0 = sv[sp + nb] if (b >> lo) & 1 else 0
                                if (b >> lo) & 1:
                                    nb += 1
                                x1 = sv[sp + nb] if (b >> (lo + 1)) & 1 else 0
                                sp += bin(b).count("1")
                                by += [x0, x1]
                            row = y * 64 + warp * 16 + lane // 4 + 8 * j
                            k0 = kb * 64 + i * 16 + (lane % 4) * 4
                            out[row, k0:k0 + 4] = by
    return out


# --------------------------------------------------------------------------
# Re-tiled layout used by the sm_100a library (independent restatement, kept
# here so the product packer can be checked against something it does not
# import).  Same four arrays and sizes; only the order of the 4096 weights of
# a 64x64 tile differs: bit index = lane*128 + word*32 + nibble*4 + e with
# lane = 4g+q, row = 16*word + g + 8*(nibble&1),
# k = 16q + 8*(nibble>>2) + 4*((nibble>>1)&1) + e.
# --------------------------------------------------------------------------


def _b200_walk(w: np.ndarray) -> np.ndarray:
    N, K = w.shape
    rt, kt = N // 64, K // 64
    v = w.reshape(rt, 4, 2, 8, kt, 4, 2, 2, 4)  # rt, r, h, g, kt, q, s, kh, e
    v = v.transpose(0, 4, 3, 5, 1, 6, 7, 2, 8)  # rt, kt, g, q, r, s, kh, h, e
    return v.reshape(rt * kt, 4096)


def _b200_unwalk(t: np.ndarray, N: int, K: int) -> np.ndarray:
    rt, kt = N // 64, K // 64
    v = t.reshape(rt, kt, 8, 4, 4, 2, 2, 2, 4).transpose(0, 4, 7, 2, 1, 3, 5, 6, 8)
    return v.reshape(N, K).copy()


def compress_weight_b200(w: np.ndarray):
    assert w.dtype == np.int8 and w.shape[0] % 64 == 0 and w.shape[1] % 64 == 0
    return _pack_walked(_b200_walk(w))


def decode_weight_b200(words, tile_off, median, bitmap, N, K) -> np.ndarray:
    t = _unpack_walked(words, tile_off, bitmap, (N // 64) * (K // 64))
    return _b200_unwalk(t, N, K)


def compressed_bytes(words, tile_off, median, bitmap) -> int:
    """Algorithmic size of a packed weight: bitmap + sign words + offsets."""
    tiles = len(tile_off) - 1
    return int(bitmap.size * 8 + int(tile_off[-1]) // 8 + 4 * (tiles + 1) + 6 * tiles)


# --------------------------------------------------------------------------
# Seeded synthetic inputs of the benchmark configurations
# --------------------------------------------------------------------------


def make_ternary(N, K, p_zero=0.45, seed=1234) -> np.ndarray:
    rng = np.random.default_rng(seed)
    r = rng.random((N, K))
    sign = rng.integers(0, 2, size=(N, K), dtype=np.int8) * 2 - 1
    return np.where(r < p_zero, 0, sign).astype(np.int8)


def make_activations(M, K, seed=1235):
    rng = np.random.default_rng(seed)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    return quant_input(x)


def make_ws(ws_num, seed=1236):
    rng = np.random.default_rng(seed)
    ws = np.zeros(4, dtype=np.float32)
    ws[:ws_num] = bf16_round(rng.uniform(0.01, 0.05, size=ws_num).astype(np.float32))
    return ws
