"""Weight packer for the B200 TernaSpMM layout.

Mirrors the interface of the reference's ``convert/convert_utils.py``
(``reorder_weight`` :8-49, ``compress_weight`` :52-228 in Gu-J/TernaInfer):
``compress_weight(weight_int8)`` returns the same four tensors with the same
dtypes and shapes - ``compressed_val`` (uint32), ``TileOffsets_global``
(int32), ``TileOffsets_median`` (uint16, three per 64x64 tile) and ``bitmap``
(uint64) - so checkpoints keep their schema.  What changes is the order of the
4096 weights inside a tile, which follows the lane/word/nibble order the
sm_100a kernels decode (see ``csrc/packer_host.cu``), and the speed: the
packing is vectorised instead of looping over 8x8 blocks in Python.

``compressed_val`` carries four extra zero words so that a 16-byte aligned
bulk copy of the last tile's sign words stays inside the tensor.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np
import torch

_PAD_WORDS = 4


def reorder_weight(weight: torch.Tensor) -> torch.Tensor:
    """Kept for interface parity with the reference: the B200 layout needs no
    separate 16x16 block permutation, so this returns the weight unchanged."""
    assert weight.dtype == torch.int8
    assert weight.shape[0] % 16 == 0 and weight.shape[1] % 16 == 0, "Must be a multiple of 16"
    return weight.clone()


def _tile_view(w: np.ndarray) -> np.ndarray:
    """[N,K] -> [tiles, 4096] in tile bit order: lane(g,q) > word r > nibble
    (s,kh,h) > e, with row = 16r+8h+g and k = 16q+8s+4kh+e."""
    N, K = w.shape
    rt, kt = N // 64, K // 64
    v = w.reshape(rt, 4, 2, 8, kt, 4, 2, 2, 4)   # rt r h g kt q s kh e
    return v.transpose(0, 4, 3, 5, 1, 6, 7, 2, 8).reshape(rt * kt, 4096)


def _tile_unview(t: np.ndarray, N: int, K: int) -> np.ndarray:
    rt, kt = N // 64, K // 64
    v = t.reshape(rt, kt, 8, 4, 4, 2, 2, 2, 4)   # rt kt g q r s kh h e
    return v.transpose(0, 4, 7, 2, 1, 3, 5, 6, 8).reshape(N, K)


def _pack_tiles(t: np.ndarray):
    tiles = t.shape[0]
    nz = t != 0
    bitmap = np.packbits(nz, axis=-1, bitorder="little").reshape(tiles * 64, 8).view("<u8").reshape(-1)
    csum = np.cumsum(nz, axis=1, dtype=np.int32)
    cnt = csum[:, -1].astype(np.int64)
    tile_off = np.zeros(tiles + 1, dtype=np.int64)
    np.cumsum((cnt + 31) // 32 * 32, out=tile_off[1:])
    quarters = csum[:, [1023, 2047, 3071]].astype(np.uint16).reshape(-1)
    total = int(tile_off[-1])
    bits = np.zeros(total + 32 * _PAD_WORDS, dtype=np.uint8)
    pos = (tile_off[:-1, None] + csum - 1)[nz]
    bits[pos] = (t < 0)[nz]
    words = np.packbits(bits, bitorder="little").view("<u4")
    return words, tile_off.astype(np.int32), quarters, bitmap


def _compress_weight_cuda(weight: torch.Tensor):
    """Same packing with torch ops on the GPU (used for large models)."""
    N, K = weight.shape
    rt, kt = N // 64, K // 64
    dev = weight.device
    t = weight.reshape(rt, 4, 2, 8, kt, 4, 2, 2, 4).permute(0, 4, 3, 5, 1, 6, 7, 2, 8).reshape(rt * kt, 4096)
    tiles = t.shape[0]
    nz = t != 0
    pow2 = torch.ones(32, dtype=torch.int64, device=dev) << torch.arange(32, dtype=torch.int64, device=dev)

    def pack32(bits):  # [..., 32] bool -> uint32 words (as int32 bit patterns)
        v = (bits.to(torch.int64) * pow2).sum(-1)
        return torch.where(v >= 2 ** 31, v - 2 ** 32, v).to(torch.int32)

    bm_words = pack32(nz.reshape(tiles, 128, 32)).reshape(-1)
    csum = nz.cumsum(1, dtype=torch.int32)
    cnt = csum[:, -1].to(torch.int64)
    tile_off = torch.zeros(tiles + 1, dtype=torch.int64, device=dev)
    tile_off[1:] = ((cnt + 31) // 32 * 32).cumsum(0)
    quarters = csum[:, [1023, 2047, 3071]].to(torch.int16).reshape(-1)
    total = int(tile_off[-1].item())
    bits = torch.zeros(total + 32 * _PAD_WORDS, dtype=torch.bool, device=dev)
    pos = (tile_off[:-1, None] + csum.to(torch.int64) - 1)[nz]
    bits[pos] = (t < 0)[nz]
    words = pack32(bits.reshape(-1, 32))
    return (words.view(torch.uint32), tile_off.to(torch.int32), quarters.view(torch.uint16),
            bm_words.reshape(-1, 2).contiguous().view(torch.int64).reshape(-1).view(torch.uint64))


def compress_weight(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """int8 ternary [N, K] (N, K multiples of 64) -> (compressed_val,
    TileOffsets_global, TileOffsets_median, bitmap).  CPU tensors are packed
    with numpy, CUDA tensors on the GPU; results stay on the input's device."""
    assert weight.dtype == torch.int8 and weight.dim() == 2
    N, K = weight.shape
    assert N % 64 == 0 and K % 64 == 0, "N and K must be multiples of 64"
    if weight.is_cuda:
        return _compress_weight_cuda(weight.detach().contiguous())
    w = weight.detach().contiguous().numpy()
    words, tile_off, quarters, bitmap = _pack_tiles(_tile_view(w))
    return (torch.from_numpy(words.astype(np.uint32)), torch.from_numpy(tile_off),
            torch.from_numpy(quarters.copy()), torch.from_numpy(bitmap.astype(np.uint64)))


def _unpack_tiles(words: np.ndarray, tile_off: np.ndarray, bitmap: np.ndarray) -> np.ndarray:
    tiles = tile_off.shape[0] - 1
    nz = np.unpackbits(np.ascontiguousarray(bitmap, dtype="<u8").view(np.uint8).reshape(tiles, 512),
                       axis=-1, bitorder="little").astype(bool)
    bits = np.unpackbits(np.ascontiguousarray(words, dtype="<u4").view(np.uint8), bitorder="little")
    pos = (tile_off[:-1, None].astype(np.int64) + np.cumsum(nz, axis=1) - 1)[nz]
    t = np.zeros((tiles, 4096), dtype=np.int8)
    t[nz] = np.where(bits[pos] == 1, -1, 1)
    return t


def _np(x) -> np.ndarray:
    return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)


def decompress_weight(compressed_val, TileOffsets_global, TileOffsets_median, bitmap, N: int, K: int) -> torch.Tensor:
    """Inverse of :func:`compress_weight`."""
    t = _unpack_tiles(_np(compressed_val), _np(TileOffsets_global), _np(bitmap))
    return torch.from_numpy(np.ascontiguousarray(_tile_unview(t, N, K)))


# Position, in the reference's tile order, of every bit of the B200 tile order.
def _reference_bit_table() -> np.ndarray:
    b = np.arange(4096)
    lane, word, nib, e = b >> 7, (b >> 5) & 3, (b >> 2) & 7, b & 3
    g, q = lane >> 2, lane & 3
    row = 16 * word + g + 8 * (nib & 1)
    k = 16 * q + 8 * (nib >> 2) + 4 * ((nib >> 1) & 1) + e
    i, kk = row & 15, k & 15
    upper = i < 8
    odd = (kk & 2) != 0
    ri = np.where(upper, i + 8 * odd, i - 8 * (~odd))
    rk = np.where(upper, (kk + 1) // 2 - odd, (kk + 1) // 2 + 8 - odd)
    med, lkg = row >> 4, k >> 4
    return (((med * 4 + lkg) * 2 + (rk >> 3)) * 2 + (ri >> 3)) * 64 + (ri & 7) * 8 + (rk & 7)


_REF_BIT = _reference_bit_table()


def transcode_reference_layout(compressed_val, TileOffsets_global, TileOffsets_median, bitmap):
    """Arrays written by the reference's ``compress_weight`` (reorder to
    mma.m16n8k16 fragment order + 8x8 bitmap walk, convert/convert_utils.py:
    8-228) -> the same four arrays in B200 order.  Sizes do not change."""
    tile_off = _np(TileOffsets_global)
    t_ref = _unpack_tiles(_np(compressed_val), tile_off, _np(bitmap))
    words, tile_off2, quarters, bm = _pack_tiles(t_ref[:, _REF_BIT])
    assert (tile_off2 == tile_off).all()
    return (torch.from_numpy(words.astype(np.uint32)), torch.from_numpy(tile_off2),
            torch.from_numpy(quarters.copy()), torch.from_numpy(bm.astype(np.uint64)))


def compressed_nbytes(compressed_val, TileOffsets_global, TileOffsets_median, bitmap) -> int:
    """Algorithmic size in bytes: bitmaps + sign words (without the alignment
    pad) + both offset arrays."""
    tile_off = _np(TileOffsets_global)
    tiles = tile_off.shape[0] - 1
    return int(_np(bitmap).size * 8 + int(tile_off[-1]) // 8 + 4 * (tiles + 1) + 6 * tiles)
