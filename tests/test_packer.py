"""CPU: the product packers (Python and C) against the oracle's independent
restatement of the B200 tile order, round trips, the transcoder from the
reference layout, and sparsity extremes."""
import os

import numpy as np
import pytest
import torch

import ternaspmm_oracle as o
from ternainfer_b200.convert import (compress_weight, decompress_weight, transcode_reference_layout,
                                     compressed_nbytes, reorder_weight)

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_packer_golden.npz"))
NAMES = sorted({k.split("/")[0] for k in GOLD.files})


def c_pack(lib, w):
    N, K = w.shape
    tiles = N * K // 4096
    bm = np.zeros(N * K // 64, np.uint64)
    tg = np.zeros(tiles + 1, np.int32)
    tm = np.zeros(3 * tiles, np.uint16)
    cv = np.zeros(N * K // 32 + 4, np.uint32)
    nw = lib.ternaspmm_pack_i8(w.ctypes.data, N, K, bm.ctypes.data, tg.ctypes.data, tm.ctypes.data, cv.ctypes.data)
    return nw, cv, tg, tm, bm


@pytest.mark.parametrize("name", NAMES)
def test_python_and_c_packers_match_oracle(lib, name):
    w = GOLD[name + "/w"]
    N, K = w.shape
    ocv, otg, otm, obm = o.compress_weight_b200(w)
    cv, tg, tm, bm = compress_weight(torch.from_numpy(w))
    assert cv.dtype == torch.uint32 and tg.dtype == torch.int32 and tm.dtype == torch.uint16 and bm.dtype == torch.uint64
    assert cv.numel() == ocv.size + 4 and (cv.numpy()[:ocv.size] == ocv).all() and (cv.numpy()[ocv.size:] == 0).all()
    assert (tg.numpy() == otg).all() and (tm.numpy() == otm).all() and (bm.numpy() == obm).all()
    assert (decompress_weight(cv, tg, tm, bm, N, K).numpy() == w).all()
    nw, ccv, ctg, ctm, cbm = c_pack(lib, w)
    assert nw == ocv.size and (ccv[:nw] == ocv).all() and (ctg == otg).all() and (ctm == otm).all() and (cbm == obm).all()
    w2 = np.zeros_like(w)
    assert lib.ternaspmm_unpack_i8(cbm.ctypes.data, ctg.ctypes.data, ccv.ctypes.data, N, K, w2.ctypes.data) == 0
    assert (w2 == w).all()


@pytest.mark.parametrize("name", NAMES)
def test_transcode_from_reference_layout(lib, name):
    w = GOLD[name + "/w"]
    N, K = w.shape
    want = compress_weight(torch.from_numpy(w))
    ref = [np.ascontiguousarray(GOLD[name + "/" + k]) for k in
           ("compressed_val", "tile_offsets", "median_offsets", "bitmap")]
    got = transcode_reference_layout(*ref)
    for a, b in zip(got, want):
        assert (a.numpy() == b.numpy()).all()
    # sizes are identical in both layouts, so are the algorithmic bytes
    assert compressed_nbytes(*want) == o.compressed_bytes(*ref)
    obm = np.zeros_like(ref[3])
    otm = np.zeros_like(ref[2])
    ocv = np.zeros(ref[0].size + 4, np.uint32)
    rc = lib.ternaspmm_transcode_reference_layout(ref[3].ctypes.data, ref[1].ctypes.data, ref[0].ctypes.data, N, K,
                                                  obm.ctypes.data, otm.ctypes.data, ocv.ctypes.data)
    assert rc == 0
    assert (obm == want[3].numpy()).all() and (otm == want[2].numpy()).all() and (ocv == want[0].numpy()).all()


@pytest.mark.parametrize("p_zero", [0.0, 0.45, 0.9, 1.0])
def test_round_trip_sparsity_extremes(p_zero):
    w = o.make_ternary(128, 256, p_zero, seed=21)
    packed = compress_weight(torch.from_numpy(w))
    assert (decompress_weight(*packed, 128, 256).numpy() == w).all()
    tg = packed[1].numpy()
    assert (tg % 32 == 0).all() and tg[0] == 0
    nnz = int((w != 0).sum())
    assert nnz <= tg[-1] < nnz + 32 * (len(tg) - 1) + 1


def test_bits_per_weight_at_benchmark_sparsity():
    w = o.make_ternary(2560, 2560, 0.45, seed=1234)
    b = compressed_nbytes(*compress_weight(torch.from_numpy(w)))
    assert abs(b * 8 / w.size - 1.5733) < 0.003


def test_packer_rejects_bad_shapes(lib):
    with pytest.raises(AssertionError):
        compress_weight(torch.zeros(60, 64, dtype=torch.int8))
    w = np.zeros((64, 96), np.int8)
    assert lib.ternaspmm_pack_i8(w.ctypes.data, 64, 96, 0, 0, 0, 0) == -1
    assert reorder_weight(torch.zeros(64, 64, dtype=torch.int8)).shape == (64, 64)
