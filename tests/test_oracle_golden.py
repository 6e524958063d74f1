"""CPU: the oracle against the reference packer's golden vectors and against
the reference's procedural known answer."""
import os

import numpy as np
import pytest

import ternaspmm_oracle as o
import c_oracle

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_packer_golden.npz"))
NAMES = sorted({k.split("/")[0] for k in GOLD.files})


@pytest.mark.parametrize("name", NAMES)
def test_reference_layout_matches_reference_packer(name):
    w = GOLD[name + "/w"]
    assert (o.reorder_weight_ref(w) == GOLD[name + "/reordered"]).all()
    cv, tg, tm, bm = o.compress_weight_ref(w)
    for mine, key in ((cv, "compressed_val"), (tg, "tile_offsets"), (tm, "median_offsets"), (bm, "bitmap")):
        ref = GOLD[name + "/" + key]
        assert mine.shape == ref.shape and mine.dtype == ref.dtype and (mine == ref).all(), key
    N, K = w.shape
    assert (o.decode_weight_ref(cv, tg, tm, bm, N, K) == w).all()


@pytest.mark.parametrize("name", ["t64x64_p45", "t128x192_p45", "t192x64_p00"])
def test_lanewise_kernel_emulation_reconstructs_weights(name):
    w = GOLD[name + "/w"]
    N, K = w.shape
    got = o.decode_weight_ref_lanewise(GOLD[name + "/compressed_val"], GOLD[name + "/tile_offsets"],
                                       GOLD[name + "/median_offsets"], GOLD[name + "/bitmap"], N, K)
    assert (got == w).all()


def test_known_answer_all_ones_activations():
    # tests/test_kernel.cu of the reference: x == 1, s == 1, ws == 1 -> out = row sums of W
    M, N, K = 8, 256, 320
    w = o.make_ternary(N, K, 0.45, seed=7)
    xq = np.ones((M, K), np.int8)
    one = np.ones(M, np.float32)
    ws = np.ones(4, np.float32)
    out = o.bf16_bits_to_f32(o.ternaspmm(xq, w, one, ws, 4))
    want = np.broadcast_to(w.sum(axis=1, dtype=np.int32).astype(np.float32), (M, N))
    assert (out == o.bf16_round(want)).all()


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e38, 0.0, 1e-40], np.float32)
    import torch
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert (o.f32_to_bf16_bits(x) == want).all()
    r = np.random.default_rng(0).standard_normal(10000).astype(np.float32) * 100
    want = torch.from_numpy(r).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert (o.f32_to_bf16_bits(r) == want).all()


def test_scale_group_rules():
    n = np.arange(3840)
    g = o.ws_group_decode(n, 3840, 3)
    assert g[0] == 0 and g[2559] == 0 and g[2560] == 1 and g[3199] == 1 and g[3200] == 2 and g[3839] == 2
    g = o.ws_group_prefill(n, 3840, 3)
    assert g[2559] == 0 and g[2560] == 1 and g[3200] == 2
    n = np.arange(13824)
    assert (o.ws_group_decode(n, 13824, 2) == (n >= 6912)).all()
    # prefill picks the group of the 128-column block's first column and clamps
    g = o.ws_group_prefill(np.arange(192), 192, 3)
    assert (g[:128] == 0).all() and (g[128:] == 2).all()
    assert o.ws_group_prefill(np.arange(2560), 2560, 4).max() == 3


@pytest.mark.parametrize("M,N,K,ws_num", [(8, 128, 192, 1), (70, 192, 128, 3), (16, 3840, 64, 3)])
def test_c_oracle_equals_numpy_oracle(M, N, K, ws_num):
    w = o.make_ternary(N, K, 0.45, seed=11)
    xq, s = o.make_activations(M, K, seed=12)
    ws = o.make_ws(ws_num, seed=13)
    acc, out = c_oracle.ternaspmm(xq, w, o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws), ws_num)
    ref = o.gemm_i32(xq, w)
    assert (acc == ref).all()
    assert (out == o.ternaspmm(xq, w, s, ws, ws_num)).all()
    for mode, name in ((0, "decode"), (1, "prefill")):
        _, out = c_oracle.ternaspmm(xq, w, o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws), ws_num, mode)
        assert (out == o.ternaspmm(xq, w, s, ws, ws_num, name)).all()


def test_gemm_matches_integer_loop_on_a_small_case():
    w = o.make_ternary(64, 64, 0.3, seed=3)
    rng = np.random.default_rng(4)
    xq = rng.integers(-128, 128, size=(5, 64), dtype=np.int8)
    want = np.array([[sum(int(a) * int(b) for a, b in zip(xr, wr)) for wr in w] for xr in xq], np.int32)
    assert (o.gemm_i32(xq, w) == want).all()


def test_quant_input_matches_torch_eager_bf16():
    import torch
    torch.manual_seed(0)
    x = torch.randn(9, 320).to(torch.bfloat16)
    s = 127 / x.abs().max(dim=-1, keepdim=True).values.clamp_(min=1e-5)
    xq = (x * s).round().clamp(-128, 127).to(torch.int8)
    oxq, os_ = o.quant_input(x.float().numpy())
    assert (oxq == xq.numpy()).all()
    assert (os_ == s.float().numpy()).all()


def test_weight_ternarisation_rule():
    rng = np.random.default_rng(5)
    w = rng.standard_normal((64, 64)).astype(np.float32) * 0.02
    wt, scale = o.quant_weight_ternary(w)
    assert set(np.unique(wt)) <= {-1, 0, 1}
    assert abs(float(scale[0]) - float(np.abs(w).mean())) / float(np.abs(w).mean()) < 2 ** -8
