"""GPU: the CUDA library, called through its C ABI, against the CPU oracle.

Bars: int32 accumulators bit-exact; bf16 outputs within max relative error
2**-7 of the reference formula (the implementation uses the same IEEE
operations in the same order, so the tests also assert bit equality)."""
import os

import numpy as np
import pytest
import torch

import ternaspmm_oracle as o
import c_oracle
from gpu_util import Packed, call, accumulate, inputs, max_rel_err, dev

pytestmark = pytest.mark.gpu
TOL = 2.0 ** -7

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_packer_golden.npz"))


def check(lib, M, N, K, ws_num, entry="bitlinear_TernaSpMM", p_zero=0.45, seed=100, pad=64):
    w, xq, s, ws = inputs(M, N, K, ws_num, p_zero, seed)
    pk = Packed(w)
    sb, wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
    mode = {"bitlinear_TernaSpMM": "auto", "bitlinear_TernaSpMM_decode": "decode",
            "bitlinear_TernaSpMM_prefill": "prefill"}[entry]
    want = o.ternaspmm(xq, w, s, ws, ws_num, mode)
    got = call(lib, entry, xq, pk, sb, wb, ws_num, pad=pad)
    assert lib.ternaspmm_last_status() == 0
    assert max_rel_err(got, want) <= TOL
    assert (got == want).all()
    return pk, xq


@pytest.mark.parametrize("M", [1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64])
def test_config1_shape_all_small_token_counts(lib, M):
    # the single call of the reference's kernel test: N = K = 2560, P(0) = 0.45, per-tensor scale
    check(lib, M, 2560, 2560, 1)


@pytest.mark.parametrize("M", [1, 8, 16])
@pytest.mark.parametrize("N,K,ws_num", [(3840, 2560, 3), (2560, 2560, 1), (13824, 2560, 2), (2560, 6912, 1)])
def test_bitnet2b_layer_shapes(lib, M, N, K, ws_num):
    check(lib, M, N, K, ws_num)


@pytest.mark.parametrize("M", [1, 8, 16, 32])
@pytest.mark.parametrize("N,K", [(64, 64), (64, 128), (128, 64), (192, 320), (256, 1088), (64, 2176)])
def test_accumulators_bit_exact_small_shapes(lib, M, N, K):
    w = o.make_ternary(N, K, 0.45, seed=N + K + M)
    rng = np.random.default_rng(M)
    xq = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    pk = Packed(w)
    assert (accumulate(lib, xq, pk) == o.gemm_i32(xq, w)).all()
    assert lib.ternaspmm_last_status() == 0


@pytest.mark.parametrize("N,K", [(2560, 2560), (2560, 6912), (3840, 2560)])
def test_accumulators_bit_exact_layer_shapes(lib, N, K):
    w = o.make_ternary(N, K, 0.45, seed=5)
    xq = np.random.default_rng(6).integers(-128, 128, size=(16, K), dtype=np.int8)
    assert (accumulate(lib, xq, Packed(w)) == o.gemm_i32(xq, w)).all()


@pytest.mark.parametrize("p_zero", [0.0, 0.9, 1.0])
def test_sparsity_extremes(lib, p_zero):
    check(lib, 8, 128, 640, 1, p_zero=p_zero)
    check(lib, 16, 128, 640, 2, p_zero=p_zero)


@pytest.mark.parametrize("ws_num", [1, 2, 3, 4])
@pytest.mark.parametrize("entry", ["bitlinear_TernaSpMM_decode", "bitlinear_TernaSpMM_prefill"])
def test_scale_segments_both_epilogues(lib, ws_num, entry):
    check(lib, 8, 768, 256, ws_num, entry=entry)
    check(lib, 5, 3840, 128, ws_num, entry=entry)   # the hard-coded 2560/640/640 split


@pytest.mark.parametrize("M", [65, 128, 200])
def test_dispatcher_switches_epilogue_above_64_tokens(lib, M):
    check(lib, M, 256, 512, 2)


def test_saturated_activations_and_extreme_scales(lib):
    N, K, M = 128, 1024, 8
    w = o.make_ternary(N, K, 0.0, seed=1)          # every weight non-zero
    xq = np.full((M, K), -128, np.int8)
    xq[1::2] = 127
    s = o.bf16_round(np.array([1e-5, 1e5, 1.0, 127.0, 3.0e-3, 7.5e2, 0.33, 42.0], np.float32))
    ws = o.bf16_round(np.array([1e-4, 0, 0, 0], np.float32))
    pk = Packed(w)
    for entry, mode in (("bitlinear_TernaSpMM_decode", "decode"), ("bitlinear_TernaSpMM_prefill", "prefill")):
        got = call(lib, entry, xq, pk, o.f32_to_bf16_bits(s), o.f32_to_bf16_bits(ws), 1)
        assert (got == o.ternaspmm(xq, w, s, ws, 1, mode)).all()


def test_prefill_epilogue_zero_scale_gives_zero(lib):
    w, xq, s, ws = inputs(4, 64, 128, 1)
    s = s.copy()
    s[2] = 0.0
    got = call(lib, "bitlinear_TernaSpMM_prefill", xq, Packed(w), o.f32_to_bf16_bits(s.reshape(-1)),
               o.f32_to_bf16_bits(ws), 1)
    assert (o.bf16_bits_to_f32(got[2]) == 0).all()   # +0 or -0, as float(acc) * 0.f gives
    assert (got == o.ternaspmm(xq, w, s, ws, 1, "prefill")).all()


def test_reference_known_answer_all_ones(lib):
    # tests/test_kernel.cu of the reference: x == 1, s == 1, ws == {1,1,1,1}, ws_num = 4
    M, N, K = 8, 2560, 2560
    w = o.make_ternary(N, K, 0.45, seed=45)
    xq = np.ones((M, K), np.int8)
    one = o.f32_to_bf16_bits(np.ones(M, np.float32))
    got = call(lib, "bitlinear_TernaSpMM", xq, Packed(w), one, o.f32_to_bf16_bits(np.ones(4, np.float32)), 4)
    want = o.bf16_round(w.sum(axis=1, dtype=np.int32).astype(np.float32))
    assert np.abs(o.bf16_bits_to_f32(got) - want[None, :]).sum() == 0.0


@pytest.mark.parametrize("name", ["t128x192_p45", "t256x320_p45", "t64x256_p90", "t192x64_p00", "t64x128_p100"])
def test_reference_packed_golden_weights_after_transcoding(lib, name):
    """Weights packed by the reference's own packer (committed fixtures), converted
    by the C transcoder, must multiply like the dense matrix they came from."""
    w = GOLD[name + "/w"]
    N, K = w.shape
    ref = [np.ascontiguousarray(GOLD[name + "/" + k]) for k in ("compressed_val", "tile_offsets", "median_offsets", "bitmap")]
    obm, otm, ocv = np.zeros_like(ref[3]), np.zeros_like(ref[2]), np.zeros(ref[0].size + 4, np.uint32)
    assert lib.ternaspmm_transcode_reference_layout(ref[3].ctypes.data, ref[1].ctypes.data, ref[0].ctypes.data, N, K,
                                                    obm.ctypes.data, otm.ctypes.data, ocv.ctypes.data) == 0
    pk = Packed(w, [ocv, ref[1], otm, obm])
    xq, s = o.make_activations(8, K, seed=9)
    ws = o.make_ws(1)
    got = call(lib, "bitlinear_TernaSpMM", xq, pk, o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws), 1)
    assert (got == o.ternaspmm(xq, w, s, ws, 1)).all()


def test_c_packer_through_the_abi(lib):
    """convert_reorderd / reorder_WT_h as tests/test_kernel.cu of the reference uses them."""
    import ctypes
    N, K = 128, 192
    w = o.make_ternary(N, K, 0.45, seed=77)
    wb = o.f32_to_bf16_bits(w.astype(np.float32))
    wr = np.zeros_like(wb)
    lib.reorder_WT_h(wb.ctypes.data, wr.ctypes.data, N, K)
    bm, tg, tm, cv = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
    mx = ctypes.c_int(0)
    tiles = lib.convert_reorderd(wr.ctypes.data, N, K, 64, 16, 8, 64, 64, 8, ctypes.byref(bm), ctypes.byref(tg),
                                 ctypes.byref(tm), ctypes.byref(cv), ctypes.byref(mx))
    assert tiles == N * K // 4096
    ocv, otg, otm, obm = o.compress_weight_b200(w)
    a_tg = np.ctypeslib.as_array(ctypes.cast(tg, ctypes.POINTER(ctypes.c_int32)), (tiles + 1,))
    a_tm = np.ctypeslib.as_array(ctypes.cast(tm, ctypes.POINTER(ctypes.c_uint16)), (3 * tiles,))
    a_bm = np.ctypeslib.as_array(ctypes.cast(bm, ctypes.POINTER(ctypes.c_uint64)), (N * K // 64,))
    a_cv = np.ctypeslib.as_array(ctypes.cast(cv, ctypes.POINTER(ctypes.c_uint32)), (ocv.size,))
    assert (a_tg == otg).all() and (a_tm == otm).all() and (a_bm == obm).all() and (a_cv == ocv).all()
    assert mx.value == int(np.diff(otg).max())


def test_bad_arguments_are_reported_not_run(lib):
    w, xq, s, ws = inputs(8, 64, 128, 1)
    pk = Packed(w)
    x_d = dev(xq)
    out = torch.zeros(8 * 64, dtype=torch.int16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    sb, wb = dev(o.f32_to_bf16_bits(s.reshape(-1))), dev(o.f32_to_bf16_bits(ws))
    lib.bitlinear_TernaSpMM(x_d.data_ptr(), pk.bm.data_ptr(), pk.tg.data_ptr(), pk.tm.data_ptr(), pk.cv.data_ptr(),
                            out.data_ptr(), sb.data_ptr(), wb.data_ptr(), 1, 8, 64, 100, 7, 0, st)
    assert lib.ternaspmm_last_status() == 1
    lib.bitlinear_TernaSpMM(x_d.data_ptr() + 1, pk.bm.data_ptr(), pk.tg.data_ptr(), pk.tm.data_ptr(),
                            pk.cv.data_ptr(), out.data_ptr(), sb.data_ptr(), wb.data_ptr(), 1, 8, 64, 128, 7, 0, st)
    assert lib.ternaspmm_last_status() == 2
    torch.cuda.synchronize()
    assert (out == 0).all()


def test_deterministic_across_runs_and_streams(lib):
    w, xq, s, ws = inputs(16, 2560, 2560, 1, seed=3)
    pk = Packed(w)
    sb, wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
    a = call(lib, "bitlinear_TernaSpMM", xq, pk, sb, wb, 1)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        b = call(lib, "bitlinear_TernaSpMM", xq, pk, sb, wb, 1, stream=side.cuda_stream)
    assert (a == b).all()


def test_capture_in_cuda_graph_and_replay(lib):
    """generate.py of the reference captures the whole forward into a CUDA graph
    (:132-144, :204-216); the entry point must be capture-safe."""
    w, xq, s, ws = inputs(8, 3840, 2560, 3, seed=8)
    pk = Packed(w)
    x_d, s_d = dev(xq), dev(o.f32_to_bf16_bits(s.reshape(-1)))
    ws_d = dev(o.f32_to_bf16_bits(ws))
    out = torch.zeros(8 * 3840, dtype=torch.int16, device="cuda")

    def run():
        lib.bitlinear_TernaSpMM(x_d.data_ptr(), pk.bm.data_ptr(), pk.tg.data_ptr(), pk.tm.data_ptr(),
                                pk.cv.data_ptr(), out.data_ptr(), s_d.data_ptr(), ws_d.data_ptr(), 3, 8, 3840, 2560,
                                7, 0, torch.cuda.current_stream().cuda_stream)

    run()  # first call outside capture (one-time set-up)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    want = o.ternaspmm(xq, w, s, ws, 3)
    for _ in range(20):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert (out.cpu().numpy().view(np.uint16).reshape(8, 3840) == want).all()


def test_python_call_site_matches_oracle(lib):
    """SpBitLinear / TernaInfer_linear (the model.py call site) end to end,
    including the activation quantiser."""
    from ternainfer_b200.linear import SpBitLinear
    from ternainfer_b200.convert import compress_weight
    N, K = 3840, 2560
    w = o.make_ternary(N, K, 0.45, seed=31)
    cv, tg, tm, bm = compress_weight(torch.from_numpy(w))
    ws = o.make_ws(3, seed=32)
    dic = {"l.weight_compressed_val": cv, "l.weight_TileOffsets_global": tg, "l.weight_TileOffsets_median": tm,
           "l.weight_bitmap": bm, "l.weight_scale": torch.from_numpy(ws).to(torch.bfloat16)}
    layer = SpBitLinear(K, N, dic, "l")
    assert layer.ws_num == 3
    x = torch.randn(2, 5, K, generator=torch.Generator().manual_seed(33)).to(torch.bfloat16)
    y = layer(x.cuda())
    assert y.shape == (2, 5, N) and y.dtype == torch.bfloat16
    xq, s = o.quant_input(x.float().numpy().reshape(10, K))
    want = o.ternaspmm(xq, w, s, ws, 3)
    got = y.reshape(10, N).view(torch.int16).cpu().numpy().view(np.uint16)
    assert (got == want).all()


def test_full_size_linearity_property(lib):
    """At the largest BitNet-2B shape: accumulators are linear in the activations
    (acc(x1 + x2) == acc(x1) + acc(x2)) and match the C oracle."""
    N, K, M = 13824, 2560, 16
    w = o.make_ternary(N, K, 0.45, seed=51)
    rng = np.random.default_rng(52)
    x1 = rng.integers(-60, 60, size=(M, K), dtype=np.int8)
    x2 = rng.integers(-60, 60, size=(M, K), dtype=np.int8)
    pk = Packed(w)
    a1, a2, a12 = accumulate(lib, x1, pk), accumulate(lib, x2, pk), accumulate(lib, (x1 + x2).astype(np.int8), pk)
    assert (a1 + a2 == a12).all()
    acc, _ = c_oracle.ternaspmm(x1, w, np.full(M, 0x3F80, np.uint16), np.full(4, 0x3F80, np.uint16), 1)
    assert (a1 == acc).all()


# ---- large token counts: the tcgen05 (tensor memory) kernel ------------------

@pytest.mark.parametrize("M", [33, 64, 100, 128, 129, 256, 257, 512])
@pytest.mark.parametrize("N,K", [(64, 64), (128, 128), (192, 320), (256, 1088)])
def test_large_batch_accumulators_bit_exact(lib, M, N, K):
    w = o.make_ternary(N, K, 0.45, seed=N + K + M)
    xq = np.random.default_rng(M).integers(-128, 128, size=(M, K), dtype=np.int8)
    assert (accumulate(lib, xq, Packed(w)) == o.gemm_i32(xq, w)).all()
    assert lib.ternaspmm_last_status() == 0


@pytest.mark.parametrize("M,N,K,ws_num", [(256, 3840, 2560, 3), (300, 2560, 6912, 1), (64, 2560, 2560, 1),
                                          (2048, 2560, 2560, 1), (130, 13824, 2560, 2)])
def test_large_batch_layer_shapes_outputs(lib, M, N, K, ws_num):
    check(lib, M, N, K, ws_num)


@pytest.mark.parametrize("entry", ["bitlinear_TernaSpMM_decode", "bitlinear_TernaSpMM_prefill"])
def test_large_batch_both_epilogues_and_segments(lib, entry):
    check(lib, 96, 768, 256, 3, entry=entry)
    check(lib, 160, 3840, 128, 3, entry=entry)
    check(lib, 140, 192, 192, 2, entry=entry, p_zero=0.0)
    check(lib, 140, 192, 192, 2, entry=entry, p_zero=1.0)


def test_full_size_prefill_against_c_oracle(lib):
    """The largest case of the layer sweep: gate-up 2560 -> 13824 at 2048 tokens."""
    N, K, M = 13824, 2560, 2048
    w = o.make_ternary(N, K, 0.45, seed=61)
    xq, s = o.make_activations(M, K, seed=62)
    ws = o.make_ws(2, seed=63)
    sb, wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
    pk = Packed(w)
    acc, want = c_oracle.ternaspmm(xq, w, sb, wb, 2)
    assert (accumulate(lib, xq, pk) == acc).all()
    got = call(lib, "bitlinear_TernaSpMM", xq, pk, sb, wb, 2)
    assert (got == want).all()




@pytest.mark.parametrize("M,N,K", [(600, 13888, 320), (1030, 9536, 192), (100, 38464, 128), (40, 38464, 192)])
def test_persistent_ctas_with_several_tiles_each(lib, M, N, K):
    """More output tiles than SMs, so every CTA of the tensor-core kernel walks through several
    tiles and both accumulator buffers of tensor memory are reused; ragged last token tile and a
    last row block of 64 rows.  Accumulators bit-exact against the C oracle, bf16 identical."""
    w = o.make_ternary(N, K, 0.45, seed=M)
    xq, s = o.make_activations(M, K, seed=M + 1)
    ws = o.make_ws(2, seed=M + 2)
    sb, wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
    pk = Packed(w)
    acc, want = c_oracle.ternaspmm(xq, w, sb, wb, 2)
    assert (accumulate(lib, xq, pk) == acc).all()
    got = call(lib, "bitlinear_TernaSpMM", xq, pk, sb, wb, 2)
    assert lib.ternaspmm_last_status() == 0
    assert (got == want).all()


@pytest.mark.parametrize("M,N,K,ws_num", [(256, 1024, 2560, 1), (200, 2560, 2560, 1), (300, 2560, 6912, 1),
                                          (130, 512, 4096, 2), (1000, 1152, 1024, 3), (512, 3840, 2560, 3)])
def test_cluster_k_split_of_the_tensor_core_kernel(lib, M, N, K, ws_num):
    """Few output tiles: the tcgen05 kernel runs as clusters of 8 / 4 / 2 CTAs per tile, each with a
    slice of K, partial accumulators reduce-scattered through distributed shared memory.  Integer
    addition is exact, so accumulators and bf16 outputs must not change by a bit."""
    check(lib, M, N, K, ws_num)
    w = o.make_ternary(N, K, 0.45, seed=M + N)
    xq = np.random.default_rng(K).integers(-128, 128, size=(M, K), dtype=np.int8)
    assert (accumulate(lib, xq, Packed(w)) == c_oracle.ternaspmm(xq, w, np.full(M, 0x3F80, np.uint16),
                                                               np.full(4, 0x3F80, np.uint16), 1)[0]).all()
    assert lib.ternaspmm_last_status() == 0


@pytest.mark.parametrize("M", [1, 8, 16, 32])
@pytest.mark.parametrize("N,K", [(150 * 64, 64), (150 * 64, 320), (296 * 64, 192), (216 * 64, 1088)])
def test_two_row_tiles_per_cta_shapes(lib, M, N, K):
    """Between one and two row tiles per SM (an even count): the small-batch kernel puts two row tiles
    into one fat CTA, half of the warps on each - also when a row tile has fewer k-tiles than warps."""
    w = o.make_ternary(N, K, 0.45, seed=N + K + M)
    xq = np.random.default_rng(M + K).integers(-128, 128, size=(M, K), dtype=np.int8)
    assert (accumulate(lib, xq, Packed(w)) == o.gemm_i32(xq, w)).all()
    assert lib.ternaspmm_last_status() == 0
    check(lib, M, N, K, 2)
