"""GPU: the new library against the reference's OWN CUDA kernels.

oracle/_ref/libternaspmm_ref_decode.so holds the reference's small-batch SpMM
and split-K reduction kernels compiled for sm_100a from the reference checkout
(oracle/Makefile, oracle/ref_decode_wrapper.cu).  Same seeded dense weights,
packed by each side's own packer; same int8 activations and scales.  The bf16
outputs must be bit-identical (the bar is max relative error 2**-7).  The
reference's prefill GEMM needs an un-vendored CUTLASS and cannot be built, so
only its decode path (8, 16, 32, 64 tokens) is compared end to end; of the
prefill path the first stage - the kernel that decompresses the packed weight
into the dense int8 operand - is run and pinned.  The second stage (CUTLASS
int8 GEMM + the scale epilogue visitor, acc * (ws/s)) has NO reference output
here: for it parity is unpinned, the oracle restates
epilogue_visitor_scale_ws.h:135-148,183-210 and an exact integer product.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

import ternaspmm_oracle as o
from gpu_util import Packed, call, dev, max_rel_err

pytestmark = pytest.mark.gpu
REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                      "libternaspmm_ref_decode.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    lib = ctypes.CDLL(REF_SO)
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.ref_bitlinear_TernaSpMM_decode.argtypes = [P] * 8 + [I] * 5 + [P, P]
    lib.ref_bitlinear_TernaSpMM_decode.restype = I
    if hasattr(lib, "ref_decompress_prefill"):
        lib.ref_decompress_prefill.argtypes = [P] * 5 + [I] * 3 + [P]
        lib.ref_decompress_prefill.restype = I
    return lib


def run_reference(ref, w, xq, s_bits, ws_bits, ws_num, split_k):
    M, K = xq.shape
    N = w.shape[0]
    cv, tg, tm, bm = o.compress_weight_ref(w)
    # the reference kernels prefetch a little past the ends of their arrays
    cv = np.concatenate([cv, np.zeros(16, np.uint32)])
    tg = np.concatenate([tg, np.full(8, tg[-1], np.int32)])
    tm = np.concatenate([tm, np.zeros(16, np.uint16)])
    d = [dev(a) for a in (xq, bm, tg, tm, cv)]
    out = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    s_d, ws_d = dev(np.asarray(s_bits, np.uint16)), dev(np.asarray(ws_bits, np.uint16))
    wsp = torch.zeros(split_k * M * N, dtype=torch.int32, device="cuda")
    rc = ref.ref_bitlinear_TernaSpMM_decode(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                                            d[4].data_ptr(), out.data_ptr(), s_d.data_ptr(), ws_d.data_ptr(), ws_num,
                                            M, N, K, split_k, wsp.data_ptr(), 0)
    assert rc == 0
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint16).reshape(M, N)


@pytest.mark.parametrize("M", [8, 16, 32, 64])
@pytest.mark.parametrize("N,K,ws_num,split_k", [(2560, 2560, 1, 7), (3840, 2560, 3, 7), (2560, 6912, 1, 7),
                                                (256, 512, 2, 1)])
def test_outputs_identical_to_reference_kernels(lib, ref, M, N, K, ws_num, split_k):
    w = o.make_ternary(N, K, 0.45, seed=N + M)
    xq, s = o.make_activations(M, K, seed=K + M)
    ws = o.make_ws(ws_num, seed=5)
    sb, wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
    theirs = run_reference(ref, w, xq, sb, wb, ws_num, split_k)
    mine = call(lib, "bitlinear_TernaSpMM_decode", xq, Packed(w), sb, wb, ws_num)
    assert max_rel_err(mine, theirs) <= 2.0 ** -7
    assert (mine == theirs).all()
    # and both equal the CPU oracle
    assert (theirs == o.ternaspmm(xq, w, s, ws, ws_num, "decode")).all()


def test_reference_known_answer_on_reference_kernels(ref):
    """The reference's documented check (tests/test_kernel.cu with 8 2560 2560 45 7):
    all-ones activations, unit scales -> row sums, total error 0."""
    M, N, K = 8, 2560, 2560
    w = o.make_ternary(N, K, 0.45, seed=45)
    one = o.f32_to_bf16_bits(np.ones(M, np.float32))
    got = run_reference(ref, w, np.ones((M, K), np.int8), one, o.f32_to_bf16_bits(np.ones(4, np.float32)), 4, 7)
    want = o.bf16_round(w.sum(axis=1, dtype=np.int32).astype(np.float32))
    assert np.abs(o.bf16_bits_to_f32(got) - want[None, :]).sum() == 0.0


@pytest.mark.parametrize("args", [["8", "2560", "2560", "45", "7"], ["16", "3840", "2560", "45", "7"],
                                  ["64", "2560", "6912", "45", "7"], ["256", "2560", "2560", "45", "7"]])
def test_reference_kernel_test_program_unchanged(args):
    """tests/test_kernel.cu of the reference, compiled unchanged and linked against this
    library (oracle/Makefile): its cuBLAS comparison must report TotalError 0.00."""
    import subprocess
    exe = os.path.join(os.path.dirname(REF_SO), "test_kernel")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/test_kernel not built (needs the reference checkout at build time)")
    r = subprocess.run([exe] + args, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith("TernaSpMM")]
    assert line and "TotalError: 0.00" in line[0], r.stdout


@pytest.mark.parametrize("N,K,p_zero,split", [(2560, 2560, 0.45, 7), (3840, 2560, 0.45, 7), (256, 6912, 0.45, 7),
                                              (128, 640, 0.0, 5), (128, 640, 0.9, 5), (64, 448, 1.0, 7)])
def test_reference_decompress_kernel_restores_the_dense_weight(lib, ref, N, K, p_zero, split):
    """Stage 1 of the reference's prefill path (mySpMM_Kernel_bitmap_prefill; split 7 as model.py
    passes it where the kernel's own split arithmetic allows it: with K/64 k-blocks the last split
    gets ceil - padding blocks, which must not be negative, so the 10-block case uses 5)
    on weights packed in the reference layout writes exactly the dense ternary matrix -
    the operand its int8 GEMM multiplies.  The same dense matrix, packed in the B200 order, gives
    bit-exact int32 accumulators in the tcgen05 kernel, so both prefill paths contract identical
    operands.  (The reference's GEMM + epilogue stage cannot be built: unpinned.)"""
    if not hasattr(ref, "ref_decompress_prefill"):
        pytest.skip("oracle/_ref was built without the decompress wrapper")
    from gpu_util import accumulate
    w = o.make_ternary(N, K, p_zero, seed=N + K)
    cv, tg, tm, bm = o.compress_weight_ref(w)
    cv = np.concatenate([cv, np.zeros(16, np.uint32)])
    tg = np.concatenate([tg, np.full(8, tg[-1], np.int32)])
    tm = np.concatenate([tm, np.zeros(16, np.uint16)])
    d = [dev(a) for a in (bm, tg, tm, cv)]
    dense = torch.full((N * K,), 0x55, dtype=torch.int8, device="cuda")
    rc = ref.ref_decompress_prefill(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                                    dense.data_ptr(), N, K, split, 0)
    assert rc == 0
    torch.cuda.synchronize()
    assert (dense.cpu().numpy().reshape(N, K) == w).all()
    M = 130
    xq = np.random.default_rng(N).integers(-128, 128, size=(M, K), dtype=np.int8)
    assert (accumulate(lib, xq, Packed(w)) == o.gemm_i32(xq, w)).all()
