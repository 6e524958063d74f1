"""GPU: the large-batch path through a dense workspace (bitlinear_TernaSpMM_ws): the weight is decoded
once per call into a caller-provided N*K-byte workspace and a tcgen05 kernel takes both operands by
TMA - on CTA pairs (256 x 256 tiles, launch kind 7) above 128 tokens, on single CTAs (kind 6) up to 128.  Integer contraction and the same epilogue code as the on-chip path: outputs must equal the CPU
oracle bit for bit, and the workspace must hold exactly the dense ternary matrix afterwards."""
import ctypes

import numpy as np
import pytest
import torch

import ternaspmm_oracle as o
import c_oracle
from gpu_util import Packed, dev

pytestmark = pytest.mark.gpu


def run_ws(lib, M, N, K, ws_num, path, seed, residual=False, slack=0, skew=0):
    w = o.make_ternary(N, K, 0.45, seed)
    xq, s = o.make_activations(M, K, seed + 1)
    ws = o.make_ws(ws_num, seed + 2)
    sb, wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
    pk = Packed(w)
    _, want = c_oracle.ternaspmm(xq, w, sb, wb, ws_num, -1)
    res_d = None
    if residual:
        res = o.bf16_round(np.random.default_rng(seed + 3).standard_normal((M, N)).astype(np.float32))
        res_d = dev(o.f32_to_bf16_bits(res))
        want = o.f32_to_bf16_bits(res + o.bf16_bits_to_f32(want))
    x_d, s_d, ws_d = dev(xq), dev(sb), dev(wb)
    out = torch.full((M * N + 128 + skew,), 0x7B7B, dtype=torch.int16, device="cuda")
    work = torch.full((N * K + slack + 256,), 0x55, dtype=torch.int8, device="cuda")
    lib.bitlinear_TernaSpMM_ws(x_d.data_ptr(), pk.bm.data_ptr(), pk.tg.data_ptr(), pk.tm.data_ptr(), pk.cv.data_ptr(),
                               out.data_ptr() + 2 * skew, s_d.data_ptr(), ws_d.data_ptr(), ws_num, M, N, K,
                               res_d.data_ptr() if res_d is not None else None, work.data_ptr(), N * K + slack, path,
                               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert lib.ternaspmm_last_status() == 0
    got = out.cpu().numpy().view(np.uint16)
    assert (got[:skew] == 0x7B7B).all(), "wrote in front of the output"
    got = got[skew:]
    assert (got[M * N:] == 0x7B7B).all(), "wrote past the output"
    assert (got[:M * N].reshape(M, N) == want).all(), "bf16 outputs differ from the oracle"
    shape = (ctypes.c_int * 6)()
    lib.ternaspmm_last_launch_shape(shape)
    wk = work.cpu().numpy()
    return shape[0], wk, w


@pytest.mark.parametrize("M,N,K,ws_num", [(2048, 13824, 2560, 2), (256, 13824, 2560, 2), (512, 3840, 2560, 3),
                                          (1000, 2560, 6912, 1), (130, 13824, 2560, 2), (300, 9536, 192, 2),
                                          (128, 3840, 2560, 3), (4096, 2560, 2560, 1), (2049, 9472, 320, 2)])
def test_layer_shapes_through_the_workspace(lib, M, N, K, ws_num):
    kind, wk, w = run_ws(lib, M, N, K, ws_num, path=2, seed=M + N)
    assert kind == (7 if M > 128 else 6)
    assert (wk[:N * K].reshape(N, K) == w).all(), "the workspace does not hold the dense weight"
    assert (wk[N * K:] == 0x55).all(), "wrote past N*K bytes of the workspace"


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (129, 192, 320), (257, 64, 2176), (700, 320, 128), (300, 1088, 256)])
def test_small_and_ragged_shapes_forced_through_the_workspace(lib, M, N, K):
    """A last row block of 64 rows, fewer k than one pipeline step, ragged token tiles, residual."""
    kind, wk, w = run_ws(lib, M, N, K, 2, path=2, seed=M + N + K, residual=True)
    assert kind == (7 if M > 128 else 6)
    assert (wk[:N * K].reshape(N, K) == w).all()


@pytest.mark.parametrize("M,path", [(300, 2), (100, 2), (300, 1), (100, 1)])
def test_output_that_is_not_16_byte_aligned(lib, M, path):
    """The bf16 epilogues store 16 bytes per lane when the output (and residual) allow it; an output that
    starts at an odd element takes the two-byte stores instead.  Same bits, nothing written outside."""
    run_ws(lib, M, 320, 256, 2, path=path, seed=M + path, skew=3)
    run_ws(lib, M, 320, 256, 2, path=path, seed=M + path + 1, skew=8, residual=True)


def test_auto_choice_and_fallbacks(lib):
    kind, _, _ = run_ws(lib, 2048, 13824, 2560, 2, path=0, seed=1)           # big: through the workspace
    assert kind == 7
    kind, _, _ = run_ws(lib, 512, 3840, 2560, 3, path=0, seed=5)             # two token tiles already pay
    assert kind == 7
    kind, wk, _ = run_ws(lib, 256, 2560, 2560, 1, path=0, seed=2)            # one token tile: on chip (cluster K split)
    assert kind == 3 and (wk == 0x55).all()
    kind, wk, _ = run_ws(lib, 512, 2560, 6912, 1, path=0, seed=6)            # deep and narrow: on chip up to 1024 tokens
    assert kind == 3 and (wk == 0x55).all()
    kind, wk, _ = run_ws(lib, 64, 13824, 2560, 2, path=0, seed=3)            # decode-sized: never
    assert kind in (1, 2, 3) and (wk == 0x55).all()
    kind, wk, _ = run_ws(lib, 2048, 13824, 2560, 2, path=1, seed=4)          # forced on chip
    assert kind == 3 and (wk == 0x55).all()


def test_workspace_too_small_is_rejected_or_ignored(lib):
    w = o.make_ternary(256, 256, 0.45, 5)
    xq, s = o.make_activations(200, 256, 6)
    pk = Packed(w)
    x_d, s_d = dev(xq), dev(o.f32_to_bf16_bits(s.reshape(-1)))
    ws_d = dev(o.f32_to_bf16_bits(o.make_ws(1)))
    out = torch.zeros(200 * 256, dtype=torch.int16, device="cuda")
    work = torch.full((1024,), 0x55, dtype=torch.int8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    args = (x_d.data_ptr(), pk.bm.data_ptr(), pk.tg.data_ptr(), pk.tm.data_ptr(), pk.cv.data_ptr(), out.data_ptr(),
            s_d.data_ptr(), ws_d.data_ptr(), 1, 200, 256, 256, None, work.data_ptr(), 1024)
    lib.bitlinear_TernaSpMM_ws(*args, 2, st)          # forced, but the workspace is too small: refused
    assert lib.ternaspmm_last_status() == 2
    torch.cuda.synchronize()
    assert (out == 0).all() and (work == 0x55).all()
    lib.bitlinear_TernaSpMM_ws(*args, 0, st)          # free choice: the on-chip path
    torch.cuda.synchronize()
    assert lib.ternaspmm_last_status() == 0 and (work == 0x55).all() and not (out == 0).all()


def test_python_call_site_uses_the_workspace_at_prefill(lib):
    from ternainfer_b200.linear import SpBitLinear, get_global_workspace, quant_input
    from ternainfer_b200.convert import compress_weight
    N, K = 13824, 2560
    w = o.make_ternary(N, K, 0.45, seed=71)
    cv, tg, tm, bm = compress_weight(torch.from_numpy(w))
    wsv = o.make_ws(2, seed=72)
    dic = {"l.weight_compressed_val": cv, "l.weight_TileOffsets_global": tg, "l.weight_TileOffsets_median": tm,
           "l.weight_bitmap": bm, "l.weight_scale": torch.from_numpy(wsv).to(torch.bfloat16)}
    layer = SpBitLinear(K, N, dic, "l")
    x = torch.randn(2048, K, generator=torch.Generator().manual_seed(73)).to(torch.bfloat16).cuda()
    y = layer(x)
    shape = (ctypes.c_int * 6)()
    lib.ternaspmm_last_launch_shape(shape)
    assert shape[0] == 7
    xq, s = o.quant_input(x.float().cpu().numpy())
    _, want = c_oracle.ternaspmm(xq, w, o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(wsv), 2, -1)
    assert (y.view(torch.int16).cpu().numpy().view(np.uint16) == want).all()
    assert get_global_workspace("cuda").numel() >= N * K


def test_int8_mma_issue_rate_hook(lib):
    """The measurement hook that bench.py quotes the tensor-core kernels against: returns a plausible rate
    (the part issues int8 MMAs at about twice its bf16 rate) and leaves the status word clean."""
    rate = lib.ternaspmm_debug_int8_mma_rate(3200, torch.cuda.current_stream().cuda_stream)
    assert lib.ternaspmm_last_status() == 0
    assert 1.0e15 < rate < 8.0e15, rate
