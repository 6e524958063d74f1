"""GPU: every launch variant the dispatcher can pick, and the full shape grids.

Each case goes through the C ABI, is compared with the CPU oracle (int32
accumulators bit-exact, bf16 outputs identical) and asserts - through the
test hook ``ternaspmm_last_launch_shape`` - that the intended kernel variant
really ran:
  kind 1  small-batch kernel, one fat CTA per SM (<1,28,1> <2,20,1> <4,16,1>)
  kind 2  small-batch kernel, thin CTAs, two per SM (<1,14,2> <2,10,2> <4,8,2>),
          with or without a cluster K split
  kind 3  tcgen05 kernel (NT = 64 / 128 / 256 tokens per tile), with or without
          its cluster K split
"""
import ctypes

import numpy as np
import pytest
import torch

import ternaspmm_oracle as o
import c_oracle
from gpu_util import Packed, call, accumulate, dev
from ternainfer_b200.convert import compress_weight

pytestmark = pytest.mark.gpu

ONE = 0x3F80   # bf16 1.0


def launch_shape(lib):
    a = (ctypes.c_int * 6)()
    lib.ternaspmm_last_launch_shape(a)
    return dict(zip(("kind", "tokens_per_pass", "splits", "warps", "row_tiles_per_cta", "ctas"), list(a)))


def gpu_packed(w: np.ndarray) -> Packed:
    """Pack on the GPU (large weights); same arrays as the CPU packer."""
    arrays = [t.cpu().numpy() for t in compress_weight(torch.from_numpy(w).cuda())]
    return Packed(w, arrays)


_WEIGHTS = {}   # (N, K) -> (dense, packed); the last few only, the largest weight is 470 MB dense


def weight(N, K):
    if (N, K) not in _WEIGHTS:
        while len(_WEIGHTS) >= 3:
            _WEIGHTS.pop(next(iter(_WEIGHTS)))
        w = o.make_ternary(N, K, 0.45, seed=N * 7 + K)
        _WEIGHTS[(N, K)] = (w, gpu_packed(w) if N * K > (1 << 24) else Packed(w))
    return _WEIGHTS[(N, K)]


def check_against_c_oracle(lib, M, N, K, ws_num, seed, entry="bitlinear_TernaSpMM", mode=-1):
    w, pk = weight(N, K)
    xq, s = o.make_activations(M, K, seed + 1)
    ws = o.make_ws(ws_num, seed + 2)
    sb, wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
    acc, want = c_oracle.ternaspmm(xq, w, sb, wb, ws_num, mode)
    assert (accumulate(lib, xq, pk) == acc).all(), "int32 accumulators differ from the oracle"
    got = call(lib, entry, xq, pk, sb, wb, ws_num, pad=64)
    assert lib.ternaspmm_last_status() == 0
    assert (got == want).all(), "bf16 outputs differ from the oracle"
    return launch_shape(lib), pk, w


# ---- thin small-batch variants ------------------------------------------------

@pytest.mark.parametrize("N,K", [(149 * 64, 64), (149 * 64, 320), (149 * 64, 4096), (300 * 64, 192), (300 * 64, 1088)])
@pytest.mark.parametrize("M", [1, 8, 16, 32])
def test_thin_variants_odd_and_many_row_tiles(lib, M, N, K):
    """An odd number of row tiles above the SM count, and more than two row tiles per SM: neither
    the one-CTA-per-SM shape nor its two-row-tiles form applies, so the thin variants run."""
    shape, _, _ = check_against_c_oracle(lib, M, N, K, 2, seed=N + K + M)
    assert shape["kind"] == 2, shape
    assert shape["tokens_per_pass"] == (8 if M <= 8 else 16 if M <= 16 else 32), shape
    assert shape["row_tiles_per_cta"] == 1


@pytest.mark.parametrize("M", [40, 64])
def test_thin_variant_with_two_token_blocks(lib, M):
    """33-64 tokens on a small narrow weight stay on the small-batch kernel as two blocks of 32
    tokens; with more (row tile, token block) pairs than SMs the thin <4,8,2> variant runs."""
    shape, _, _ = check_against_c_oracle(lib, M, 100 * 64, 320, 1, seed=M)
    assert shape["kind"] == 2 and shape["tokens_per_pass"] == 32, shape


def test_thin_variant_uses_a_cluster_split_when_it_fits(lib):
    """149 row tiles of 64 k-tiles each: two thin CTAs per SM leave room for a K split."""
    shape, _, _ = check_against_c_oracle(lib, 8, 149 * 64, 4096, 1, seed=5)
    assert shape["kind"] == 2
    # (recorded, not required: the cost model may prefer more warps over a split)
    assert shape["splits"] >= 1 and shape["ctas"] == 149 * shape["splits"]


@pytest.mark.parametrize("M", [1, 8, 16])
def test_gate_up_of_the_8192_wide_model_at_small_batch(lib, M):
    """57344 x 8192 (896 row tiles): the largest weight of the 8192-wide model at decode batch sizes."""
    shape, _, _ = check_against_c_oracle(lib, M, 57344, 8192, 2, seed=900 + M)
    assert shape["kind"] == 2, shape


# ---- fat variants, recorded ----------------------------------------------------

@pytest.mark.parametrize("N,K,ws_num", [(3840, 2560, 3), (2560, 2560, 1), (13824, 2560, 2), (2560, 6912, 1)])
@pytest.mark.parametrize("M,mt", [(8, 8), (16, 16), (32, 32)])
def test_fat_variants_on_the_bitnet2b_layers(lib, M, mt, N, K, ws_num):
    shape, _, _ = check_against_c_oracle(lib, M, N, K, ws_num, seed=N + M)
    assert shape["kind"] == 1 and shape["tokens_per_pass"] == mt, shape
    if N == 13824:
        assert shape["row_tiles_per_cta"] == 2
    if K == 6912 and M <= 16:
        assert shape["splits"] > 1     # the down projection is the one BitNet-2B layer with a cluster K split


# ---- the full layer sweep: 4 shapes x 6 token counts --------------------------------

SWEEP_SHAPES = [(3840, 2560, 3), (2560, 2560, 1), (13824, 2560, 2), (2560, 6912, 1)]


@pytest.mark.parametrize("N,K,ws_num", SWEEP_SHAPES)
@pytest.mark.parametrize("M", [1, 8, 16, 64, 256, 2048])
def test_layer_sweep_grid(lib, M, N, K, ws_num):
    """QKV / O / gate-up / down of BitNet-b1.58-2B at 1, 8, 16, 64, 256 and 2048 tokens: all 24 cells."""
    shape, _, _ = check_against_c_oracle(lib, M, N, K, ws_num, seed=M)
    if M <= 32:
        assert shape["kind"] in (1, 2)
    elif M >= 256:
        assert shape["kind"] == 3 and shape["tokens_per_pass"] == 256


# ---- the 8192-wide model's linears and their tensor-parallel shards -----------------

def _big_shapes():
    dim, H, Hkv, D, ffn = 8192, 64, 8, 128, 28672
    cases = []
    for tp in (1, 2, 4, 8):
        cases += [("wqkv", (H + 2 * Hkv) * D // tp, dim, 3, tp), ("wo", dim, dim // tp, 1, tp),
                  ("w13", 2 * ffn // tp, dim, 2, tp), ("w2", dim, ffn // tp, 1, tp)]
    return cases


@pytest.mark.parametrize("name,N,K,ws_num,tp", _big_shapes())
@pytest.mark.parametrize("M", [8, 64])
def test_8192_wide_model_linears_and_shards(lib, name, N, K, ws_num, tp, M):
    """hidden 8192, 64/8 heads, ffn 28672: QKV 10240x8192, O 8192x8192, gate-up 57344x8192, down
    8192x28672, and the per-rank shapes at tensor-parallel sizes 2, 4 and 8 (N/T for the
    column-parallel pair, K/T for the row-parallel pair)."""
    if name == "w13" and tp == 1 and M == 8:
        pytest.skip("covered by test_gate_up_of_the_8192_wide_model_at_small_batch")
    shape, pk, w = check_against_c_oracle(lib, M, N, K, ws_num, seed=tp * 100 + M + len(name))
    if M == 8:
        assert shape["kind"] in (1, 2), shape
    elif N * K > (32 << 20):
        assert shape["kind"] == 3 and shape["tokens_per_pass"] == 64, shape   # small narrow shards stay on the small-batch kernel
    if name == "wqkv":
        # explicit segment boundaries, as the sharded layers pass them
        H, Hkv, D = 64 // tp, 8 // tp, 128
        b = [H * D, (H + Hkv) * D]
        xq, s = o.make_activations(M, K, 77)
        ws = o.make_ws(3, 78)
        sb, wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
        acc = accumulate(lib, xq, pk)
        col = np.arange(N)
        g = (col >= b[0]).astype(np.int64) + (col >= b[1])
        v = (acc.astype(np.float32) / o.bf16_bits_to_f32(sb).reshape(-1, 1)).astype(np.float32) * \
            o.bf16_bits_to_f32(wb)[g][None, :]
        want = o.f32_to_bf16_bits(v)
        x_d, s_d, ws_d = dev(xq), dev(sb), dev(wb)
        out = torch.zeros(M * N, dtype=torch.int16, device="cuda")
        lib.ternaspmm_linear_segments(x_d.data_ptr(), pk.bm.data_ptr(), pk.tg.data_ptr(), pk.tm.data_ptr(),
                                      pk.cv.data_ptr(), out.data_ptr(), s_d.data_ptr(), ws_d.data_ptr(), 3, M, N, K,
                                      b[0], b[1], 2 ** 31 - 1, 0, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert lib.ternaspmm_last_status() == 0
        assert (out.cpu().numpy().view(np.uint16).reshape(M, N) == want).all()
