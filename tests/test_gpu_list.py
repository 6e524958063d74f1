"""GPU: the work-list entry points (many independent small-batch linears in one persistent launch)
through the C ABI, every item against the CPU oracle: bf16 outputs identical to the reference
formula, hence to the per-call entry points."""
import ctypes

import numpy as np
import pytest
import torch

import ternaspmm_oracle as o
import c_oracle
from gpu_util import Packed, dev
from ternainfer_b200.lib import ListItem

pytestmark = pytest.mark.gpu


class Case:
    def __init__(self, M, N, K, ws_num, seed, residual=False, segs=None, form=-1):
        self.M, self.N, self.K, self.ws_num, self.form = M, N, K, ws_num, form
        self.w = o.make_ternary(N, K, 0.45, seed)
        self.xq, s = o.make_activations(M, K, seed + 1)
        ws = o.make_ws(ws_num, seed + 2)
        self.sb, self.wb = o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws)
        self.pk = Packed(self.w)
        self.x_d, self.s_d, self.ws_d = dev(self.xq), dev(self.sb), dev(self.wb)
        self.out = torch.full((M * N,), 0x7B7B, dtype=torch.int16, device="cuda")
        self.segs = segs
        acc = o.gemm_i32(self.xq, self.w)
        sf, wf = o.bf16_bits_to_f32(self.sb).reshape(-1, 1), o.bf16_bits_to_f32(self.wb)
        if segs:        # explicit boundaries: column n uses ws[(n >= b1) + (n >= b2) + ...], decode form
            b = [sum(segs[:i + 1]) for i in range(len(segs) - 1)]
            g = sum((np.arange(N) >= v).astype(np.int64) for v in b)
            self.want = o.f32_to_bf16_bits((acc.astype(np.float32) / sf).astype(np.float32) * wf[g][None, :])
            self.bounds = b + [0] * (3 - len(b))
        else:
            self.want = o.ternaspmm(self.xq, self.w, s, ws, ws_num, {-1: "auto", 0: "decode", 1: "prefill"}[form])
            self.bounds = [0, 0, 0]
        self.res_d = None
        if residual:
            res = o.bf16_round(np.random.default_rng(seed + 3).standard_normal((M, N)).astype(np.float32))
            self.res_d = dev(o.f32_to_bf16_bits(res))
            self.want = o.f32_to_bf16_bits(res + o.bf16_bits_to_f32(self.want))

    def item(self):
        it = ListItem()
        it.x, it.bitmap, it.tile_offsets = self.x_d.data_ptr(), self.pk.bm.data_ptr(), self.pk.tg.data_ptr()
        it.quarter_offsets, it.sign_words, it.out = self.pk.tm.data_ptr(), self.pk.cv.data_ptr(), self.out.data_ptr()
        it.s, it.ws = self.s_d.data_ptr(), self.ws_d.data_ptr()
        it.residual = self.res_d.data_ptr() if self.res_d is not None else None
        it.ws_num, it.M, it.N, it.K = self.ws_num, self.M, self.N, self.K
        it.seg1, it.seg2, it.seg3 = self.bounds
        it.prefill_form = 0 if self.segs else self.form
        return it

    def check(self):
        got = self.out.cpu().numpy().view(np.uint16).reshape(self.M, self.N)
        assert (got == self.want).all(), (self.M, self.N, self.K)


class List:
    def __init__(self, lib, cases):
        self.lib, self.cases = lib, cases
        self.arr = (ListItem * len(cases))(*[c.item() for c in cases])
        tb, sb = ctypes.c_longlong(), ctypes.c_longlong()
        self.entries = lib.ternaspmm_list_plan(self.arr, len(cases), ctypes.byref(tb), ctypes.byref(sb))
        assert self.entries >= len(cases)
        self.table = torch.empty(tb.value, dtype=torch.uint8, device="cuda")
        self.scratch = torch.empty(sb.value, dtype=torch.uint8, device="cuda")
        self.handle = lib.ternaspmm_list_create(self.arr, len(cases), self.table.data_ptr(), self.scratch.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream)
        assert self.handle

    def run(self):
        self.lib.ternaspmm_list_run(self.handle, torch.cuda.current_stream().cuda_stream)

    def close(self):
        self.lib.ternaspmm_list_destroy(self.handle)


def run_and_check(lib, cases, runs=2):
    lst = List(lib, cases)
    for _ in range(runs):            # the second run finds the scratch area re-armed by the first
        for c in cases:
            c.out.fill_(0x7B7B)
        lst.run()
        torch.cuda.synchronize()
        assert lib.ternaspmm_last_status() == 0
        for c in cases:
            c.check()
    # the whole scratch area (abort flag, arrival counters, boundary areas) is back at zero
    assert (lst.scratch == 0).all()
    return lst


def test_one_layer_of_four_linears(lib):
    cases = [Case(8, 3840, 2560, 3, 1), Case(8, 2560, 2560, 1, 2), Case(8, 13824, 2560, 2, 3), Case(8, 2560, 6912, 1, 4)]
    run_and_check(lib, cases).close()


def test_mixed_items_token_counts_residual_segments_and_tiny_shapes(lib):
    cases = [Case(1, 64, 64, 1, 10), Case(3, 192, 320, 2, 11), Case(8, 2560, 2560, 1, 12, residual=True),
             Case(5, 3840, 128, 3, 13), Case(7, 1280, 1088, 3, 14, segs=[1024, 128, 128]), Case(8, 64, 2176, 1, 15),
             Case(2, 128, 64, 4, 16), Case(8, 768, 256, 2, 17, form=1), Case(8, 9536, 192, 2, 18),
             Case(4, 256, 1088, 1, 19, residual=True), Case(8, 64, 64, 1, 20), Case(6, 3840, 2560, 3, 21)]
    run_and_check(lib, cases).close()


def test_very_wide_and_very_short_layers(lib):
    """Hundreds of row tiles with one or two k-tiles each (every CTA's share holds many whole row
    tiles), next to a deep narrow layer (one row tile spread over many CTAs)."""
    cases = [Case(8, 400 * 64, 128, 2, 30), Case(8, 2560, 2560, 1, 31), Case(3, 640 * 64, 64, 3, 32, residual=True),
             Case(8, 64, 28672, 1, 33), Case(5, 128, 8192, 2, 34)]
    lst = run_and_check(lib, cases)
    assert lst.entries == 5
    lst.close()


def test_tiny_lists(lib):
    """Fewer tiles than SMs: only some CTAs get a share."""
    run_and_check(lib, [Case(8, 64, 64, 1, 70)]).close()
    run_and_check(lib, [Case(2, 128, 192, 2, 71), Case(8, 64, 128, 1, 72)]).close()
    run_and_check(lib, [Case(8, 64, 64 * 200, 1, 73)]).close()


def test_sixteen_tokens(lib):
    cases = [Case(16, 3840, 2560, 3, 40), Case(9, 2560, 2560, 1, 41, residual=True), Case(16, 13824, 2560, 2, 42),
             Case(12, 2560, 6912, 1, 43), Case(1, 192, 320, 2, 44), Case(16, 64, 64, 1, 45)]
    run_and_check(lib, cases).close()


def test_long_list_in_a_cuda_graph(lib):
    """Forty items (ten layers), captured once and replayed: every replay bit-identical to the oracle."""
    shapes = [(3840, 2560, 3), (2560, 2560, 1), (13824, 2560, 2), (2560, 6912, 1)]
    base = [Case(8, n, k, w, 50 + i) for i, (n, k, w) in enumerate(shapes)]
    cases = []
    for layer in range(10):
        for b in base:
            c = Case.__new__(Case)
            c.__dict__.update(b.__dict__)
            c.out = torch.full((c.M * c.N,), 0x7B7B, dtype=torch.int16, device="cuda")
            cases.append(c)
    lst = List(lib, cases)
    lst.run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        lst.run()
    for _ in range(5):
        for c in cases:
            c.out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert lib.ternaspmm_last_status() == 0
        for c in cases:
            c.check()
    lst.close()


def test_bad_items_are_rejected(lib):
    c = Case(8, 64, 64, 1, 60)
    it = c.item()
    it.M = 17
    arr = (ListItem * 1)(it)
    assert lib.ternaspmm_list_plan(arr, 1, None, None) == -1
    assert lib.ternaspmm_last_status() == 1
    it = c.item()
    it.x = it.x + 1
    arr = (ListItem * 1)(it)
    assert lib.ternaspmm_list_plan(arr, 1, None, None) == -1
    assert lib.ternaspmm_last_status() == 2
