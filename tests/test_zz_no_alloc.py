"""GPU: the output-head entry point that needs no scratch memory from its caller.

Some users of the library may not allocate device memory where they call it (operators inside a
runtime that owns the GPU's memory, latency-critical loops, code under stream capture), so
``ternaspmm_lm_head_argmax_noalloc`` keeps its arg-max candidates in an array inside the library
itself.  It launches the same kernel as ``ternaspmm_lm_head_argmax``; the two must return the same
logits and greedy tokens (the floating-point tolerance of the head tests, and in fact identical
bits), also on the second of two calls in a row, when the built-in area still holds the first
call's leftovers.  This file sorts last on purpose: a run that stops at the first failure has then
already been through every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def both(lib, h, emb, round_bf16=1):
    M, K = h.shape
    V = emb.shape[0]
    st = torch.cuda.current_stream().cuda_stream
    scratch = torch.zeros(int(lib.ternaspmm_lm_head_scratch_bytes()), dtype=torch.uint8, device="cuda")
    want_l = torch.full((M, V), float("nan"), dtype=torch.float32, device="cuda")
    want_t = torch.full((M,), -7, dtype=torch.int64, device="cuda")
    lib.ternaspmm_lm_head_argmax(h.data_ptr(), emb.data_ptr(), M, V, K, want_l.data_ptr(), want_t.data_ptr(), round_bf16,
                                 scratch.data_ptr(), st)
    got_l = torch.full((M, V), float("nan"), dtype=torch.float32, device="cuda")
    got_t = torch.full((M,), -7, dtype=torch.int64, device="cuda")
    lib.ternaspmm_lm_head_argmax_noalloc(h.data_ptr(), emb.data_ptr(), M, V, K, got_l.data_ptr(), got_t.data_ptr(),
                                         round_bf16, st)
    torch.cuda.synchronize()
    assert lib.ternaspmm_last_status() == 0
    return want_l, want_t, got_l, got_t


@pytest.mark.parametrize("M,V,K", [(8, 128256, 2560), (1, 4099, 320), (5, 16, 64)])
def test_no_alloc_head_matches_the_entry_point_with_caller_scratch(lib, M, V, K):
    g = torch.Generator(device="cuda").manual_seed(M * 31 + V + K)
    for call in range(2):             # the second call finds the first one's candidates in the built-in area
        h = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
        emb = (0.02 * torch.randn((V, K), generator=g, device="cuda")).to(torch.bfloat16)
        want_l, want_t, got_l, got_t = both(lib, h, emb)
        tol = want_l.abs() * 2.0 ** -8 + 1e-6     # the tolerance of the head tests; the bits are equal in practice
        assert ((got_l - want_l).abs() <= tol).all()
        assert torch.equal(got_l, want_l)
        assert torch.equal(got_t, want_t)
        assert (got_t.cpu().numpy() == np.argmax(got_l.cpu().numpy(), axis=1)).all()


def test_no_alloc_head_rejects_what_its_built_in_area_cannot_hold(lib):
    h = torch.zeros((9, 64), dtype=torch.bfloat16, device="cuda")
    emb = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    out = torch.full((9,), -7, dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    lib.ternaspmm_lm_head_argmax_noalloc(h.data_ptr(), emb.data_ptr(), 9, 64, 64, None, out.data_ptr(), 1, st)
    assert lib.ternaspmm_last_status() == 1          # more rows than the area has candidate slots for
    lib.ternaspmm_lm_head_argmax_noalloc(h.data_ptr(), emb.data_ptr(), 8, 64, 16384, None, out.data_ptr(), 1, st)
    assert lib.ternaspmm_last_status() == 1
    torch.cuda.synchronize()
    assert (out == -7).all()
