"""GPU: the output-head kernel (logits of up to 8 rows over the vocabulary + greedy token) through
the C ABI, against a float64 product of the same bf16 inputs.

Floating-point kernel: fp32 accumulation in the tensor cores in an order of its own, result rounded
to bf16 like the reference's bf16 linear.  Tolerance per logit: one bf16 rounding step of the exact
value (2**-8 relative) plus the fp32 accumulation error (1e-5 of sum |h||e|).  The arg-max must be
exactly the first index of the maximum of the kernel's own logits, and its exact logit must be
within the same tolerance of the exact maximum.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def run(lib, h, emb, want_logits=True, want_argmax=True, round_bf16=1, scratch=None):
    M, K = h.shape
    V = emb.shape[0]
    if scratch is None:
        scratch = torch.zeros(int(lib.ternaspmm_lm_head_scratch_bytes()), dtype=torch.uint8, device="cuda")
    logits = torch.full((M, V), float("nan"), dtype=torch.float32, device="cuda") if want_logits else None
    toks = torch.full((M,), -7, dtype=torch.int64, device="cuda") if want_argmax else None
    lib.ternaspmm_lm_head_argmax(h.data_ptr(), emb.data_ptr(), M, V, K, logits.data_ptr() if want_logits else None,
                                 toks.data_ptr() if want_argmax else None, round_bf16, scratch.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert lib.ternaspmm_last_status() == 0
    return logits, toks, scratch


def inputs(M, V, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    h = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    emb = (0.02 * torch.randn((V, K), generator=g, device="cuda")).to(torch.bfloat16)
    return h, emb


def exact(h, emb):
    ref = torch.empty((h.shape[0], emb.shape[0]), dtype=torch.float64, device="cuda")
    mag = torch.empty_like(ref)
    for v0 in range(0, emb.shape[0], 16384):        # in slabs: float64 copies of the full embedding are large
        e = emb[v0:v0 + 16384].double()
        ref[:, v0:v0 + 16384] = h.double() @ e.t()
        mag[:, v0:v0 + 16384] = h.double().abs() @ e.abs().t()
    return ref, mag


@pytest.mark.parametrize("M,V,K", [(1, 128256, 2560), (8, 128256, 2560), (3, 1000, 2560), (8, 16, 64), (5, 4099, 8192),
                                   (2, 33, 96), (8, 50000, 320)])
def test_logits_and_greedy_token(lib, M, V, K):
    h, emb = inputs(M, V, K, seed=M + V + K)
    logits, toks, scratch = run(lib, h, emb)
    ref, mag = exact(h, emb)
    tol = ref.abs() * 2.0 ** -8 + mag * 1e-5 + 1e-30
    assert not torch.isnan(logits).any()
    assert ((logits.double() - ref).abs() <= tol).all()
    assert torch.equal(logits, logits.to(torch.bfloat16).float())          # every logit is a bf16 value
    lg = logits.cpu().numpy()
    assert (toks.cpu().numpy() == np.argmax(lg, axis=1)).all()             # first index of the maximum
    picked = ref.gather(1, toks.view(-1, 1)).view(-1)
    best = ref.max(dim=1).values
    assert ((best - picked) <= (best.abs() * 2.0 ** -7 + mag.max(dim=1).values * 2e-5)).all()
    # a second call on the same scratch area (its counter must be back at zero), arg-max only
    _, toks2, _ = run(lib, h, emb, want_logits=False, scratch=scratch)
    assert torch.equal(toks, toks2)
    # and logits only, unrounded fp32
    raw, none, _ = run(lib, h, emb, want_argmax=False, round_bf16=0, scratch=scratch)
    assert none is None and ((raw.double() - ref).abs() <= mag * 1e-5 + 1e-30).all()
    assert torch.equal(raw.to(torch.bfloat16).float(), logits)


def test_ties_resolve_to_the_smallest_index(lib):
    M, V, K = 4, 5000, 256
    h, emb = inputs(M, V, K, seed=5)
    emb[:] = 0
    emb[[17, 18, 900, 4099]] = h[0]        # four identical rows: the same (largest) logit for token 0
    emb[4999] = h[1]
    emb[33] = h[1]
    logits, toks, _ = run(lib, h, emb)
    assert toks[0].item() == 17 and toks[1].item() == 33
    assert (toks.cpu().numpy() == np.argmax(logits.cpu().numpy(), axis=1)).all()


def test_matches_the_dense_bf16_gemm_closely(lib):
    """Against torch's bf16 F.linear (what the reference's head computes): both round the same exact
    value to bf16, so logits agree up to one bf16 step and the greedy tokens' logits are equal-valued."""
    h, emb = inputs(8, 128256, 2560, seed=77)
    logits, toks, _ = run(lib, h, emb)
    dense = torch.nn.functional.linear(h, emb).float()
    assert ((logits - dense).abs() <= dense.abs() * 2.0 ** -7 + 1e-6).all()
    t_dense = dense.argmax(-1)
    same = toks == t_dense
    # where they differ, the two candidates are one bf16 step apart at most
    a, b = logits.gather(1, toks.view(-1, 1)), logits.gather(1, t_dense.view(-1, 1))
    assert (same | ((a - b).abs().view(-1) <= a.abs().view(-1) * 2.0 ** -7)).all()


def test_bad_arguments(lib):
    h, emb = inputs(2, 64, 64, seed=1)
    sc = torch.zeros(int(lib.ternaspmm_lm_head_scratch_bytes()), dtype=torch.uint8, device="cuda")
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    lib.ternaspmm_lm_head_argmax(h.data_ptr(), emb.data_ptr(), 9, 64, 64, None, out.data_ptr(), 1, sc.data_ptr(), st)
    assert lib.ternaspmm_last_status() == 1
    lib.ternaspmm_lm_head_argmax(h.data_ptr(), emb.data_ptr(), 2, 64, 48, None, out.data_ptr(), 1, sc.data_ptr(), st)
    assert lib.ternaspmm_last_status() == 1
    lib.ternaspmm_lm_head_argmax(h.data_ptr(), emb.data_ptr(), 2, 64, 64, None, out.data_ptr(), 1, None, st)
    assert lib.ternaspmm_last_status() == 2
    torch.cuda.synchronize()
    assert (out == 0).all()


def test_python_call_site(lib):
    from ternainfer_b200.linear import lm_head_argmax
    h, emb = inputs(8, 4096, 2560, seed=9)
    logits, toks = lm_head_argmax(h.view(8, 1, 2560), emb)
    assert logits.shape == (8, 4096) and toks.shape == (8,)
    assert (toks.cpu().numpy() == np.argmax(logits.cpu().numpy(), axis=1)).all()
