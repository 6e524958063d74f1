"""GPU: one decoder block and a small full model, end to end, against the same
torch model whose ternary linears use the exact reference formula (integer GEMM
in fp32, exact because |acc| < 2**24, then the decode/prefill epilogue chosen by
token count) - not the dense bf16 comparator, which rounds twice."""
import numpy as np
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


class FormulaLinear(nn.Module):
    """acc = x_q @ W^T exactly, out = bf16(acc / s * ws[g]) (<= 64 tokens) or
    bf16(acc * (ws[g] / s)) (more), segments = the layer's real q/k/v or gate/up rows."""

    def __init__(self, in_features, out_features, dic, key, bias=False):
        super().__init__()
        self.w = dic[key + ".weight_int8"].float().cuda()
        ws = dic[key + ".weight_scale"].float().cuda()
        n = int((ws != 0).sum())
        N = out_features
        if key + ".weight_segments" in dic:
            seg = dic[key + ".weight_segments"].clone()
        elif n == 3 and N == 3840:
            seg = torch.tensor([2560, 640, 640])
        else:
            seg = torch.full((n,), N // n)
        self.ws_row = torch.repeat_interleave(ws[:n], seg.cuda())[None, :]

    def forward(self, x):
        from ternainfer_b200.linear import quant_input
        shape = list(x.shape[:-1]) + [self.w.shape[0]]
        xq, s = quant_input(x.reshape(-1, x.shape[-1]))
        acc = xq.float() @ self.w.t()
        s = s.float()
        out = acc / s * self.ws_row if xq.shape[0] <= 64 else acc * (self.ws_row / s)
        return out.to(torch.bfloat16).reshape(shape)


def build(n_layers, vocab, seed=7, max_len=96):
    from ternainfer_b200.model import ModelArgs, Transformer
    from ternainfer_b200.convert.convert_TernaInfer import random_checkpoint
    args = ModelArgs(n_layers=n_layers, vocab_size=vocab)
    dic = random_checkpoint(args.dim, n_layers, args.n_heads, args.n_kv_heads, args.ffn_dim, vocab, seed=seed, dense=True)
    with torch.device("cuda"):
        ours = Transformer(args, dic, max_seq_len=max_len).to(torch.bfloat16)
        ref = Transformer(args, dic, linear_cls=FormulaLinear, max_seq_len=max_len).to(torch.bfloat16)
    return args, ours, ref


# ---- the fused front-end's arithmetic restated with elementwise torch ops -----------------------
# (every torch op below is one correctly rounded IEEE operation per element, in the order the
# kernel's header states; nothing here calls a torch reduction)

def ordered_sum_of_squares(v: torch.Tensor) -> torch.Tensor:
    """v bf16 [M, K] -> fp32 [M, 1]: thread t of T adds f*f over elements (j*T + t)*8 + 0..7,
    warps combine by the xor butterfly 16..1, warp sums are added in warp order."""
    M, K = v.shape
    T = min(1024, max(64, (K // 8 + 31) // 32 * 32))
    J = (K // 8 + T - 1) // T
    f = torch.zeros((M, J * T * 8), dtype=torch.float32, device=v.device)
    f[:, :K] = v.float()
    f = f.view(M, J, T, 8)
    acc = torch.zeros((M, T), dtype=torch.float32, device=v.device)
    for j in range(J):
        for i in range(8):
            e = f[:, j, :, i]
            acc = acc + e * e
    acc = acc.view(M, T // 32, 32)
    lanes = torch.arange(32, device=v.device)
    for d in (16, 8, 4, 2, 1):
        acc = acc + acc[:, :, lanes ^ d]
    r = acc[:, 0, 0]
    for wi in range(1, T // 32):
        r = r + acc[:, wi, 0]
    return r.reshape(M, 1)


def ordered_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm(x) * w in the kernel's order: 1 / sqrt(ss / K + eps), (x * rstd) * w, bf16."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    ss = ordered_sum_of_squares(x2)
    kk = torch.full_like(ss, float(x2.shape[1]))            # tensor divisor: a true division per element
    rstd = torch.ones_like(ss) / torch.sqrt(ss / kk + eps)
    return ((x2.float() * rstd) * w.float()).to(torch.bfloat16).reshape(shape)


def ordered_norm_quant(x, w, eps, gated=False):
    from ternainfer_b200.linear import quant_input
    if gated:
        x1, x3 = x.chunk(2, -1)
        x = torch.relu(x1) ** 2 * x3
    return quant_input(ordered_norm(x, w, eps))


def build_pair_same_glue(n_layers, vocab, seed=7, max_len=96):
    """(fused-glue model on this library's kernels, the SAME model in eager torch with every ternary
    linear on the exact reference formula and every norm in the fused kernels' stated
    order).  Both use flash_attn's kv-cache kernel for the attention glue (library code)."""
    import types
    from ternainfer_b200.model import ModelArgs, Transformer, RMSNorm
    from ternainfer_b200.convert.convert_TernaInfer import random_checkpoint
    fargs = ModelArgs(n_layers=n_layers, vocab_size=vocab, fused_glue=True, flash_attention=True)
    rargs = ModelArgs(n_layers=n_layers, vocab_size=vocab, fused_glue=False, flash_attention=True)
    dic = random_checkpoint(fargs.dim, n_layers, fargs.n_heads, fargs.n_kv_heads, fargs.ffn_dim, vocab, seed=seed,
                            dense=True)
    with torch.device("cuda"):
        fused = Transformer(fargs, dic, max_seq_len=max_len).to(torch.bfloat16)
        ref = Transformer(rargs, dic, linear_cls=FormulaLinear, max_seq_len=max_len).to(torch.bfloat16)

    def fwd(self, x):
        return ordered_norm(x, self.weight, self.eps)

    for m in ref.modules():      # every norm of the model, the final one in front of the output head included
        if isinstance(m, RMSNorm):
            m.forward = types.MethodType(fwd, m)
    return fused, ref


@torch.inference_mode()
def test_decoder_block_bs1_decode_against_reference_formula(lib):
    """One BitNet-2B decoder block (bs1 decode against a filled bf16 KV cache), at a
    shorter cache so the test stays small."""
    args, ours, ref = build(1, 512, max_len=128)
    g = torch.Generator(device="cuda").manual_seed(3)
    c1, c2 = ours.make_cache(1, "cuda"), ref.make_cache(1, "cuda")
    for (k1, v1), (k2, v2) in zip(c1, c2):
        k1.copy_(torch.randn(k1.shape, generator=g, device="cuda"))
        v1.copy_(torch.randn(v1.shape, generator=g, device="cuda"))
        k2.copy_(k1), v2.copy_(v1)
    tok = torch.randint(0, 512, (1, 1), generator=g, device="cuda")
    pos = torch.tensor([100], device="cuda")
    a, b = ours(tok, c1, pos), ref(tok, c2, pos)
    assert torch.equal(a, b)


@torch.inference_mode()
def test_small_model_greedy_tokens_identical(lib):
    from ternainfer_b200.generate import FastGen, GenArgs
    args, ours, ref = build(2, 1024, max_len=96)
    g = torch.Generator(device="cuda").manual_seed(11)
    for bsz in (1, 8):
        prompt = torch.randint(0, 1024, (bsz, 64), generator=g, device="cuda")
        t1, _ = FastGen(ours, GenArgs(16, bsz, 64, True)).generate(prompt)
        t2, _ = FastGen(ref, GenArgs(16, bsz, 64, False)).generate(prompt)
        assert torch.equal(t1, t2)


def torch_norm_quant(x, w, eps, gated=False):
    """The unfused glue: (gate ->) RMSNorm in fp32 -> bf16 -> eager quantiser."""
    from ternainfer_b200.linear import quant_input
    if gated:
        x1, x3 = x.chunk(2, -1)
        x = torch.relu(x1) ** 2 * x3
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)
    return quant_input(y)


@pytest.mark.parametrize("M,K", [(1, 2560), (8, 2560), (300, 2560), (5, 28672), (3, 64), (2, 8192)])
def test_rmsnorm_kernel_bit_exact_against_its_stated_order(lib, M, K):
    """ternaspmm_rmsnorm (the model's final norm in fused-glue mode): every bf16 output equals the
    restatement of its summation order; in place too."""
    from ternainfer_b200.linear import rmsnorm
    g = torch.Generator(device="cuda").manual_seed(M * 7 + K)
    x = (torch.randn((M, K), generator=g, device="cuda") * 3).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(K, generator=g, device="cuda")).to(torch.bfloat16)
    want = ordered_norm(x, w, 1e-5)
    assert torch.equal(rmsnorm(x, w, 1e-5), want)
    y = x.clone()
    lib.ternaspmm_rmsnorm(y.data_ptr(), w.data_ptr(), 1e-5, M, K, y.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert lib.ternaspmm_last_status() == 0 and torch.equal(y, want)


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("M,K", [(1, 2560), (8, 2560), (8, 6912), (33, 8192), (5, 28672), (3, 64)])
def test_fused_norm_quant_against_torch(lib, gated, M, K):
    """Floating-point kernel: the scale must agree within one bf16 ulp and the int8 values
    within one step on at most 0.5 % of the elements (the sum of squares is accumulated in a
    different order than torch's reduction); everything else must be identical."""
    from ternainfer_b200.linear import rmsnorm_quant
    g = torch.Generator(device="cuda").manual_seed(M * 7 + K)
    x = torch.randn((M, 2 * K if gated else K), generator=g, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(K, generator=g, device="cuda")).to(torch.bfloat16)
    q, s = rmsnorm_quant(x, w, 1e-5, gated=gated)
    q_ref, s_ref = torch_norm_quant(x, w, 1e-5, gated)
    assert q.shape == q_ref.shape and s.shape == s_ref.shape
    rel = ((s.float() - s_ref.float()).abs() / s_ref.float()).max().item()
    assert rel <= 2.0 ** -7
    d = (q.int() - q_ref.int()).abs()
    assert d.max().item() <= 1
    assert (d != 0).float().mean().item() <= 0.005 or rel > 0   # a scale one ulp apart moves more values by one step
    same_scale = (s == s_ref).reshape(-1)
    if same_scale.any():
        assert (d[same_scale] != 0).float().mean().item() <= 0.005


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("M,K", [(1, 2560), (8, 2560), (8, 6912), (33, 8192), (5, 28672), (3, 64), (2, 10240)])
def test_fused_norm_quant_bit_exact_against_its_stated_order(lib, gated, M, K):
    """The fused front-end against its own formula restated op by op (fixed summation order, IEEE
    division and square root): int8 values and scales identical."""
    from ternainfer_b200.linear import rmsnorm_quant
    g = torch.Generator(device="cuda").manual_seed(M * 11 + K)
    x = torch.randn((M, 2 * K if gated else K), generator=g, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(K, generator=g, device="cuda")).to(torch.bfloat16)
    q, s = rmsnorm_quant(x, w, 1e-5, gated=gated)
    q_ref, s_ref = ordered_norm_quant(x, w, 1e-5, gated)
    assert torch.equal(s, s_ref.to(torch.bfloat16))
    assert torch.equal(q, q_ref)


@torch.inference_mode()
def test_fused_glue_model_logits_and_greedy_tokens_identical(lib):
    """The benchmarked decode path (fused norm/gate/quantiser kernels, residual add in the linear
    epilogue, flash_attn glue) against the eager model on the reference formula with the same glue
    arithmetic: logits equal bit for bit on a prefill and a decode step, greedy tokens identical."""
    pytest.importorskip("flash_attn")
    from ternainfer_b200.generate import FastGen, GenArgs
    fused, ref = build_pair_same_glue(2, 1024, max_len=96)
    g = torch.Generator(device="cuda").manual_seed(21)
    tok = torch.randint(0, 1024, (2, 40), generator=g, device="cuda")
    c1, c2 = fused.make_cache(2, "cuda"), ref.make_cache(2, "cuda")
    pos = torch.arange(40, device="cuda")
    assert torch.equal(fused(tok, c1, pos), ref(tok, c2, pos))
    nxt = torch.randint(0, 1024, (2, 1), generator=g, device="cuda")
    p1 = torch.tensor([40], device="cuda")
    assert torch.equal(fused(nxt, c1, p1), ref(nxt, c2, p1))
    for bsz in (1, 8):
        prompt = torch.randint(0, 1024, (bsz, 64), generator=g, device="cuda")
        t1, _ = FastGen(fused, GenArgs(16, bsz, 64, True)).generate(prompt)
        t2, _ = FastGen(ref, GenArgs(16, bsz, 64, False)).generate(prompt)
        assert torch.equal(t1, t2)


@torch.inference_mode()
def test_full_30_layer_model_greedy_tokens_identical(lib):
    """The full architecture (30 layers, vocabulary 128256, prompt of 512 seeded ids): greedy tokens
    of the fused-glue model under CUDA graphs equal those of the eager reference-formula model, 128
    tokens at batch 1 and 24 tokens at batch 8."""
    pytest.importorskip("flash_attn")
    from ternainfer_b200.generate import FastGen, GenArgs
    fused, ref = build_pair_same_glue(30, 128256, seed=1234, max_len=640)
    g = torch.Generator(device="cuda").manual_seed(1235)
    for bsz, n in ((1, 128), (8, 24)):
        prompt = torch.randint(0, 128256, (bsz, 512), generator=g, device="cuda")
        t1, _ = FastGen(fused, GenArgs(n, bsz, 512, True)).generate(prompt)
        t2, _ = FastGen(ref, GenArgs(n, bsz, 512, False)).generate(prompt)
        assert torch.equal(t1, t2), (bsz, (t1 != t2).nonzero()[:4].tolist())


def test_residual_epilogue_bit_exact(lib):
    from ternainfer_b200.linear import SpBitLinear, quant_input
    from ternainfer_b200.convert import compress_weight
    import ternaspmm_oracle as o
    N, K, M = 2560, 2560, 8
    w = o.make_ternary(N, K, 0.45, seed=91)
    cv, tg, tm, bm = compress_weight(torch.from_numpy(w))
    dic = {"l.weight_compressed_val": cv, "l.weight_TileOffsets_global": tg, "l.weight_TileOffsets_median": tm,
           "l.weight_bitmap": bm, "l.weight_scale": torch.tensor([0.03, 0, 0, 0]).to(torch.bfloat16)}
    layer = SpBitLinear(K, N, dic, "l")
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    res = torch.randn((M, N), generator=g, device="cuda").to(torch.bfloat16)
    xq, s = quant_input(x)
    assert torch.equal(layer.forward_quantized(xq, s, residual=res), res + layer(x))
    for big in (100, 300):    # the tensor-core kernel's epilogue
        xb = torch.randn((big, K), generator=g, device="cuda").to(torch.bfloat16)
        rb = torch.randn((big, N), generator=g, device="cuda").to(torch.bfloat16)
        xq, s = quant_input(xb)
        assert torch.equal(layer.forward_quantized(xq, s, residual=rb), rb + layer(xb))


@torch.inference_mode()
def test_fused_glue_model_close_to_unfused(lib):
    """The fused-glue model computes the same function up to the summation order of the norms:
    logits must agree closely and the greedy continuation must start identically."""
    import copy
    args, ours, _ = build(2, 1024, max_len=96)
    fused = copy.copy(ours)
    fused.args = copy.copy(args)
    fused.args.fused_glue = True
    g = torch.Generator(device="cuda").manual_seed(13)
    tok = torch.randint(0, 1024, (2, 48), generator=g, device="cuda")
    pos = torch.arange(48, device="cuda")
    a = ours(tok, ours.make_cache(2, "cuda"), pos)
    b = fused(tok, fused.make_cache(2, "cuda"), pos)
    err = (a - b).abs().max().item() / a.abs().max().item()
    assert err < 0.05, err
    assert (a.argmax(-1) == b.argmax(-1)).float().mean().item() > 0.9


@torch.inference_mode()
def test_fused_glue_with_flash_attention_close_to_unfused(lib):
    """Same check with the attention glue routed through flash_attn's kv-cache kernel
    (RoPE + cache append + attention in one library launch), prefill then one decode step."""
    pytest.importorskip("flash_attn")
    from ternainfer_b200.model import ModelArgs, Transformer
    from ternainfer_b200.convert.convert_TernaInfer import random_checkpoint
    args = ModelArgs(n_layers=2, vocab_size=1024)
    dic = random_checkpoint(args.dim, 2, args.n_heads, args.n_kv_heads, args.ffn_dim, 1024, seed=7)
    fargs = ModelArgs(n_layers=2, vocab_size=1024, fused_glue=True)
    with torch.device("cuda"):
        plain = Transformer(args, dic, max_seq_len=96).to(torch.bfloat16)
        fused = Transformer(fargs, dic, max_seq_len=96).to(torch.bfloat16)
    assert fused.flash
    g = torch.Generator(device="cuda").manual_seed(17)
    tok = torch.randint(0, 1024, (2, 40), generator=g, device="cuda")
    c1, c2 = plain.make_cache(2, "cuda"), fused.make_cache(2, "cuda")
    pos = torch.arange(40, device="cuda")
    a, b = plain(tok, c1, pos), fused(tok, c2, pos)
    assert (a - b).abs().max().item() / a.abs().max().item() < 0.05
    nxt = torch.randint(0, 1024, (2, 1), generator=g, device="cuda")
    p1 = torch.tensor([40], device="cuda")
    a, b = plain(nxt, c1, p1), fused(nxt, c2, p1)
    assert (a - b).abs().max().item() / a.abs().max().item() < 0.05
