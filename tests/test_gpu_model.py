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
        if n == 3 and N == 3840:
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


@torch.inference_mode()
def test_decoder_block_bs1_decode_against_reference_formula(lib):
    """BASELINE config 3 (one BitNet-2B block, bs1 decode against a filled bf16 KV cache), at a
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
