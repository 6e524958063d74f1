"""BitNet-b1.58 style decoder around the TernaSpMM call site.

Thin PyTorch glue so that a decoder block and the full model can be run and
timed end to end; only the four ternary linears per layer (``wqkv``, ``wo``,
``w13``, ``w2``) are the hand-written path.  Shapes and order of operations
follow ``model.py`` of Gu-J/TernaInfer (:155-386): GQA attention with RoPE on
adjacent pairs, RMSNorm before each sub-block, a sub-layer norm before ``wo``
and ``w2``, ReLU^2 gated FFN, tied bf16 embedding / output head.  The
reference's xformers ops are replaced by plain torch (RMSNorm, RoPE, SDPA over
a dense per-sequence KV cache), and nothing goes through ``torch.compile``.
With ``tp`` > 1 the linears are the column-/row-parallel versions of
``ternainfer_b200.tp``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
from torch import nn
from torch.nn import functional as F

from .linear import SpBitLinear, quant_input, rmsnorm, rmsnorm_quant, lm_head_argmax


@dataclass
class ModelArgs:
    dim: int = 2560
    n_layers: int = 30
    n_heads: int = 20
    n_kv_heads: int = 5
    vocab_size: int = 128256
    ffn_dim: int = 6912
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    use_kernel: bool = True
    fused_glue: bool = False     # fused norm+quantiser kernels and residual add in the linear epilogue
    flash_attention: Optional[bool] = None   # attention glue through flash_attn's kv-cache kernel; None = with fused_glue

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads


LayerCache = Tuple[torch.Tensor, torch.Tensor]


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y * self.weight.float()).to(x.dtype)


class BF16BitLinear(nn.Module):
    """Dense comparator (model.py:135-153 of the reference): same quantiser,
    bf16 GEMM on the de-quantised ternary weight, division by the scale."""

    def __init__(self, in_features, out_features, dic, key, bias=False):
        super().__init__()
        self.weight = nn.Parameter(dic[key + ".weight"].cuda(), requires_grad=False)

    def forward(self, input):
        xq, s = quant_input(input)
        return F.linear(xq.to(torch.bfloat16), self.weight) / s


def rope_tables(head_dim: int, max_len: int, theta: float, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    ang = torch.outer(torch.arange(max_len, device=device).float(), inv)
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
    """Rotate adjacent pairs (2i, 2i+1); x [B, T, H, D], cos/sin [B, T, D/2]."""
    xf = x.float().unflatten(-1, (-1, 2))
    a, b = xf[..., 0], xf[..., 1]
    c, s = cos.unsqueeze(2), sin.unsqueeze(2)
    return torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, args: ModelArgs, dic: dict, prefix: str, linear_cls, tp_group=None, tp: int = 1):
        super().__init__()
        self.head_dim = args.head_dim
        self.n_heads = args.n_heads // tp
        self.n_kv_heads = args.n_kv_heads // tp
        qkv_out = (args.n_heads + 2 * args.n_kv_heads) * self.head_dim
        if tp > 1:
            from .tp import ColumnParallelSpBitLinear, RowParallelSpBitLinear
            self.wqkv = ColumnParallelSpBitLinear(args.dim, qkv_out // tp, dic, prefix + ".wqkv")
            self.wo = RowParallelSpBitLinear(args.dim // tp, args.dim, dic, prefix + ".wo", tp_group,
                                             norm_weight=dic[prefix + ".attn_sub_norm.weight"], eps=args.norm_eps)
            self.attn_sub_norm = None
        else:
            self.wqkv = linear_cls(args.dim, qkv_out, dic, prefix + ".wqkv")
            self.wo = linear_cls(args.dim, args.dim, dic, prefix + ".wo")
            self.attn_sub_norm = RMSNorm(args.dim, args.norm_eps)
            with torch.no_grad():
                self.attn_sub_norm.weight.copy_(dic[prefix + ".attn_sub_norm.weight"])

    def forward(self, x, cache: LayerCache, pos, cos, sin, mask, fused=None):
        """``fused`` = (x_q, s, residual, eps): quantised input of wqkv and the residual for wo's epilogue."""
        B, T = x.shape[0], x.shape[1]
        H, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self.wqkv(x) if fused is None else self.wqkv.forward_quantized(fused[0], fused[1])
        q = qkv[..., : H * D].view(B, T, H, D)
        k = qkv[..., H * D: (H + Hkv) * D].view(B, T, Hkv, D)
        v = qkv[..., (H + Hkv) * D:].view(B, T, Hkv, D)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        ck, cv = cache                                  # [B, Hkv, L, D]
        ck.index_copy_(2, pos, k.transpose(1, 2))
        cv.index_copy_(2, pos, v.transpose(1, 2))
        o = F.scaled_dot_product_attention(q.transpose(1, 2), ck, cv, attn_mask=mask, enable_gqa=True)
        o = o.transpose(1, 2).reshape(B, T, H * D)
        return self._project(o, fused)

    def forward_flash(self, x, cache: LayerCache, seqlens, cos_tab, sin_tab, fused):
        """Attention glue through flash_attn's kv-cache kernel (library code, not part of the
        TernaSpMM path): RoPE on adjacent pairs, cache append and causal attention in one
        launch.  Cache layout [B, L, Hkv, D]."""
        from flash_attn import flash_attn_with_kvcache
        B, T = x.shape[0], x.shape[1]
        H, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self.wqkv(x) if fused is None else self.wqkv.forward_quantized(fused[0], fused[1])
        q = qkv[..., : H * D].view(B, T, H, D)
        k = qkv[..., H * D: (H + Hkv) * D].view(B, T, Hkv, D)
        v = qkv[..., (H + Hkv) * D:].view(B, T, Hkv, D)
        o = flash_attn_with_kvcache(q, cache[0], cache[1], k=k, v=v, rotary_cos=cos_tab, rotary_sin=sin_tab,
                                    cache_seqlens=seqlens, causal=True, rotary_interleaved=True)
        return self._project(o.reshape(B, T, H * D), fused)

    def _project(self, o, fused):
        if fused is not None:
            oq, os_ = rmsnorm_quant(o, self.attn_sub_norm.weight, fused[3])
            return self.wo.forward_quantized(oq, os_, residual=fused[2])
        if self.attn_sub_norm is not None:
            o = self.attn_sub_norm(o)
        return self.wo(o)


class FeedForward(nn.Module):
    def __init__(self, args: ModelArgs, dic: dict, prefix: str, linear_cls, tp_group=None, tp: int = 1):
        super().__init__()
        if tp > 1:
            from .tp import ColumnParallelSpBitLinear, RowParallelSpBitLinear
            self.w13 = ColumnParallelSpBitLinear(args.dim, 2 * args.ffn_dim // tp, dic, prefix + ".w13")
            self.w2 = RowParallelSpBitLinear(args.ffn_dim // tp, args.dim, dic, prefix + ".w2", tp_group,
                                             norm_weight=dic[prefix + ".ffn_sub_norm.weight"], eps=args.norm_eps)
            self.ffn_sub_norm = None
        else:
            self.w13 = linear_cls(args.dim, 2 * args.ffn_dim, dic, prefix + ".w13")
            self.w2 = linear_cls(args.ffn_dim, args.dim, dic, prefix + ".w2")
            self.ffn_sub_norm = RMSNorm(args.ffn_dim, args.norm_eps)
            with torch.no_grad():
                self.ffn_sub_norm.weight.copy_(dic[prefix + ".ffn_sub_norm.weight"])

    def forward_fused(self, xq, s, residual, eps):
        x13 = self.w13.forward_quantized(xq, s)
        iq, is_ = rmsnorm_quant(x13, self.ffn_sub_norm.weight, eps, gated=True)
        return self.w2.forward_quantized(iq, is_, residual=residual)

    def forward(self, x):
        x1, x3 = self.w13(x).chunk(2, -1)
        inner = F.relu(x1) ** 2 * x3
        if self.ffn_sub_norm is not None:
            inner = self.ffn_sub_norm(inner)
        return self.w2(inner)


class TransformerBlock(nn.Module):
    def __init__(self, args: ModelArgs, dic: dict, prefix: str, linear_cls, tp_group=None, tp: int = 1):
        super().__init__()
        self.attention = Attention(args, dic, prefix + ".attention", linear_cls, tp_group, tp)
        self.feed_forward = FeedForward(args, dic, prefix + ".feed_forward", linear_cls, tp_group, tp)
        self.attention_norm = RMSNorm(args.dim, args.norm_eps)
        self.ffn_norm = RMSNorm(args.dim, args.norm_eps)
        with torch.no_grad():
            self.attention_norm.weight.copy_(dic[prefix + ".attention_norm.weight"])
            self.ffn_norm.weight.copy_(dic[prefix + ".ffn_norm.weight"])

    def forward(self, x, cache, pos, cos, sin, mask, fused: bool = False, flash=None):
        if fused:
            eps = self.attention_norm.eps
            xq, s = rmsnorm_quant(x, self.attention_norm.weight, eps)
            if flash is not None:
                h = self.attention.forward_flash(x, cache, flash[0], flash[1], flash[2], (xq, s, x, eps))
            else:
                h = self.attention(x, cache, pos, cos, sin, mask, fused=(xq, s, x, eps))
            hq, hs = rmsnorm_quant(h, self.ffn_norm.weight, eps)
            return self.feed_forward.forward_fused(hq, hs, h, eps)
        if flash is not None:
            h = x + self.attention.forward_flash(self.attention_norm(x), cache, flash[0], flash[1], flash[2], None)
        else:
            h = x + self.attention(self.attention_norm(x), cache, pos, cos, sin, mask)
        return h + self.feed_forward(self.ffn_norm(h))


class Transformer(nn.Module):
    """``dic`` holds the checkpoint tensors under the reference's key names
    (``layers.<i>.attention.wqkv.weight_bitmap`` ... ``tok_embeddings.weight``,
    ``norm.weight``); the output head is tied to the embedding."""

    def __init__(self, args: ModelArgs, dic: dict, linear_cls=None, max_seq_len: int = 2048, tp_group=None,
                 tp: int = 1):
        super().__init__()
        self.args = args
        linear_cls = linear_cls or (SpBitLinear if args.use_kernel else BF16BitLinear)
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim)
        with torch.no_grad():
            self.tok_embeddings.weight.copy_(dic["tok_embeddings.weight"])
        self.layers = nn.ModuleList([TransformerBlock(args, dic, f"layers.{i}", linear_cls, tp_group, tp)
                                     for i in range(args.n_layers)])
        self.norm = RMSNorm(args.dim, args.norm_eps)
        with torch.no_grad():
            self.norm.weight.copy_(dic["norm.weight"])
        self.max_seq_len = max_seq_len
        self.tp = tp
        self._rope = None
        self.flash = False
        want_flash = args.fused_glue if args.flash_attention is None else args.flash_attention
        if want_flash and tp == 1:
            try:
                import flash_attn  # noqa: F401
                self.flash = True
            except Exception:
                if args.flash_attention:
                    raise
                self.flash = False

    def make_cache(self, batch: int, device, dtype=torch.bfloat16) -> List[LayerCache]:
        a = self.args
        shape = (batch, a.n_kv_heads // self.tp, self.max_seq_len, a.head_dim)
        if self.flash:
            shape = (batch, self.max_seq_len, a.n_kv_heads, a.head_dim)
        return [(torch.zeros(shape, device=device, dtype=dtype), torch.zeros(shape, device=device, dtype=dtype))
                for _ in range(a.n_layers)]

    def head(self, h: torch.Tensor, greedy: bool = False):
        """Final norm + tied output head.  fp32 logits [B, T, vocab] (model.py:380-386 of the
        reference); with ``greedy`` -> (None, int64 tokens [B, T]) without materialising the logits.
        Up to 8 rows run on the library's head kernel (one pass over the embedding, arg-max fused);
        more rows use the dense bf16 GEMM."""
        B, T = h.shape[0], h.shape[1]
        if self.args.fused_glue and h.is_cuda and h.dtype == torch.bfloat16 and h.shape[-1] % 16 == 0:
            h = rmsnorm(h, self.norm.weight, self.norm.eps)   # one launch, the fused front-ends' summation order
        else:
            h = self.norm(h)
        emb = self.tok_embeddings.weight
        if h.is_cuda and B * T <= 8 and emb.dtype == torch.bfloat16 and h.dtype == torch.bfloat16 and h.shape[-1] % 32 == 0:
            logits, toks = lm_head_argmax(h, emb, want_logits=not greedy, want_argmax=greedy)
            return (None, toks.view(B, T)) if greedy else logits.view(B, T, -1)
        logits = F.linear(h, emb).float()
        return (None, logits.argmax(-1)) if greedy else logits

    def forward(self, tokens: torch.Tensor, cache: List[LayerCache], pos: torch.Tensor, greedy_last: bool = False):
        """tokens [B, T]; pos [T] (device int64) = positions written in the cache.
        Returns fp32 logits [B, T, vocab] (model.py:380-386 of the reference); with ``greedy_last``
        only the greedy token of every sequence's last position, int64 [B] (what the generation
        loop needs: generate.py:274, :283, :305 of the reference)."""
        if self._rope is None or self._rope[0].device != tokens.device:
            self._rope = rope_tables(self.args.head_dim, self.max_seq_len, self.args.rope_theta, tokens.device)
            self._rope_lp = (self._rope[0].to(torch.bfloat16), self._rope[1].to(torch.bfloat16))
        B, T = tokens.shape
        h = self.tok_embeddings(tokens)
        fused = self.args.fused_glue and self.tp == 1
        flash, cos, sin, mask = None, None, None, None
        if self.flash:   # the kv-cache kernel applies RoPE from the tables and masks by sequence length itself
            flash = (pos[:1].to(torch.int32).expand(B).contiguous(), self._rope_lp[0], self._rope_lp[1])
        else:
            cos, sin = self._rope[0][pos].expand(B, T, -1), self._rope[1][pos].expand(B, T, -1)
            keys = torch.arange(self.max_seq_len, device=tokens.device)
            mask = (keys[None, :] <= pos[:, None])[None, None]      # [1, 1, T, L] causal over cache positions
        for layer, c in zip(self.layers, cache):
            h = layer(h, c, pos, cos, sin, mask, fused, flash)
        if greedy_last:
            return self.head(h[:, -1:], greedy=True)[1][:, 0]
        return self.head(h)
