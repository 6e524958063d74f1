"""Checkpoint converter for the B200 TernaSpMM layout.

Follows ``convert/convert_TernaInfer.py`` of Gu-J/TernaInfer: absmean
ternarisation per scale segment with 4-slot bf16 scale vectors (:153-199),
one packed weight = four tensors under ``<key>_compressed_val`` /
``_TileOffsets_global`` / ``_TileOffsets_median`` / ``_bitmap`` (:201-209) and
three output files (:238, :267-268): ``model_bf16.pt`` (the de-quantised dense
comparator, :111-150), ``model_TernaInfer_TernaryWeights.pt`` and
``model_embeddings_and_norms_non_ternary.pt``.  One addition: next to every
``weight_scale`` vector the lengths of its scale segments are stored as
``weight_segments`` (int64), so that the call site can pass explicit segment
boundaries instead of relying on the reference's built-in rule (equal widths,
or 2560/640/640 when there are 3840 outputs), which is wrong for any other
grouped-query shape.  The packing itself is
``convert_utils.compress_weight`` (B200 tile order, vectorised, optionally on
the GPU), so no process pool is needed.  Input is a state dict with the
reference's fused names (``layers.N.attention.wqkv.weight`` ...); the
Hugging-Face download/renaming half of the reference script is not rebuilt.
``random_checkpoint`` makes the seeded synthetic checkpoints the benchmarks use.
"""
from __future__ import annotations

import argparse
import os
from typing import Dict

import torch

from .convert_utils import compress_weight


def quant_weight_int8(weight: torch.Tensor):
    """s = 1/clamp(mean|W|,1e-5); W_t = clamp(round(W*s),-1,1); scale = bf16(1/s)."""
    s = 1.0 / weight.abs().mean().clamp_(min=1e-5)
    new_weight = (weight * s).round().clamp(-1, 1).to(torch.int8)
    return new_weight, (1.0 / s).to(torch.bfloat16).reshape(1)


def _segments(key: str, value: torch.Tensor, dim: int, n_heads: int, n_kv_heads: int, ffn_dim: int):
    """Row blocks of a fused weight that get a scale of their own (convert_TernaInfer.py:168-194
    of the reference), or None for tensors that are not ternary linears."""
    head_dim = dim // n_heads
    if "wqkv" in key:
        kv = head_dim * n_kv_heads
        return [value[:dim], value[dim:dim + kv], value[dim + kv:]]
    if "w13" in key:
        return [value[:ffn_dim], value[ffn_dim:]]
    if "w2" in key or "wo" in key:
        return [value]
    return None


def dequantise_state_dict(state: Dict[str, torch.Tensor], dim: int, n_heads: int, n_kv_heads: int, ffn_dim: int):
    """The dense comparator's weights (convert_TernaInfer.py:111-150 of the reference): every
    segment ternarised and multiplied back by its scale, other tensors copied."""
    out = {}
    for key, value in state.items():
        parts = _segments(key, value, dim, n_heads, n_kv_heads, ffn_dim)
        if parts is None:
            out[key] = value.clone()
            continue
        deq = []
        for p in parts:
            s = 1.0 / p.abs().mean().clamp_(min=1e-5)
            deq.append((p * s).round().clamp(-1, 1) / s)
        out[key] = torch.cat(deq, dim=0)
    return out


def ternarise_state_dict(state: Dict[str, torch.Tensor], dim: int, n_heads: int, n_kv_heads: int, ffn_dim: int):
    """Fused bf16/fp32 weights -> int8 ternary + ``weight_scale`` vectors
    [q,k,v,0] / [gate,up,0,0] / [w,0,0,0] (+ ``weight_segments``: the segment lengths)."""
    out = {}
    zero = torch.zeros(1, dtype=torch.bfloat16)
    for key, value in state.items():
        parts = _segments(key, value, dim, n_heads, n_kv_heads, ffn_dim)
        if parts is None:
            if "output.weight" not in key:
                out[key] = value.clone()
            continue
        q = [quant_weight_int8(p.float()) for p in parts]
        out[key] = torch.cat([w for w, _ in q], dim=0)
        scales = [s.cpu() for _, s in q] + [zero] * (4 - len(q))
        out[key.replace("weight", "weight_scale")] = torch.cat(scales, dim=0)
        out[key.replace("weight", "weight_segments")] = torch.tensor([p.shape[0] for p in parts], dtype=torch.int64)
    return out


def pack_state_dict(int8_state: Dict[str, torch.Tensor], device: str = "cpu"):
    """-> (ternary tensors dict, everything else dict), as the reference saves them."""
    ternary, other = {}, {}
    for key, value in int8_state.items():
        if value.dim() == 2 and "layer" in key and value.dtype == torch.int8:
            cv, tg, tm, bm = compress_weight(value.to(device))
            ternary[key + "_compressed_val"] = cv.cpu()
            ternary[key + "_TileOffsets_global"] = tg.cpu()
            ternary[key + "_TileOffsets_median"] = tm.cpu()
            ternary[key + "_bitmap"] = bm.cpu()
        elif "output.weight" not in key:
            other[key] = value.clone()
    return ternary, other


def random_checkpoint(dim: int, n_layers: int, n_heads: int, n_kv_heads: int, ffn_dim: int, vocab_size: int,
                      seed: int = 1234, p_zero: float = 0.45, device: str = "cuda", dense: bool = False):
    """Seeded synthetic checkpoint: ternary weights i.i.d. with P(0)=p_zero and
    +-1 equiprobable, per-segment bf16 scales in [0.01, 0.05], norm weights near 1,
    N(0, 0.02^2) tied embedding.  Returns the merged dict the model loads; with
    ``dense`` the de-quantised bf16 weights (``.weight``) are added for the
    dense comparator."""
    g = torch.Generator(device=device).manual_seed(seed)
    head_dim = dim // n_heads
    dic = {}

    def tern(n, k):
        r = torch.rand((n, k), generator=g, device=device)
        sign = torch.randint(0, 2, (n, k), generator=g, device=device, dtype=torch.int8) * 2 - 1
        return torch.where(r < p_zero, torch.zeros((), dtype=torch.int8, device=device), sign)

    def norm_w(n):
        return (1.0 + 0.05 * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)

    shapes = {"attention.wqkv": ((n_heads + 2 * n_kv_heads) * head_dim, dim, [dim, n_kv_heads * head_dim,
                                                                                 n_kv_heads * head_dim]),
              "attention.wo": (dim, dim, [dim]),
              "feed_forward.w13": (2 * ffn_dim, dim, [ffn_dim, ffn_dim]),
              "feed_forward.w2": (dim, ffn_dim, [dim])}
    for i in range(n_layers):
        for name, (n, k, segs) in shapes.items():
            key = f"layers.{i}.{name}"
            w = tern(n, k)
            cv, tg, tm, bm = compress_weight(w)
            ws = torch.zeros(4, device=device)
            ws[:len(segs)] = torch.rand(len(segs), generator=g, device=device) * 0.04 + 0.01
            dic[key + ".weight_compressed_val"], dic[key + ".weight_TileOffsets_global"] = cv, tg
            dic[key + ".weight_TileOffsets_median"], dic[key + ".weight_bitmap"] = tm, bm
            dic[key + ".weight_scale"] = ws.to(torch.bfloat16)
            if len(segs) > 1:
                dic[key + ".weight_segments"] = torch.tensor(segs, dtype=torch.int64)
            if dense:
                rows = torch.repeat_interleave(ws[:len(segs)], torch.tensor(segs, device=device))
                dic[key + ".weight"] = (w.float() * rows[:, None]).to(torch.bfloat16)
                dic[key + ".weight_int8"] = w
        dic[f"layers.{i}.attention.attn_sub_norm.weight"] = norm_w(dim)
        dic[f"layers.{i}.feed_forward.ffn_sub_norm.weight"] = norm_w(ffn_dim)
        dic[f"layers.{i}.attention_norm.weight"] = norm_w(dim)
        dic[f"layers.{i}.ffn_norm.weight"] = norm_w(dim)
    dic["tok_embeddings.weight"] = (0.02 * torch.randn((vocab_size, dim), generator=g, device=device)).to(torch.bfloat16)
    dic["norm.weight"] = norm_w(dim)
    return dic


def main():
    ap = argparse.ArgumentParser(description="fused-name state dict (.pt or .safetensors) -> TernaInfer checkpoint files")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output_dir", default="./checkpoints/")
    ap.add_argument("--dim", type=int, default=2560)
    ap.add_argument("--n_heads", type=int, default=20)
    ap.add_argument("--n_kv_heads", type=int, default=5)
    ap.add_argument("--ffn_dim", type=int, default=6912)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    if a.input.endswith(".safetensors"):
        from safetensors.torch import load_file
        state = load_file(a.input)
    else:
        state = torch.load(a.input, map_location="cpu")
    os.makedirs(a.output_dir, exist_ok=True)
    torch.save(dequantise_state_dict(state, a.dim, a.n_heads, a.n_kv_heads, a.ffn_dim),
               os.path.join(a.output_dir, "model_bf16.pt"))
    int8_state = ternarise_state_dict(state, a.dim, a.n_heads, a.n_kv_heads, a.ffn_dim)
    ternary, other = pack_state_dict(int8_state, a.device)
    torch.save(ternary, os.path.join(a.output_dir, "model_TernaInfer_TernaryWeights.pt"))
    torch.save(other, os.path.join(a.output_dir, "model_embeddings_and_norms_non_ternary.pt"))
    print(f"saved {len(ternary) // 4} packed weights to {a.output_dir}")


if __name__ == "__main__":
    main()
