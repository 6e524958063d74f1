"""CPU: the checkpoint converter's scale conventions against the oracle.

Follows convert/convert_TernaInfer.py:153-199 of Gu-J/TernaInfer: every scale
segment (q, k, v / gate, up / the whole tensor) is ternarised with its own
absmean scale, the stored scale is bf16(mean|W|) and the 4-slot vector is
[q,k,v,0] / [gate,up,0,0] / [w,0,0,0].
"""
import numpy as np
import pytest
import torch

import ternaspmm_oracle as o
from ternainfer_b200.convert import convert_TernaInfer as conv
from ternainfer_b200.convert import decompress_weight

DIM, HEADS, KV_HEADS, FFN = 256, 4, 2, 384       # head_dim 64: q 256, k 128, v 128 rows


def state_dict(seed=3):
    g = torch.Generator().manual_seed(seed)
    kv = DIM // HEADS * KV_HEADS
    sd = {
        "layers.0.attention.wqkv.weight": torch.cat([0.02 * torch.randn(DIM, DIM, generator=g),
                                                     0.05 * torch.randn(kv, DIM, generator=g),
                                                     0.11 * torch.randn(kv, DIM, generator=g)]),
        "layers.0.attention.wo.weight": 0.03 * torch.randn(DIM, DIM, generator=g),
        "layers.0.feed_forward.w13.weight": torch.cat([0.04 * torch.randn(FFN, DIM, generator=g),
                                                       0.07 * torch.randn(FFN, DIM, generator=g)]),
        "layers.0.feed_forward.w2.weight": 0.01 * torch.randn(DIM, FFN, generator=g),
        "layers.0.attention_norm.weight": torch.ones(DIM),
        "tok_embeddings.weight": torch.randn(64, DIM, generator=g),
        "output.weight": torch.randn(64, DIM, generator=g),
    }
    return sd


def test_quant_weight_int8_matches_the_oracle_rule():
    g = torch.Generator().manual_seed(1)
    w = 0.03 * torch.randn(128, 192, generator=g)
    wt, scale = conv.quant_weight_int8(w)
    want_w, want_ws = o.quant_weight_ternary(w.numpy())
    assert wt.dtype == torch.int8 and scale.dtype == torch.bfloat16 and scale.shape == (1,)
    assert (wt.numpy() == want_w).all()
    assert scale.view(torch.int16).numpy().view(np.uint16)[0] == o.f32_to_bf16_bits(want_ws.reshape(1))[0]
    # degenerate input: all zeros -> clamp(mean|W|, 1e-5)
    wt0, s0 = conv.quant_weight_int8(torch.zeros(64, 64))
    assert (wt0 == 0).all() and abs(float(s0) - 1e-5) < 1e-7


def test_ternarise_state_dict_segments_and_slot_layout():
    sd = state_dict()
    out = conv.ternarise_state_dict(sd, DIM, HEADS, KV_HEADS, FFN)
    kv = DIM // HEADS * KV_HEADS
    cases = {"layers.0.attention.wqkv.weight": [DIM, kv, kv], "layers.0.attention.wo.weight": [DIM],
             "layers.0.feed_forward.w13.weight": [FFN, FFN], "layers.0.feed_forward.w2.weight": [DIM]}
    for key, segs in cases.items():
        wt = out[key]
        ws = out[key.replace("weight", "weight_scale")]
        assert wt.dtype == torch.int8 and set(np.unique(wt.numpy())) <= {-1, 0, 1}
        assert ws.dtype == torch.bfloat16 and ws.shape == (4,)
        assert int((ws != 0).sum()) == len(segs)              # ws_num as model.py:116 of the reference counts it
        assert (ws[len(segs):] == 0).all()
        assert out[key.replace("weight", "weight_segments")].tolist() == segs
        start = 0
        for i, n in enumerate(segs):                          # every segment ternarised with its OWN scale
            want_w, want_ws = o.quant_weight_ternary(sd[key][start:start + n].numpy())
            assert (wt[start:start + n].numpy() == want_w).all(), (key, i)
            assert float(ws[i]) == float(want_ws[0]), (key, i)
            start += n
    # the three q/k/v scales differ (0.02 / 0.05 / 0.11 standard deviations)
    ws = out["layers.0.attention.wqkv.weight_scale"].float()
    assert ws[0] < ws[1] < ws[2]
    assert "output.weight" not in out                         # tied head is dropped, other tensors are copied
    assert torch.equal(out["tok_embeddings.weight"], sd["tok_embeddings.weight"])


def test_pack_state_dict_schema_and_round_trip():
    sd = state_dict()
    int8_state = conv.ternarise_state_dict(sd, DIM, HEADS, KV_HEADS, FFN)
    ternary, other = conv.pack_state_dict(int8_state, "cpu")
    key = "layers.0.feed_forward.w13.weight"
    dt = {"_compressed_val": torch.uint32, "_TileOffsets_global": torch.int32, "_TileOffsets_median": torch.uint16,
          "_bitmap": torch.uint64}
    for suffix, dtype in dt.items():
        assert ternary[key + suffix].dtype == dtype            # convert_TernaInfer.py:201-209 of the reference
    N, K = int8_state[key].shape
    assert ternary[key + "_bitmap"].numel() == N * K // 64
    assert ternary[key + "_TileOffsets_global"].numel() == N * K // 4096 + 1
    assert ternary[key + "_TileOffsets_median"].numel() == 3 * N * K // 4096
    back = decompress_weight(ternary[key + "_compressed_val"], ternary[key + "_TileOffsets_global"],
                             ternary[key + "_TileOffsets_median"], ternary[key + "_bitmap"], N, K)
    assert torch.equal(back, int8_state[key])
    assert len(ternary) == 4 * 4
    assert "layers.0.attention.wqkv.weight_scale" in other and "layers.0.attention.wqkv.weight_segments" in other
    assert "layers.0.attention_norm.weight" in other and "output.weight" not in other


def test_dequantised_comparator_weights():
    sd = state_dict()
    deq = conv.dequantise_state_dict(sd, DIM, HEADS, KV_HEADS, FFN)
    int8_state = conv.ternarise_state_dict(sd, DIM, HEADS, KV_HEADS, FFN)
    key = "layers.0.attention.wqkv.weight"
    kv = DIM // HEADS * KV_HEADS
    start = 0
    for n in (DIM, kv, kv):
        seg = sd[key][start:start + n]
        s = 1.0 / seg.abs().mean().clamp(min=1e-5)
        assert torch.allclose(deq[key][start:start + n], int8_state[key][start:start + n].float() / s)
        start += n
    assert torch.equal(deq["tok_embeddings.weight"], sd["tok_embeddings.weight"])
