"""CPU, world_size 2 (gloo): the tensor-parallel sharding and collective logic.
The GPU kernel calls are replaced by the CPU oracle so that only the host logic
(sharding, segment boundaries, statistics exchange, all-reduce) is under test."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import ternaspmm_oracle as o


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_accumulate(xq, packed, N):
    cv, tg, tm, bm = [p.numpy() for p in packed]
    K = xq.shape[1]
    w = o.decode_weight_b200(cv, tg, tm, bm, N, K)
    return torch.from_numpy(o.gemm_i32(xq.numpy(), w))


def _oracle_linear_segments(xq, s, packed, ws, bounds, N):
    acc = _oracle_accumulate(xq, packed, N).numpy()
    col = np.arange(N)
    g = sum((col >= b).astype(np.int64) for b in bounds) if bounds else np.zeros(N, np.int64)
    wsf = ws.float().numpy()[g][None, :]
    v = (acc.astype(np.float32) / s.float().numpy().reshape(-1, 1)).astype(np.float32) * wsf
    return torch.from_numpy(o.f32_to_bf16_bits(v).view(np.int16)).view(torch.bfloat16)


def _worker(rank, world, port, mode, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ternainfer_b200 import tp
    tp._accumulate_i32, tp._linear_segments = _oracle_accumulate, _oracle_linear_segments
    torch.manual_seed(0)
    dim, H, Hkv, D, ffn, M = 256, 4, 2, 64, 512, 5
    x = torch.randn(M, dim).to(torch.bfloat16)
    res = {}
    # ---- column-parallel QKV with unequal segments, then gather and compare with the unsharded layer
    segs = [H * D, Hkv * D, Hkv * D]
    wqkv = torch.from_numpy(o.make_ternary(sum(segs), dim, 0.45, 1))
    ws = torch.tensor([0.02, 0.03, 0.04, 0.0]).to(torch.bfloat16)
    dic = {}
    tp.shard_checkpoint_entry(dic, "qkv", wqkv, ws, segs, "column", rank, world)
    col = tp.ColumnParallelSpBitLinear(dim, sum(segs) // world, dic, "qkv")
    y_local = col(x)
    gathered = [torch.empty_like(y_local) for _ in range(world)]
    dist.all_gather(gathered, y_local)
    full = {}
    tp.shard_checkpoint_entry(full, "qkv", wqkv, ws, segs, "column", 0, 1)
    y_full = tp.ColumnParallelSpBitLinear(dim, sum(segs), full, "qkv")(x)
    # reassemble: rank r holds [q_r, k_r, v_r]
    loc = tp.local_segments(segs, world)
    parts = []
    for si in range(3):
        for r in range(world):
            st = sum(loc[:si])
            parts.append(gathered[r][:, st:st + loc[si]])
    res["column_equal"] = bool(torch.equal(torch.cat(parts, dim=1), y_full))
    # ---- row-parallel down projection
    w2 = torch.from_numpy(o.make_ternary(dim, ffn, 0.45, 2))
    g = (1 + 0.05 * torch.randn(ffn)).to(torch.bfloat16)
    inner = torch.randn(M, ffn).to(torch.bfloat16)
    ws2 = torch.tensor([0.025, 0, 0, 0]).to(torch.bfloat16)
    dic2, one = {}, {}
    tp.shard_checkpoint_entry(dic2, "w2", w2, ws2, None, "row", rank, world)
    tp.shard_checkpoint_entry(one, "w2", w2, ws2, None, "row", 0, 1)
    row = tp.RowParallelSpBitLinear(ffn // world, dim, dic2, "w2", None, tp.shard_vector(g, rank, world), 1e-5, mode)
    y = row(tp.shard_vector(inner.t().contiguous(), rank, world).t().contiguous())
    ref = tp.RowParallelSpBitLinear(ffn, dim, one, "w2", None, g, 1e-5, "exact")
    ref.tp = 1
    y_ref = ref(inner)
    res["row_equal"] = bool(torch.equal(y, y_ref))
    res["row_max_rel"] = float((y.float() - y_ref.float()).abs().max() / y_ref.float().pow(2).mean().sqrt())
    if rank == 0:
        q.put(res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["exact", "single"])
def test_two_rank_tensor_parallel_linears(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res["column_equal"]
    if mode == "exact":
        assert res["row_equal"], res      # bit-identical to the unsharded layer
    else:
        assert res["row_max_rel"] < 0.05, res   # one collective: max error under 5 % of the output RMS (quantisation noise)


def _leaving_worker(rank, world, port, q):
    """Rank 1 leaves between two steps (no collective in flight) after announcing it through the store;
    rank 0 checks for its peers on the host before its next step and must get an error there - it never
    enters a collective that could only time out."""
    import datetime
    import time
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    from ternainfer_b200 import tp
    tp._accumulate_i32, tp._linear_segments = _oracle_accumulate, _oracle_linear_segments
    torch.manual_seed(0)
    dim, ffn, M = 128, 256, 3
    w2 = torch.from_numpy(o.make_ternary(dim, ffn, 0.45, 2))
    dic = {}
    tp.shard_checkpoint_entry(dic, "w2", w2, torch.tensor([0.025, 0, 0, 0]).to(torch.bfloat16), None, "row", rank, world)
    row = tp.RowParallelSpBitLinear(ffn // world, dim, dic, "w2", None, torch.ones(ffn // world), 1e-5, "single")
    x = torch.randn(M, ffn // world).to(torch.bfloat16)
    store = dist.distributed_c10d._get_default_store()
    tp.check_peers(store, rank, world)
    y = row(x)                       # step 1: both ranks take part
    dist.barrier()
    if rank == 0:
        store.set("rank0_past_step1", "1")
    else:
        # leave only once rank 0 is known (through the store) to be out of the barrier: nothing of
        # step 1 is in flight any more
        store.wait(["rank0_past_step1"])
        tp.announce_leaving(store, rank)
        os._exit(0)
    store.wait(["tp_rank_left_1"])   # (the test's own synchronisation: the peer has announced itself)
    t0 = time.monotonic()
    try:
        tp.check_peers(store, rank, world)   # what a driver loop does before every step
        row(x)
        q.put(("no error", time.monotonic() - t0, bool(torch.isfinite(y.float()).all())))
    except RuntimeError as e:
        q.put((str(e), time.monotonic() - t0, bool(torch.isfinite(y.float()).all())))
    q.close()
    q.join_thread()                  # the queue's feeder thread has written the result before the process ends
    os._exit(0)


def test_rank_leaving_between_steps_raises_on_the_other_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    kind, seconds, step1_ok = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
    assert step1_ok
    assert "has left the group" in kind, kind
    assert seconds < 5


def test_shard_helpers():
    from ternainfer_b200 import tp
    w = torch.arange(12 * 128).reshape(12, 128)
    a = tp.shard_rows(w, [8, 2, 2], 1, 2)
    assert a.shape == (6, 128) and torch.equal(a[:4], w[4:8]) and torch.equal(a[4], w[9]) and torch.equal(a[5], w[11])
    b = tp.shard_cols(w, 1, 2)
    assert torch.equal(b, w[:, 64:])
    with pytest.raises(AssertionError):
        tp.shard_rows(w, [7, 3, 2], 0, 2)


def test_sharded_model_checkpoint_reassembles_the_unsharded_weights():
    """shard_model_checkpoint (CPU): the ranks' packed shards, decoded again and put back together, are the
    unsharded ternary weights - QKV and gate-up split by rows of every scale segment (whole heads per rank),
    O and down by columns - and the sub-layer norm weights are sliced like the columns they scale."""
    from ternainfer_b200 import tp
    from ternainfer_b200.convert import decompress_weight
    from ternainfer_b200.convert.convert_TernaInfer import random_checkpoint
    dim, H, Hkv, ffn, world = 256, 4, 2, 512, 2
    D = dim // H
    full = random_checkpoint(dim, 1, H, Hkv, ffn, 64, seed=3, device="cpu", dense=True)
    shards = [tp.shard_model_checkpoint(full, 1, r, world) for r in range(world)]

    def dense(dic, key, n, k):
        assert dic[key + ".weight_bitmap"].numel() * 64 == n * k
        return decompress_weight(dic[key + ".weight_compressed_val"], dic[key + ".weight_TileOffsets_global"],
                                 dic[key + ".weight_TileOffsets_median"], dic[key + ".weight_bitmap"], n, k)

    p = "layers.0."
    wqkv = full[p + "attention.wqkv.weight_int8"]
    q, k, v = wqkv[:H * D], wqkv[H * D:(H + Hkv) * D], wqkv[(H + Hkv) * D:]
    for r in range(world):
        got = torch.as_tensor(dense(shards[r], p + "attention.wqkv", (H + 2 * Hkv) * D // world, dim))
        want = torch.cat([q[r * H * D // world:(r + 1) * H * D // world], k[r * Hkv * D // world:(r + 1) * Hkv * D // world],
                          v[r * Hkv * D // world:(r + 1) * Hkv * D // world]])
        assert torch.equal(got, want)
        assert shards[r][p + "attention.wqkv.weight_segments"].tolist() == [H * D // world, Hkv * D // world, Hkv * D // world]
    for name, kind in (("attention.wo", "row"), ("feed_forward.w2", "row"), ("feed_forward.w13", "column")):
        w = full[p + name + ".weight_int8"]
        n, k = (w.shape[0], w.shape[1] // world) if kind == "row" else (w.shape[0] // world, w.shape[1])
        parts = [torch.as_tensor(dense(shards[r], p + name, n, k)) for r in range(world)]
        if kind == "row":
            assert torch.equal(torch.cat(parts, dim=1), w)
        else:   # [gate | up]: each rank holds its rows of both halves
            half = w.shape[0] // 2
            for r in range(world):
                lo, hi = r * half // world, (r + 1) * half // world
                assert torch.equal(parts[r], torch.cat([w[lo:hi], w[half + lo:half + hi]]))
    for key in ("attention.attn_sub_norm.weight", "feed_forward.ffn_sub_norm.weight"):
        assert torch.equal(torch.cat([shards[r][p + key] for r in range(world)]), full[p + key])
    assert torch.equal(shards[1]["tok_embeddings.weight"], full["tok_embeddings.weight"])
