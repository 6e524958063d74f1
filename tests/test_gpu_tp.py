"""GPU: the fused kernels of the tensor-parallel path (plain quantiser, scale + sum of squares
quantiser, fp32 partial contraction, finish kernel) against torch on the same inputs, and two
emulated K shards on one GPU against the unsharded layer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def packed_dic(w, key, ws):
    from ternainfer_b200.convert import compress_weight
    cv, tg, tm, bm = compress_weight(w)
    return {key + ".weight_compressed_val": cv, key + ".weight_TileOffsets_global": tg,
            key + ".weight_TileOffsets_median": tm, key + ".weight_bitmap": bm,
            key + ".weight_scale": torch.tensor(ws + [0] * (4 - len(ws))).to(torch.bfloat16)}


def ternary(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    r = torch.rand((n, k), generator=g)
    sign = torch.randint(0, 2, (n, k), generator=g, dtype=torch.int8) * 2 - 1
    return torch.where(r < 0.45, torch.zeros((), dtype=torch.int8), sign)


@pytest.mark.parametrize("M,K", [(1, 2560), (8, 8192), (64, 3584), (200, 28672)])
def test_plain_quant_kernel_bit_exact(lib, M, K):
    from ternainfer_b200 import tp
    from ternainfer_b200.linear import quant_input
    g = torch.Generator(device="cuda").manual_seed(M + K)
    x = (torch.randn((M, K), generator=g, device="cuda") * 3).to(torch.bfloat16)
    x[0, :16] = 0
    q, s = tp._quant_fused(x)
    q_ref, s_ref = quant_input(x)
    assert torch.equal(q, q_ref) and torch.equal(s.reshape(-1), s_ref.reshape(-1))


@pytest.mark.parametrize("M", [1, 8, 32, 64, 100, 300])
def test_partial_f32_bit_exact(lib, M):
    """fp32 partial output = float(acc) / s, on the warp-MMA kernel (M <= 64 here) and the
    tensor-core kernel (above)."""
    from ternainfer_b200 import tp
    from ternainfer_b200.linear import quant_input
    N, K = 2560, 3456 - 3456 % 64
    w = ternary(N, K, 5)
    dic = packed_dic(w, "l", [0.02])
    packed = [dic["l" + s].cuda() for s in (".weight_compressed_val", ".weight_TileOffsets_global",
                                            ".weight_TileOffsets_median", ".weight_bitmap")]
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    xq, s = quant_input(x)
    s = s.reshape(-1).contiguous()
    out = torch.full((M, N), float("nan"), device="cuda")
    cv, tg, tm, bm = packed
    lib.ternaspmm_partial_f32(xq.data_ptr(), bm.data_ptr(), tg.data_ptr(), tm.data_ptr(), cv.data_ptr(),
                              out.data_ptr(), s.data_ptr(), M, N, K, torch.cuda.current_stream().cuda_stream)
    assert lib.ternaspmm_last_status() == 0
    acc = tp._accumulate_i32(xq, packed, N)
    assert torch.equal(acc.cpu(), (xq.cpu().int() @ w.int().t()))
    assert torch.equal(out, acc.float() / s.float()[:, None])


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("M", [4, 64, 160])
def test_row_parallel_fused_matches_torch_formulation(lib, gated, M):
    """One rank (tp = 1): the three-launch GPU path against the torch formulation of the same
    arithmetic.  The int8 values and scales are identical; the sum of squares is added in a
    different order, so the output may differ by one bf16 ulp."""
    from ternainfer_b200 import tp
    N, K = 1024, 2048
    w = ternary(N, K, 9)
    dic = packed_dic(w, "l", [0.03])
    g = torch.Generator(device="cuda").manual_seed(M + gated)
    nw = (1 + 0.1 * torch.randn(K, generator=g, device="cuda")).to(torch.bfloat16)
    layer = tp.RowParallelSpBitLinear(K, N, dic, "l", None, nw, 1e-5, "single", gated=gated)
    x = torch.randn((M, 2 * K if gated else K), generator=g, device="cuda").to(torch.bfloat16)
    res = torch.randn((M, N), generator=g, device="cuda").to(torch.bfloat16)
    a = layer(x, residual=res)
    layer.fused = False
    b = layer(x, residual=res)
    # one ulp of the linear's own output (before the residual add, which can cancel)
    ulp = (torch.maximum(b.float().abs(), (b.float() - res.float()).abs()) * 2.0 ** -6).clamp(min=2.0 ** -9)
    assert ((a.float() - b.float()).abs() <= ulp).all()
    assert (a != b).float().mean().item() < 0.02


def test_two_emulated_k_shards_against_unsharded_layer(lib):
    """Two K shards computed one after the other on one GPU, their buffers added as the
    all-reduce would, then the finish kernel: within bf16 rounding of the unsharded
    RMSNorm -> quantiser -> linear."""
    from ternainfer_b200.linear import SpBitLinear, quant_input
    N, K, M, eps = 1024, 4096, 16, 1e-5
    w = ternary(N, K, 21)
    g = torch.Generator(device="cuda").manual_seed(2)
    nw = (1 + 0.1 * torch.randn(K, generator=g, device="cuda")).to(torch.bfloat16)
    x = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    full = SpBitLinear(K, N, packed_dic(w, "l", [0.03]), "l")
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * nw.float()).to(torch.bfloat16)
    want = full(y).float()

    st = torch.cuda.current_stream().cuda_stream
    total = torch.zeros(M * N + M, device="cuda")
    for r in range(2):
        ks = slice(r * K // 2, (r + 1) * K // 2)
        d = packed_dic(w[:, ks].contiguous(), "l", [0.03])
        cv, tg, tm, bm = [d["l" + s].cuda() for s in (".weight_compressed_val", ".weight_TileOffsets_global",
                                                     ".weight_TileOffsets_median", ".weight_bitmap")]
        xs, ws_ = x[:, ks].contiguous(), nw[ks].contiguous()
        q = torch.empty((M, K // 2), dtype=torch.int8, device="cuda")
        s = torch.empty(M, dtype=torch.bfloat16, device="cuda")
        buf = torch.empty(M * N + M, device="cuda")
        lib.ternaspmm_scale_quant_sumsq(xs.data_ptr(), ws_.data_ptr(), 0, M, K // 2, q.data_ptr(), s.data_ptr(),
                                        buf.data_ptr() + 4 * M * N, st)
        lib.ternaspmm_partial_f32(q.data_ptr(), bm.data_ptr(), tg.data_ptr(), tm.data_ptr(), cv.data_ptr(),
                                  buf.data_ptr(), s.data_ptr(), M, N, K // 2, st)
        total += buf
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    wsb = torch.tensor([0.03]).to(torch.bfloat16).cuda()
    lib.ternaspmm_tp_finish(total.data_ptr(), wsb.data_ptr(), eps, K, M, N, None, out.data_ptr(), st)
    torch.cuda.synchronize()
    assert torch.allclose(total[M * N:], xf.pow(2).sum(-1), rtol=1e-5)
    err = (out.float() - want).abs()
    # quantisation noise of int8 activations: ~0.4 % of the row's output RMS per element
    assert err.max().item() <= 0.05 * want.abs().max().item()
    assert (err.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()).item() < 0.02


def test_allreduce_finish_kernel_with_one_rank(lib):
    """World size 1: the fused tail degenerates to the plain finish kernel (no peer to wait for);
    two calls in a row exercise the run counter."""
    import ctypes as C
    M, N, W = 24, 1024, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    buf = torch.randn(M * N + M, generator=g, device="cuda")
    buf[M * N:] = buf[M * N:].abs() * W
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    counters = torch.zeros(2, dtype=torch.int32, device="cuda")
    ws = torch.tensor([0.03]).to(torch.bfloat16).cuda()
    res = torch.randn((M, N), generator=g, device="cuda").to(torch.bfloat16)
    want = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    got = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    lib.ternaspmm_tp_finish(buf.data_ptr(), ws.data_ptr(), 1e-5, W, M, N, res.data_ptr(), want.data_ptr(), st)
    bufs, flg = (C.c_void_p * 1)(buf.data_ptr()), (C.c_void_p * 1)(flags.data_ptr())
    for call in range(2):
        got.zero_()
        lib.ternaspmm_tp_allreduce_finish(bufs, flg, 0, 1, counters.data_ptr(), ws.data_ptr(), 1e-5, W, M, N,
                                          res.data_ptr(), got.data_ptr(), st)
        torch.cuda.synchronize()
        assert lib.ternaspmm_last_status() == 0
        assert torch.equal(got, want)
        assert counters.tolist() == [call + 1, 0]


def _two_rank_worker(rank, world, port, ok):
    import os
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from ternainfer_b200 import tp
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    K, N, M = 2048, 1024, 40
    g = torch.Generator(device=dev).manual_seed(11)
    w = ternary(N, K, 5)
    nw = (1 + 0.1 * torch.randn(K, generator=g, device=dev)).to(torch.bfloat16)
    x = torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16)
    res = torch.randn((M, N), generator=g, device=dev).to(torch.bfloat16)

    def make(mode):
        dic = {}
        tp.shard_checkpoint_entry(dic, "l", w, torch.tensor([0.03, 0, 0, 0]).to(torch.bfloat16), None, "row", rank, world)
        return tp.RowParallelSpBitLinear(K // world, N, dic, "l", None, tp.shard_vector(nw, rank, world), 1e-5, mode,
                                         max_tokens=M)

    a, b, c = make("single"), make("fused"), make("fused")
    xs = x[:, rank * (K // world):(rank + 1) * (K // world)].contiguous()
    ya = a(xs, residual=res)
    good = True
    for _ in range(3):
        yb, yc = b(xs, residual=res), c(xs, residual=res)
        good = good and torch.equal(ya, yb) and torch.equal(yb, yc)
    torch.cuda.synchronize()
    ok[rank] = int(good and load_ok())
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


def load_ok():
    from ternainfer_b200 import load_library
    return load_library().ternaspmm_last_status() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_collective_matches_nccl_on_two_gpus(lib):
    """Two ranks, one per GPU: the finish kernel with the all-reduce over peer memory gives the same
    bits as the NCCL all-reduce followed by the plain finish kernel, on both of two call sites."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0, 0])
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, 29577, ok)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    for p in procs:
        if p.is_alive():
            p.kill()
    assert list(ok) == [1, 1]
