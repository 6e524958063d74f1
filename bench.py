#!/usr/bin/env python
"""Benchmark of the TernaSpMM hot path on B200.

Workload (BASELINE.json configs[1], the linear-layer sweep): the four ternary
linears of a BitNet-b1.58-2B decoder layer - QKV 2560->3840 (3 scale segments),
O 2560->2560, gate-up 2560->13824 (2 segments), down 6912->2560 - for
``--layers`` layers with distinct random weights (30 layers = 410 MB of
compressed weights, more than three times the L2, so every call streams its
weights from HBM) at ``--tokens`` tokens.  One step = one pass over all
4 * layers linears.  Synthetic seeded inputs: weights i.i.d. over {-1,0,+1}
with P(0)=0.45, activations N(0,1) quantised per token to int8.

Prints ONE JSON line.  ``value`` = algorithmic bytes (compressed weights +
activations + scales + bf16 outputs) of all ranks per second with every input
resident in HBM, the step replayed as a CUDA graph; ``e2e`` = the same metric
through the Python call site (``TernaInfer_linear``) with the activations
copied from pinned host memory and the outputs copied back every step.
``--impl reference`` times the CPU restatement of the reference's arithmetic
(the reference has no CPU implementation of this path and its CUDA library
does not build without an un-vendored CUTLASS) on the host cores.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np

SHAPES = [  # name, N, K, ws_num
    ("wqkv", 3840, 2560, 3),
    ("wo", 2560, 2560, 1),
    ("w13", 13824, 2560, 2),
    ("w2", 2560, 6912, 1),
]
P_ZERO = 0.45


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------
# CPU arm: the oracle port timed on the host cores (checker code, used here
# only as the thing to compare against, never on the GPU arm's path).
# ----------------------------------------------------------------------------

# dram__bytes_read.sum + dram__bytes_write.sum per launch of spmm_small_m_kernel from one ncu capture of the
# four layer shapes at full size (profiles/spmm_small_m_bitnet2b_sweep_M8.md: 1.990 + 1.346 + 7.017 + 3.572 MB),
# averaged like the step's launches (each shape once per layer); token count -> bytes.
NCU_DRAM_BYTES_PER_LAUNCH = {8: (1.990e6 + 1.346e6 + 7.017e6 + 3.572e6) / 4}


def cpu_sample(tokens, seconds_budget, seed=1234):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ternaspmm_oracle as o
    import c_oracle
    lib = c_oracle.load()
    cores = int(lib.oracle_num_threads())
    items, alg = [], 0
    for li, (name, N, K, ws_num) in enumerate(SHAPES):
        rng = np.random.default_rng(seed + li)
        w = (rng.random((N, K), dtype=np.float32) >= P_ZERO).astype(np.int8)
        w *= (rng.integers(0, 2, size=(N, K), dtype=np.int8) * 2 - 1)
        xq, s = o.make_activations(tokens, K, seed + 100 + li)
        ws = o.make_ws(ws_num, seed + 200 + li)
        nnz = int(np.count_nonzero(w))
        tiles = N * K // 4096
        wbytes = N * K // 8 + (nnz + 16 * tiles) // 8 + 4 * (tiles + 1) + 6 * tiles   # padding estimated at 16 bits/tile
        alg += wbytes + tokens * K + 2 * tokens + 8 + 2 * tokens * N
        items.append((xq, w, o.f32_to_bf16_bits(s.reshape(-1)), o.f32_to_bf16_bits(ws), ws_num))
    def one_pass():
        for xq, w, sb, wb, ws_num in items:
            c_oracle.ternaspmm(xq, w, sb, wb, ws_num)
    one_pass()
    t0 = time.perf_counter()
    one_pass()
    dt = time.perf_counter() - t0
    reps = max(1, min(2000, int(seconds_budget / max(dt, 1e-6))))
    return one_pass, alg, cores, reps, dt


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # a step = a bounded sample of the sweep (some passes over one layer); the whole run stays near a minute
    one_pass, alg, cores, reps, _ = cpu_sample(args.tokens, max(0.1, 60.0 / max(1, args.steps)))
    for _ in range(args.warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(reps):
            one_pass()
    dt = time.perf_counter() - t0
    val = alg * reps * args.steps / dt / 1e9
    sample = f"{reps} passes over one layer (4 linears) per step at {args.tokens} tokens, dense ternary int8 weights"
    line = {
        "impl": "reference", "metric": "ternaspmm_algorithmic_GBps", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xternary->int32->bf16",
        "data": "synthetic",
        "config": {"workload": f"bitnet2b_linear_sweep_M{args.tokens}", "tokens": args.tokens, "p_zero": P_ZERO,
                   "note": "CPU restatement of the reference arithmetic (C, OpenMP); the reference has no CPU path"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

def build_workload(torch, layers, tokens, seed, device):
    from ternainfer_b200.convert import compress_weight, compressed_nbytes
    gen = torch.Generator(device=device)
    work, wbytes_total = [], 0
    for layer in range(layers):
        for si, (name, N, K, ws_num) in enumerate(SHAPES):
            gen.manual_seed(seed + 1000 * layer + si)
            r = torch.rand((N, K), generator=gen, device=device)
            sign = (torch.randint(0, 2, (N, K), generator=gen, device=device, dtype=torch.int8) * 2 - 1)
            w = torch.where(r < P_ZERO, torch.zeros((), dtype=torch.int8, device=device), sign)
            cv, tg, tm, bm = compress_weight(w)
            nbytes = compressed_nbytes(cv, tg, tm, bm)
            ws = torch.zeros(4, device=device)
            ws[:ws_num] = torch.rand(ws_num, generator=gen, device=device) * 0.04 + 0.01
            item = dict(name=name, N=N, K=K, ws_num=ws_num, cv=cv, tg=tg, tm=tm, bm=bm, ws=ws.to(torch.bfloat16),
                        wbytes=nbytes, alg=nbytes + tokens * K + 2 * tokens + 8 + 2 * tokens * N)
            if layer == 0:
                item["dense"] = w.cpu().numpy()
            work.append(item)
            wbytes_total += nbytes
            del w, r, sign
    return work, wbytes_total


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from ternainfer_b200 import load_library
    from ternainfer_b200.linear import TernaInfer_linear, quant_input

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU: the TernaSpMM library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = load_library()   # raises if the CUDA library is missing
    M = args.tokens

    work, wbytes_total = build_workload(torch, args.layers, M, args.seed + 7919 * rank, device)
    alg_step = sum(it["alg"] for it in work)

    # activations: one bf16 matrix per input width, quantised once (resident leg)
    gen = torch.Generator(device="cpu").manual_seed(args.seed + 5)
    x_host = {K: torch.randn((M, K), generator=gen).to(torch.bfloat16).pin_memory() for K in (2560, 6912)}
    xq, s = {}, {}
    for K, xh in x_host.items():
        xq[K], s[K] = quant_input(xh.to(device))
        s[K] = s[K].contiguous()
    xq_host = {K: v.cpu().pin_memory() for K, v in xq.items()}
    s_host = {K: v.cpu().pin_memory() for K, v in s.items()}
    outs = [torch.empty((M, it["N"]), dtype=torch.bfloat16, device=device) for it in work]
    stream = torch.cuda.Stream(device=device)

    def launch_all():
        st = torch.cuda.current_stream().cuda_stream
        for it, out in zip(work, outs):
            K = it["K"]
            lib.bitlinear_TernaSpMM(xq[K].data_ptr(), it["bm"].data_ptr(), it["tg"].data_ptr(), it["tm"].data_ptr(),
                                    it["cv"].data_ptr(), out.data_ptr(), s[K].data_ptr(), it["ws"].data_ptr(),
                                    it["ws_num"], M, it["N"], K, 7, 0, st)

    # sanity (outside the timed region): layer 0 against the CPU oracle
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ternaspmm_oracle as o
    with torch.cuda.stream(stream):
        launch_all()
    stream.synchronize()
    for it, out in zip(work[:len(SHAPES)], outs[:len(SHAPES)]):
        K = it["K"]
        want = o.ternaspmm(xq[K].cpu().numpy(), it["dense"], s[K].float().cpu().numpy().reshape(-1),
                           it["ws"].float().cpu().numpy(), it["ws_num"])
        got = out.view(torch.int16).cpu().numpy().view(np.uint16)
        if not (got == want).all():
            raise SystemExit(f"bench sanity check failed for {it['name']}: GPU result differs from the oracle")
    if lib.ternaspmm_last_status() != 0:
        raise SystemExit("bench: library reported a non-zero status")

    # resident leg: the whole step as one CUDA graph
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            launch_all()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            graph.replay()
        barrier()
        if rank == 0:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        ev1.record(stream)
        barrier()
    ms = ev0.elapsed_time(ev1)
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())

    # end-to-end leg: Python call site, host buffers in and out every step
    out_host = [torch.empty((M, it["N"]), dtype=torch.bfloat16).pin_memory() for it in work]
    xq_dev = {K: torch.empty_like(v, device=device) for K, v in xq_host.items()}
    s_dev = {K: torch.empty_like(v, device=device) for K, v in s_host.items()}
    h2d = sum(v.numel() * v.element_size() for v in xq_host.values()) + \
        sum(v.numel() * v.element_size() for v in s_host.values())
    d2h = sum(v.numel() * v.element_size() for v in out_host)

    # The calls go through the Python call site (TernaInfer_linear) once, under CUDA-graph capture,
    # exactly as the reference's generate.py captures its forward.  The copies are part of the
    # captured step: this step's activations come from pinned host memory on the main stream, and
    # every output goes back to pinned host memory on a side stream that forks after its producer,
    # so the device-to-host copies overlap the following linears.  A step is one replay.
    e2e_outs = []
    e2e_graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=device)
    with torch.cuda.stream(stream):
        with torch.cuda.graph(e2e_graph, stream=stream):
            for K in xq_host:
                xq_dev[K].copy_(xq_host[K], non_blocking=True)
                s_dev[K].copy_(s_host[K], non_blocking=True)
            for it, oh in zip(work, out_host):
                K = it["K"]
                y = TernaInfer_linear(xq_dev[K], it["cv"], it["tg"], it["tm"], it["bm"], None, s_dev[K],
                                      it["ws"], it["ws_num"], it["N"])
                e2e_outs.append(y)
                done = torch.cuda.Event()
                done.record(stream)
                side.wait_event(done)
                with torch.cuda.stream(side):
                    oh.copy_(y, non_blocking=True)
            joined = torch.cuda.Event()
            joined.record(side)
            stream.wait_event(joined)

    def e2e_step():
        e2e_graph.replay()

    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        e1.record(stream)
        barrier()
    clocks = sampler.stop() if rank == 0 else None
    t2 = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = float(t2.item())

    if rank == 0:
        peak, peak_kind = measured_peak()
        launches = len(work)
        value = alg_step * world * args.steps / (ms_max * 1e-3) / 1e9
        per_launch_us = ms_max * 1e3 / (args.steps * launches)
        achieved = (alg_step / launches) / (per_launch_us * 1e-6) / 1e9
        e2e_val = alg_step * world * args.steps / (e2e_ms * 1e-3) / 1e9
        cpu_baseline = None            # timed at N = 1 only (rank 0's host cores)
        if world == 1:
            one_pass, cpu_alg, cores, reps, dt = cpu_sample(M, 10.0)
            t0 = time.perf_counter()
            for _ in range(reps):
                one_pass()
            cpu_dt = time.perf_counter() - t0
            cpu_baseline = {"value": cpu_alg * reps / cpu_dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                            "sample": f"{reps} passes over one layer (4 linears) at {M} tokens, dense int8 ternary "
                                      f"weights, {cpu_dt:.1f} s"}
        line = {
            "metric": "ternaspmm_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_max / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8xternary->int32->bf16", "data": "synthetic",
            "config": {"workload": f"bitnet2b_linear_sweep_M{M}", "tokens": M, "layers": args.layers,
                       "linears_per_step": launches, "p_zero": P_ZERO, "seed": args.seed,
                       "compressed_weight_bytes_per_rank": wbytes_total,
                       "l2_policy": "inputs larger than L2: each step streams %.0f MB of distinct weights" %
                                    (wbytes_total / 1e6),
                       "parallelism": "replicas only" if world > 1 else "single GPU",
                       "launch": "one CUDA graph replay per step"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": "of " + peak_kind,
                         "frac_of_nominal_8000": achieved / 8000.0,
                         "kernel": "spmm_small_m_kernel", "avg_launch_us": per_launch_us,
                         "algorithmic_bytes_per_launch": alg_step / launches,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(M)},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps, "api": "ternainfer_b200.linear.TernaInfer_linear captured in a CUDA graph together with its H2D and (side-stream) D2H copies; one replay per step"},
            "gpu_launches": launches * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    _finish(world)


# ----------------------------------------------------------------------------
# Tensor-parallel arm (BASELINE config 5 shapes): hidden 8192, 64/8 heads,
# ffn 28672, batch 64.  Per layer: QKV and gate-up column-parallel, O and down
# row-parallel with ONE all-reduce each; the attention itself is not part of
# the path and is skipped (its output is a fixed synthetic tensor).  Strong
# scaling: the model is fixed, each rank holds 1/N of every weight.
# ----------------------------------------------------------------------------

def run_tp_arm(args):
    import torch
    import torch.distributed as dist
    from ternainfer_b200 import load_library, tp
    from ternainfer_b200.convert import compress_weight, compressed_nbytes

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    load_library()
    dim, H, Hkv, D, ffn, M = 8192, 64, 8, 128, 28672, args.tokens if args.tokens != 8 else 64
    L = args.layers if args.layers != 30 else 4
    gen = torch.Generator(device=device)

    def tern(n, k, seed):
        gen.manual_seed(seed)
        r = torch.rand((n, k), generator=gen, device=device)
        sign = torch.randint(0, 2, (n, k), generator=gen, device=device, dtype=torch.int8) * 2 - 1
        return torch.where(r < P_ZERO, torch.zeros((), dtype=torch.int8, device=device), sign)

    layers, wbytes = [], 0
    for li in range(L):
        dic = {}
        specs = [("wqkv", "column", (H + 2 * Hkv) * D // world, dim, [H * D // world, Hkv * D // world, Hkv * D // world]),
                 ("wo", "row", dim, dim // world, None),
                 ("w13", "column", 2 * ffn // world, dim, [ffn // world, ffn // world]),
                 ("w2", "row", dim, ffn // world, None)]
        for si, (name, kind, n, k, segs) in enumerate(specs):
            w = tern(n, k, args.seed + 100003 * rank + 101 * li + si)
            cv, tg, tm, bm = compress_weight(w)
            wbytes += compressed_nbytes(cv, tg, tm, bm)
            dic[name + ".weight_compressed_val"], dic[name + ".weight_TileOffsets_global"] = cv, tg
            dic[name + ".weight_TileOffsets_median"], dic[name + ".weight_bitmap"] = tm, bm
            ws = torch.zeros(4, device=device)
            ws[:len(segs) if segs else 1] = 0.02
            dic[name + ".weight_scale"] = ws.to(torch.bfloat16)
            if segs:
                dic[name + ".weight_segments"] = torch.tensor(segs)
            del w
        ones_d = torch.ones(dim // world, device=device)
        ones_f = torch.ones(ffn // world, device=device)
        layers.append((tp.ColumnParallelSpBitLinear(dim, specs[0][2], dic, "wqkv"),
                       tp.RowParallelSpBitLinear(dim // world, dim, dic, "wo", None, ones_d, 1e-5, args.tp_mode,
                                                 max_tokens=M),
                       tp.ColumnParallelSpBitLinear(dim, specs[2][2], dic, "w13"),
                       tp.RowParallelSpBitLinear(ffn // world, dim, dic, "w2", None, ones_f, 1e-5, args.tp_mode,
                                                 gated=True, max_tokens=M)))
    gen.manual_seed(args.seed)
    x0 = torch.randn((M, dim), generator=gen, device=device).to(torch.bfloat16)
    attn = torch.randn((M, dim // world), generator=gen, device=device).to(torch.bfloat16)
    if world > 1:
        dist.broadcast(x0, 0)

    def step():
        x = x0
        for qkv, wo, w13, w2 in layers:
            qkv(x)
            h = wo(attn, residual=x)
            x = w2(w13(h), residual=h)
        return x

    def log(msg):
        if rank == 0 and args.verbose:
            print("[tp] " + msg, file=sys.stderr, flush=True)

    class _Eager:
        def replay(self):
            step()

    stream = torch.cuda.Stream(device=device)
    with torch.cuda.stream(stream):
        log("weights built; eager warm-up")
        for _ in range(2):
            step()
        stream.synchronize()
        log("eager steps done")
        if args.no_graph:
            graph = _Eager()
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                y = step()
            log("graph captured")
        for _ in range(args.warmup):
            graph.replay()
        log("warm-up replays done")
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    wb = torch.tensor([float(wbytes)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(wb)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        ms = float(t.item())
        peak, kind = measured_peak()
        val = float(wb.item()) * args.steps / (ms * 1e-3) / 1e9
        line = {"metric": "ternaspmm_tp_compressed_weight_GBps", "value": val, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "int8xternary->int32->bf16", "data": "synthetic",
                "config": {"workload": f"tp_linear_stack_8192x28672_bs{M}", "layers": L, "tokens": M, "tp": world,
                           "row_parallel_mode": args.tp_mode,
                           "collective": {"single": "one NCCL all-reduce per row-parallel linear",
                                          "fused": "all-reduce inside the finish kernel over peer memory (plain NVLink loads)",
                                          "exact": "three all-reduces per row-parallel linear (bit-exact mode)"}[args.tp_mode],
                           "l2_policy": "inputs larger than L2: %.0f MB of weights per step over all ranks" % (wb.item() / 1e6)},
                "roofline": {"bound": "hbm", "achieved": val / world, "peak": peak, "unit": "GB/s",
                             "frac": val / world / peak, "peak_kind": "of " + kind, "traffic": None,
                             "note": "per-GPU compressed-weight bytes per second"},
                "gpu_launches": (6 if args.tp_mode == "exact" else 10) * L * args.steps, "clocks": clocks}
        print(json.dumps(line), flush=True)
    _finish(world)


# ----------------------------------------------------------------------------
# End-to-end decode arm (BASELINE config 4): the 30-layer BitNet-2B architecture
# with random-init ternary weights and a dense bf16 tied embedding / head, prompt
# of seeded random ids, greedy generation; value = decode tokens per second.
# ----------------------------------------------------------------------------

def cpu_decode_sample(bsz, layers, seconds_budget=10.0, seed=1234):
    """PyTorch-CPU model path of one decode step, timed on the host cores: one decoder layer of the
    BitNet-2B architecture as the reference's dense comparator computes it (quant_input, F.linear on
    the de-quantised ternary weight, division by the scale; RMSNorm and sub-layer norms, RoPE,
    attention over a 640-token bf16 cache, relu^2 gate) plus the tied output head, all float32
    torch CPU ops.  A step costs `layers` x the layer time + the head time; returns tokens/s."""
    import torch
    import torch.nn.functional as F
    torch.manual_seed(seed)
    dim, H, Hkv, D, ffn, vocab, L = 2560, 20, 5, 128, 6912, 128256, 640
    cores = torch.get_num_threads()

    def tern(n, k):
        r = torch.rand(n, k)
        return torch.where(r < P_ZERO, torch.zeros(()), torch.where(torch.rand(n, k) < 0.5, -torch.ones(()), torch.ones(())))

    wqkv, wo, w13, w2 = tern((H + 2 * Hkv) * D, dim), tern(dim, dim), tern(2 * ffn, dim), tern(dim, ffn)
    head = torch.randn(vocab, dim) * 0.02
    ck, cv = torch.randn(bsz, Hkv, L, D), torch.randn(bsz, Hkv, L, D)
    g = [torch.ones(dim), torch.ones(dim), torch.ones(dim), torch.ones(ffn)]

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w

    def lin(x, w):
        s = 127 / x.abs().max(-1, keepdim=True).values.clamp(min=1e-5)
        return F.linear((x * s).round().clamp(-128, 127), w) / s * 0.02

    def layer(x):
        qkv = lin(norm(x, g[0]), wqkv)
        q = qkv[:, : H * D].view(bsz, 1, H, D).transpose(1, 2)
        k = qkv[:, H * D: (H + Hkv) * D].view(bsz, Hkv, 1, D)
        v = qkv[:, (H + Hkv) * D:].view(bsz, Hkv, 1, D)
        ck[:, :, L - 1: L], cv[:, :, L - 1: L] = k, v
        o = F.scaled_dot_product_attention(q, ck.repeat_interleave(H // Hkv, 1), cv.repeat_interleave(H // Hkv, 1))
        h = x + lin(norm(o.transpose(1, 2).reshape(bsz, H * D), g[1]), wo)
        x13 = lin(norm(h, g[2]), w13)
        inner = torch.relu(x13[:, :ffn]) ** 2 * x13[:, ffn:]
        return h + lin(norm(inner, g[3]), w2)

    x = torch.randn(bsz, dim)
    with torch.inference_mode():
        layer(x), F.linear(x, head)
        t0 = time.perf_counter()
        layer(x)
        one = time.perf_counter() - t0
        reps = max(2, min(200, int(0.7 * seconds_budget / max(one, 1e-6))))
        t0 = time.perf_counter()
        for _ in range(reps):
            x = layer(x)
        t_layer = (time.perf_counter() - t0) / reps
        hreps = max(2, min(50, int(0.3 * seconds_budget / max(one * 4, 1e-6))))
        t0 = time.perf_counter()
        for _ in range(hreps):
            F.linear(x, head)
        t_head = (time.perf_counter() - t0) / hreps
    step = layers * t_layer + t_head
    return bsz / step, cores, f"{reps} passes of one decoder layer and {hreps} of the output head at batch {bsz}, " \
                               f"float32 torch CPU ops; step = {layers} x layer + head"


def run_decode_arm(args):
    import torch
    from ternainfer_b200.generate import FastGen, GenArgs, build_random_model
    from ternainfer_b200.model import ModelArgs
    torch.cuda.set_device(0)
    bsz = args.tokens if args.tokens in (1, 8) else 1
    margs = ModelArgs(n_layers=args.layers, fused_glue=not args.unfused)
    model, _ = build_random_model(margs, 512 + 128, args.seed)
    gen = FastGen(model, GenArgs(128, bsz, 512, True))
    g = torch.Generator(device="cuda").manual_seed(args.seed + 1)
    prompt = torch.randint(0, margs.vocab_size, (bsz, 512), generator=g, device="cuda")
    for _ in range(max(1, args.warmup // 3)):
        gen.generate(prompt)
    sampler = ClockSampler(0)
    sampler.start()
    best = None
    for _ in range(max(1, args.steps // 10)):
        _, st = gen.generate(prompt)
        if best is None or st["decode_tokens_per_s"] > best["decode_tokens_per_s"]:
            best = st
    clocks = sampler.stop()
    line = {"metric": "decode_tokens_per_s", "value": best["decode_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * bsz / best["decode_tokens_per_s"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xternary->int32->bf16",
            "data": "synthetic",
            "config": {"workload": f"bitnet2b_greedy_decode_bs{bsz}", "layers": args.layers, "prompt": 512,
                       "generate": 128, "fused_glue": not args.unfused, "seed": args.seed,
                       "prefill_tokens_per_s": best["prefill_tokens_per_s"]},
            "clocks": clocks}
    cpu_tps, cores, sample = cpu_decode_sample(bsz, args.layers)
    line["cpu_baseline"] = {"value": cpu_tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)


def _finish(world):
    """Leave without tearing NCCL down: destroying a process group while CUDA
    graphs that hold NCCL kernels are alive blocks at exit, so every rank meets
    at a barrier, flushes and exits the process directly."""
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--layers", type=int, default=30)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--workload", default="sweep", choices=["sweep", "tp", "decode"])
    ap.add_argument("--unfused", action="store_true", help="decode workload: plain torch glue between the linears")
    ap.add_argument("--tp_mode", default="single", choices=["single", "fused", "exact"])
    ap.add_argument("--no_graph", action="store_true", help="tp workload: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "tp":
        run_tp_arm(args)
    elif args.workload == "decode":
        run_decode_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
