#!/usr/bin/env python
"""Benchmark of the TernaSpMM hot path on B200.

Headline workload (the linear-layer sweep): the four ternary linears of a
BitNet-b1.58-2B decoder layer - QKV 2560->3840 (3 scale segments), O
2560->2560, gate-up 2560->13824 (2 segments), down 6912->2560 - for
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
On one GPU the line also carries ``list_entry`` (the same step as ONE persistent
launch over a work list), ``by_tokens`` (the same sweep at 1 and 16 tokens),
``ref_kernels_b200`` (the reference's own small-batch CUDA kernels, built for
sm_100a from the reference checkout, timed in the same loop at 8, 16 and 64
tokens next to this library), ``lm_head`` (output head + greedy token),
``prefill`` (the large-batch paths against a bf16 GEMM and against the measured
int8 tensor-core issue rate) and ``decode`` (greedy decode tokens/s of the
30-layer model at batch 1 and 8).  On N > 1 GPUs the sweep runs as
independent replicas (the 2B model's 5 KV heads do not shard) and the line
carries ``tp``: the sharded linear stack of the 8192-wide model with one
collective per row-parallel linear, NCCL and fused.
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

def ncu_traffic(kernel, tokens):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of ``kernel`` at ``tokens`` tokens,
    averaged over the step's launches, from the table that is written next to the ncu summaries
    when a capture is processed (profiles/ncu_traffic.json); None when there is no entry."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        return float(json.load(open(path))[kernel][str(tokens)])
    except Exception:
        return None


def sweep_config(args, world):
    """The workload description both arms print (the driver compares them)."""
    return {"workload": f"bitnet2b_linear_sweep_M{args.tokens}", "tokens": args.tokens, "layers": args.layers,
            "linears_per_step": 4 * args.layers, "p_zero": P_ZERO, "seed": args.seed,
            "l2_policy": "inputs larger than L2: each step streams the distinct compressed weights of all layers "
                         "(410 MB at 30 layers)",
            "parallelism": "replicas only" if world > 1 else "single GPU"}


def cpu_sample(tokens, seconds_budget, seed=1234):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ternaspmm_oracle as o
    import c_oracle
    lib = c_oracle.load()
    lib.oracle_set_num_threads(os.cpu_count() or 1)    # launchers export OMP_NUM_THREADS=1; use the host's cores
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
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    # a step = a bounded sample of the sweep (some passes over one layer); the whole run stays near a minute.
    # The value is what ALL host cores of the box deliver, whatever N is: there is one host.
    one_pass, alg, cores, reps, _ = cpu_sample(args.tokens, max(0.1, 60.0 / max(1, args.steps)))
    for _ in range(args.warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(reps):
            one_pass()
    dt = time.perf_counter() - t0
    val = alg * reps * args.steps / dt / 1e9
    sample = (f"{reps} passes over one layer (4 linears) per step at {args.tokens} tokens, dense ternary int8 weights; "
              "CPU restatement of the reference arithmetic (C, OpenMP) - the reference has no CPU path")
    line = {
        "impl": "reference", "metric": "ternaspmm_algorithmic_GBps", "value": val, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xternary->int32->bf16",
        "data": "synthetic", "config": sweep_config(args, world),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

def build_workload(torch, layers, seed, device):
    """The packed weights of `layers` layers (distinct seeded random ternary matrices)."""
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
                        wbytes=nbytes)
            if layer == 0:
                item["dense"] = w.cpu().numpy()
            work.append(item)
            wbytes_total += nbytes
            del w, r, sign
    return work, wbytes_total


def algorithmic_bytes(it, tokens):
    """Compressed weight + int8 activations + per-token scales + weight scales + bf16 outputs of one call."""
    return it["wbytes"] + tokens * it["K"] + 2 * tokens + 8 + 2 * tokens * it["N"]


class Env:
    """Process-wide state of a GPU run."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA GPU: the TernaSpMM library has no CPU path")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer memory by plain loads/stores only
            dist.init_process_group("nccl", device_id=self.device)
        from ternainfer_b200 import load_library
        self.lib = load_library()   # raises if the CUDA library is missing
        self.stream = torch.cuda.Stream(device=self.device)

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        t = self.torch.tensor([ms], dtype=self.torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def time_replays(self, replay, steps, warmup, min_load_s=0.0):
        """`warmup` untimed replays (plus, with min_load_s, enough further ones to keep the GPU under
        this load for that long, so that the clock sampler sees it), then EXACTLY `steps` timed ones
        between CUDA events on the launching stream, barrier + synchronize on both sides; max over ranks."""
        torch = self.torch
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                replay()
            if min_load_s > 0:
                self.stream.synchronize()
                t0 = time.perf_counter()
                replay()
                self.stream.synchronize()
                one = max(time.perf_counter() - t0, 1e-6)
                extra = min(20000, int(min_load_s / one))
                if self.world > 1:   # the same count on every rank: the replayed graph may hold collectives
                    cnt = torch.tensor([extra], dtype=torch.int64, device=self.device)
                    self.dist.broadcast(cnt, 0)
                    extra = int(cnt.item())
                for _ in range(extra):
                    replay()
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(steps):
                replay()
            e1.record(self.stream)
            self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1))


def quantised_inputs(env, M, seed):
    torch = env.torch
    from ternainfer_b200.linear import quant_input
    gen = torch.Generator(device="cpu").manual_seed(seed + 5)
    x_host = {K: torch.randn((M, K), generator=gen).to(torch.bfloat16).pin_memory() for K in (2560, 6912)}
    xq, s = {}, {}
    for K, xh in x_host.items():
        xq[K], s[K] = quant_input(xh.to(env.device))
        s[K] = s[K].contiguous()
    return xq, s


def check_layer0_against_oracle(env, work, outs, xq, s):
    """Sanity check outside the timed region: the first layer's outputs against the CPU oracle."""
    torch = env.torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ternaspmm_oracle as o
    for it, out in zip(work[:len(SHAPES)], outs[:len(SHAPES)]):
        K = it["K"]
        want = o.ternaspmm(xq[K].cpu().numpy(), it["dense"], s[K].float().cpu().numpy().reshape(-1),
                           it["ws"].float().cpu().numpy(), it["ws_num"])
        got = out.view(torch.int16).cpu().numpy().view(np.uint16)
        if not (got == want).all():
            raise SystemExit(f"bench sanity check failed for {it['name']}: GPU result differs from the oracle")
    if env.lib.ternaspmm_last_status() != 0:
        raise SystemExit("bench: library reported a non-zero status")


def sweep_leg(env, work, M, args, headline):
    """One pass over all linears at M tokens per step, inputs resident in HBM, the step replayed as one
    CUDA graph.  Returns value / ms_per_step / roofline for that token count."""
    torch, lib = env.torch, env.lib
    xq, s = quantised_inputs(env, M, args.seed)
    outs = [torch.empty((M, it["N"]), dtype=torch.bfloat16, device=env.device) for it in work]
    alg_step = sum(algorithmic_bytes(it, M) for it in work)

    def launch_all():
        st = torch.cuda.current_stream().cuda_stream
        for it, out in zip(work, outs):
            K = it["K"]
            lib.bitlinear_TernaSpMM(xq[K].data_ptr(), it["bm"].data_ptr(), it["tg"].data_ptr(), it["tm"].data_ptr(),
                                    it["cv"].data_ptr(), out.data_ptr(), s[K].data_ptr(), it["ws"].data_ptr(),
                                    it["ws_num"], M, it["N"], K, 7, 0, st)

    with torch.cuda.stream(env.stream):
        launch_all()
    env.stream.synchronize()
    check_layer0_against_oracle(env, work, outs, xq, s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(env.stream):
        with torch.cuda.graph(graph, stream=env.stream):
            launch_all()
    ms = env.time_replays(graph.replay, args.steps, args.warmup, min_load_s=1.0 if headline else 0.2)
    peak, peak_kind = measured_peak()
    launches = len(work)
    per_launch_us = ms * 1e3 / (args.steps * launches)
    achieved = (alg_step / launches) / (per_launch_us * 1e-6) / 1e9
    res = {"value": alg_step * env.world * args.steps / (ms * 1e-3) / 1e9, "unit": "GB/s",
           "ms_per_step": ms / args.steps,
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "peak_kind": "of " + peak_kind, "frac_of_nominal_8000": achieved / 8000.0,
                        "kernel": "spmm_small_m_kernel", "avg_launch_us": per_launch_us,
                        "algorithmic_bytes_per_launch": alg_step / launches,
                        "traffic": ncu_traffic("spmm_small_m_kernel", M)},
           "gpu_launches": launches * args.steps}
    return res, (xq, s, alg_step)


def e2e_leg(env, work, M, args, xq, s, alg_step):
    """The same step through the Python call site with HOST buffers: this step's activations come from
    pinned host memory, every output goes back to pinned host memory (on a side stream that forks after
    its producer, so the copies overlap the following linears).  Captured once, exactly as the reference's
    generate.py captures its forward; a step is one replay."""
    torch = env.torch
    from ternainfer_b200.linear import TernaInfer_linear
    xq_host = {K: v.cpu().pin_memory() for K, v in xq.items()}
    s_host = {K: v.cpu().pin_memory() for K, v in s.items()}
    out_host = [torch.empty((M, it["N"]), dtype=torch.bfloat16).pin_memory() for it in work]
    xq_dev = {K: torch.empty_like(v, device=env.device) for K, v in xq_host.items()}
    s_dev = {K: torch.empty_like(v, device=env.device) for K, v in s_host.items()}
    h2d = sum(v.numel() * v.element_size() for v in xq_host.values()) + \
        sum(v.numel() * v.element_size() for v in s_host.values())
    d2h = sum(v.numel() * v.element_size() for v in out_host)
    keep = []
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=env.device)
    with torch.cuda.stream(env.stream):
        with torch.cuda.graph(graph, stream=env.stream):
            for K in xq_host:
                xq_dev[K].copy_(xq_host[K], non_blocking=True)
                s_dev[K].copy_(s_host[K], non_blocking=True)
            for it, oh in zip(work, out_host):
                K = it["K"]
                y = TernaInfer_linear(xq_dev[K], it["cv"], it["tg"], it["tm"], it["bm"], None, s_dev[K],
                                      it["ws"], it["ws_num"], it["N"])
                keep.append(y)
                done = torch.cuda.Event()
                done.record(env.stream)
                side.wait_event(done)
                with torch.cuda.stream(side):
                    oh.copy_(y, non_blocking=True)
            joined = torch.cuda.Event()
            joined.record(side)
            env.stream.wait_event(joined)
    ms = env.time_replays(graph.replay, args.steps, max(3, args.warmup))
    return {"value": alg_step * env.world * args.steps / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms / args.steps,
            "api": "ternainfer_b200.linear.TernaInfer_linear captured in a CUDA graph together with its H2D and "
                   "(side-stream) D2H copies; one replay per step"}


def ref_kernels_leg(env, work, args):
    """The reference's own small-batch CUDA kernels (SpMM + split-K reduction, SPLIT_K = 7 as model.py
    passes it), compiled for sm_100a from the reference checkout into oracle/_ref, next to this library
    in the same loop: one pass over `layers` x 4 linears per step, every call on its own copy of the
    packed weights so that all of them stream from HBM.  The reference supports 8, 16, 32 and 64 tokens."""
    torch = env.torch
    so = os.path.join(ROOT, "oracle", "_ref", "libternaspmm_ref_decode.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/libternaspmm_ref_decode.so not built (needs the reference checkout)"}
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ternaspmm_oracle as o
    ref = ctypes.CDLL(so)
    P, I = ctypes.c_void_p, ctypes.c_int
    ref.ref_bitlinear_TernaSpMM_decode.argtypes = [P] * 8 + [I] * 5 + [P, P]
    ref.ref_bitlinear_TernaSpMM_decode.restype = I

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1).copy()).to(env.device)

    layers = len(work) // len(SHAPES)
    packed = []   # per shape: `layers` device copies of the reference-layout arrays of layer 0's weight
    for it in work[:len(SHAPES)]:
        cv, tg, tm, bm = o.compress_weight_ref(it["dense"])
        cv = np.concatenate([cv, np.zeros(16, np.uint32)])        # the reference kernels prefetch past the ends
        tg = np.concatenate([tg, np.full(8, tg[-1], np.int32)])
        tm = np.concatenate([tm, np.zeros(16, np.uint16)])
        base = [dev(a) for a in (bm, tg, tm, cv)]
        packed.append([base] + [[t.clone() for t in base] for _ in range(layers - 1)])
    out = {"split_k": 7, "layers": layers, "note": "same weights, activations and scales on both sides; ours = "
           "bitlinear_TernaSpMM of this library; reference = mySpMM_Kernel_bitmap_v3 + SplitK_Reduction"}
    for M in (8, 16, 64):
        xq, s = quantised_inputs(env, M, args.seed)
        outs = [torch.empty((M, it["N"]), dtype=torch.bfloat16, device=env.device) for it in work[:len(SHAPES)]]
        wsp = torch.zeros(7 * M * 13824, dtype=torch.int32, device=env.device)

        def launch_ref():
            st = torch.cuda.current_stream().cuda_stream
            for layer in range(layers):
                for si, it in enumerate(work[:len(SHAPES)]):
                    bm, tg, tm, cv = packed[si][layer]
                    K = it["K"]
                    rc = ref.ref_bitlinear_TernaSpMM_decode(xq[K].data_ptr(), bm.data_ptr(), tg.data_ptr(), tm.data_ptr(),
                                                            cv.data_ptr(), outs[si].data_ptr(), s[K].data_ptr(),
                                                            it["ws"].data_ptr(), it["ws_num"], M, it["N"], K, 7,
                                                            wsp.data_ptr(), st)
                    if rc != 0:
                        raise SystemExit(f"reference kernels: CUDA error {rc}")

        ours_outs = [torch.empty((M, it["N"]), dtype=torch.bfloat16, device=env.device) for it in work]

        def launch_ours():
            st = torch.cuda.current_stream().cuda_stream
            for it, o_ in zip(work, ours_outs):
                K = it["K"]
                env.lib.bitlinear_TernaSpMM(xq[K].data_ptr(), it["bm"].data_ptr(), it["tg"].data_ptr(),
                                            it["tm"].data_ptr(), it["cv"].data_ptr(), o_.data_ptr(), s[K].data_ptr(),
                                            it["ws"].data_ptr(), it["ws_num"], M, it["N"], K, 7, 0, st)

        res = {}
        for name, fn in (("reference", launch_ref), ("ours", launch_ours)):
            with torch.cuda.stream(env.stream):
                fn()
            env.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(env.stream):
                with torch.cuda.graph(g, stream=env.stream):
                    fn()
            ms = env.time_replays(g.replay, args.steps, args.warmup)
            res[name + "_ms_per_step"] = ms / args.steps
        # layer 0: both sides must agree bit for bit
        same = all(torch.equal(a, b) for a, b in zip(outs, ours_outs[:len(SHAPES)]))
        alg = sum(algorithmic_bytes(it, M) for it in work)
        res.update({"reference_GBps": alg / (res["reference_ms_per_step"] * 1e-3) / 1e9,
                    "ours_GBps": alg / (res["ours_ms_per_step"] * 1e-3) / 1e9,
                    "speedup": res["reference_ms_per_step"] / res["ours_ms_per_step"], "outputs_identical": bool(same)})
        out[str(M)] = res
        del wsp
    return out


def list_leg(env, work, M, args):
    """The same step through the work-list entry points: all linears of the step in ONE persistent
    launch (ternaspmm_list_run), inputs resident in HBM, replayed as a CUDA graph."""
    torch, lib = env.torch, env.lib
    from ternainfer_b200.lib import ListItem
    xq, s = quantised_inputs(env, M, args.seed)
    outs = [torch.empty((M, it["N"]), dtype=torch.bfloat16, device=env.device) for it in work]
    arr = (ListItem * len(work))()
    for a, it, out in zip(arr, work, outs):
        K = it["K"]
        a.x, a.bitmap, a.tile_offsets, a.quarter_offsets = xq[K].data_ptr(), it["bm"].data_ptr(), it["tg"].data_ptr(), it["tm"].data_ptr()
        a.sign_words, a.out, a.s, a.ws, a.residual = it["cv"].data_ptr(), out.data_ptr(), s[K].data_ptr(), it["ws"].data_ptr(), None
        a.ws_num, a.M, a.N, a.K, a.seg1, a.seg2, a.seg3, a.prefill_form = it["ws_num"], M, it["N"], K, 0, 0, 0, -1
    tb, sb = ctypes.c_longlong(), ctypes.c_longlong()
    entries = lib.ternaspmm_list_plan(arr, len(work), ctypes.byref(tb), ctypes.byref(sb))
    if entries < 0:
        raise SystemExit("bench: the work list was rejected")
    table = torch.empty(tb.value, dtype=torch.uint8, device=env.device)
    scratch = torch.empty(sb.value, dtype=torch.uint8, device=env.device)
    with torch.cuda.stream(env.stream):
        handle = lib.ternaspmm_list_create(arr, len(work), table.data_ptr(), scratch.data_ptr(), env.stream.cuda_stream)
        if not handle:
            raise SystemExit("bench: could not create the work list")
        lib.ternaspmm_list_run(handle, env.stream.cuda_stream)
    env.stream.synchronize()
    check_layer0_against_oracle(env, work, outs, xq, s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(env.stream):
        with torch.cuda.graph(graph, stream=env.stream):
            lib.ternaspmm_list_run(handle, env.stream.cuda_stream)
    ms = env.time_replays(graph.replay, args.steps, args.warmup, min_load_s=0.3)
    if lib.ternaspmm_last_status() != 0:
        raise SystemExit("bench: the work-list run reported a non-zero status")
    lib.ternaspmm_list_destroy(handle)
    alg_step = sum(algorithmic_bytes(it, M) for it in work)
    peak, peak_kind = measured_peak()
    achieved = alg_step * args.steps / (ms * 1e-3) / 1e9
    return {"value": achieved * env.world, "unit": "GB/s", "ms_per_step": ms / args.steps, "items": len(work),
            "entries": entries, "tokens": M,
            "api": "ternaspmm_list_run: one persistent launch per step over all of the step's linears",
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": "of " + peak_kind, "frac_of_nominal_8000": achieved / 8000.0,
                         "kernel": "spmm_list_kernel", "avg_launch_us": ms * 1e3 / args.steps,
                         "avg_item_us": ms * 1e3 / args.steps / len(work), "algorithmic_bytes_per_launch": alg_step,
                         "traffic": ncu_traffic("spmm_list_kernel", M)},
            "gpu_launches": args.steps}


def lm_head_leg(env, args):
    """The output-head kernel alone: logits-free greedy token of M rows over the 128256 x 2560 bf16
    embedding (657 MB, five times the L2: every call streams it from HBM)."""
    torch, lib = env.torch, env.lib
    V, K = 128256, 2560
    g = torch.Generator(device=env.device).manual_seed(args.seed)
    emb = (0.02 * torch.randn((V, K), generator=g, device=env.device)).to(torch.bfloat16)
    scratch = torch.zeros(int(lib.ternaspmm_lm_head_scratch_bytes()), dtype=torch.uint8, device=env.device)
    peak, peak_kind = measured_peak()
    out = {}
    for M in (1, 8):
        h = torch.randn((M, K), generator=g, device=env.device).to(torch.bfloat16)
        toks = torch.empty(M, dtype=torch.int64, device=env.device)

        def run():
            lib.ternaspmm_lm_head_argmax(h.data_ptr(), emb.data_ptr(), M, V, K, None, toks.data_ptr(), 1,
                                         scratch.data_ptr(), torch.cuda.current_stream().cuda_stream)

        with torch.cuda.stream(env.stream):
            run()
        env.stream.synchronize()
        want = torch.nn.functional.linear(h, emb).float()
        picked = want.gather(1, toks.view(-1, 1)).view(-1)
        if not (want.max(dim=1).values - picked <= want.abs().max() * 2.0 ** -6).all():
            raise SystemExit("bench: the head kernel's greedy tokens disagree with the dense product")
        ms = env.time_replays(run, args.steps, args.warmup)
        nbytes = V * K * 2 + M * K * 2 + 8 * M
        gbs = nbytes * args.steps / (ms * 1e-3) / 1e9
        dense_ms = env.time_replays(lambda: torch.nn.functional.linear(h, emb).float().argmax(-1), args.steps, args.warmup)
        out[str(M)] = {"us_per_call": ms * 1e3 / args.steps, "GBps": gbs, "frac": gbs / peak, "peak_kind": "of " + peak_kind,
                       "algorithmic_bytes": nbytes, "torch_bf16_linear_plus_argmax_us": dense_ms * 1e3 / args.steps}
    del emb
    torch.cuda.empty_cache()
    return out


def prefill_leg(env, args, token_counts=(256, 1024, 2048, 4096)):
    """Large-batch calls on the gate-up layer (13824 x 2560, the largest of the sweep): the tcgen05 kernel that
    decodes on chip, the path through the reference-sized workspace (decompress once, then tcgen05 on CTA pairs
    with both operands by TMA; `auto` names the one the library picks by itself) and torch's dense bf16 linear on the de-quantised weight (cuBLAS: the comparator of the reference's own kernel
    test).  One weight, launched back to back: the 7 MB of compressed weight stay in L2, as in that test."""
    torch, lib = env.torch, env.lib
    from ternainfer_b200.convert import compress_weight
    N, K, ws_num = 13824, 2560, 2
    g = torch.Generator(device=env.device).manual_seed(args.seed)
    r = torch.rand((N, K), generator=g, device=env.device)
    sign = torch.randint(0, 2, (N, K), generator=g, device=env.device, dtype=torch.int8) * 2 - 1
    w = torch.where(r < P_ZERO, torch.zeros((), dtype=torch.int8, device=env.device), sign)
    cv, tg, tm, bm = compress_weight(w)
    wd = w.to(torch.bfloat16)
    ws = torch.tensor([0.02, 0.03, 0.0, 0.0]).to(torch.bfloat16).to(env.device)
    work = torch.empty(N * K, dtype=torch.int8, device=env.device)
    peak_tf = None
    try:
        peak_tf = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    rate = float(lib.ternaspmm_debug_int8_mma_rate(6400, torch.cuda.current_stream().cuda_stream)) / 1e12
    out = {"layer": "gate-up 13824x2560", "note": "int8 tensor-core ops 2*M*N*K per call; frac_of_measured_bf16_peak is of "
           "the measured bf16 cuBLAS burst peak, frac_of_int8_issue_rate of the rate at which this GPU issues tcgen05 int8 "
           "MMAs from resident operands (measured here, one CTA per SM)",
           "int8_mma_issue_rate_TOPs": rate}
    for M in token_counts:
        xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=env.device)
        sc = (torch.rand(M, device=env.device) * 50 + 1).to(torch.bfloat16)
        y = torch.empty((M, N), dtype=torch.bfloat16, device=env.device)
        xb = xq.to(torch.bfloat16)

        def call(path):
            lib.bitlinear_TernaSpMM_ws(xq.data_ptr(), bm.data_ptr(), tg.data_ptr(), tm.data_ptr(), cv.data_ptr(), y.data_ptr(),
                                       sc.data_ptr(), ws.data_ptr(), ws_num, M, N, K, None, work.data_ptr(), N * K, path,
                                       torch.cuda.current_stream().cuda_stream)

        t_chip = env.time_replays(lambda: call(1), args.steps, args.warmup) / args.steps * 1e3
        a = y.clone()
        t_ws = env.time_replays(lambda: call(2), args.steps, args.warmup) / args.steps * 1e3
        if not torch.equal(a, y):
            raise SystemExit("bench: the two large-batch paths disagree")
        t_torch = env.time_replays(lambda: torch.nn.functional.linear(xb, wd), args.steps, args.warmup) / args.steps * 1e3
        call(0)
        shape = (ctypes.c_int * 6)()
        lib.ternaspmm_last_launch_shape(shape)
        ops = 2.0 * M * N * K
        best = min(t_chip, t_ws)
        out[str(M)] = {"on_chip_us": t_chip, "workspace_us": t_ws, "auto": "workspace" if shape[0] in (6, 7) else "on_chip",
                       "torch_bf16_linear_us": t_torch,
                       "tensor_TOPs": ops / best / 1e6, "frac_of_measured_bf16_peak": (ops / best / 1e6 / peak_tf) if peak_tf else None,
                       "frac_of_int8_issue_rate": (ops / best / 1e6 / rate) if rate > 0 else None,
                       "speedup_vs_torch_bf16": t_torch / best}
    del w, wd, work
    torch.cuda.empty_cache()
    return out


def run_single_leg(args):
    """--workload list | head | prefill: one leg on its own (short runs for profiling)."""
    env = Env()
    if args.workload == "list":
        work, _ = build_workload(env.torch, args.layers, args.seed + 7919 * env.rank, env.device)
        res = list_leg(env, work, args.tokens, args)
        line = {"metric": "ternaspmm_algorithmic_GBps", "value": res["value"], "unit": "GB/s", "n_gpus": env.world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "int8xternary->int32->bf16", "data": "synthetic",
                "config": dict(sweep_config(args, env.world), entry="ternaspmm_list_run"), "roofline": res["roofline"],
                "gpu_launches": res["gpu_launches"]}
    elif args.workload == "head":
        res = lm_head_leg(env, args)
        line = {"metric": "lm_head_GBps", "value": res["8"]["GBps"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["8"]["us_per_call"] / 1e3, "higher_is_better": True,
                "config": {"workload": "lm_head_argmax_128256x2560_M8"}, "lm_head": res, "gpu_launches": args.steps}
    else:
        res = prefill_leg(env, args, (args.tokens,) if args.tokens > 64 else (2048,))
        key = [k for k in res if k.isdigit()][0]
        line = {"metric": "prefill_int8_TOPs", "value": res[key]["tensor_TOPs"], "unit": "TOP/s", "n_gpus": 1,
                "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
                "config": {"workload": f"gate_up_13824x2560_M{key}"}, "prefill": res, "gpu_launches": 2 * args.steps}
    if env.rank == 0:
        print(json.dumps(line), flush=True)
    _finish(env.world)


def run_gpu_arm(args):
    env = Env()
    torch = env.torch
    M = args.tokens
    work, wbytes_total = build_workload(torch, args.layers, args.seed + 7919 * env.rank, env.device)
    sampler = ClockSampler(env.local_rank)
    if env.rank == 0:
        sampler.start()
    head, (xq, s, alg_step) = sweep_leg(env, work, M, args, headline=True)
    e2e = e2e_leg(env, work, M, args, xq, s, alg_step)
    clocks = sampler.stop() if env.rank == 0 else None

    def guarded(fn, *a):
        """The further legs of a one-GPU run must not cost the headline line: a leg that cannot run here
        (a library of the attention glue missing, memory) is reported as an error object.  A leg that finds
        WRONG results ends the run (SystemExit is not caught)."""
        try:
            return fn(*a)
        except Exception as e:      # noqa: BLE001
            torch.cuda.synchronize()
            return {"error": f"{type(e).__name__}: {e}"[:300]}

    extras = {}
    if not args.headline_only:
        if M <= 16:
            extras["list_entry"] = list_leg(env, work, M, args) if env.world > 1 else guarded(list_leg, env, work, M, args)
        if env.world == 1:
            extras["by_tokens"] = {}
            for m in (1, 16):
                if m != M:
                    def both(m=m):
                        r = sweep_leg(env, work, m, args, headline=False)[0]
                        r["list_entry"] = list_leg(env, work, m, args)
                        return r
                    extras["by_tokens"][str(m)] = guarded(both)
            extras["ref_kernels_b200"] = guarded(ref_kernels_leg, env, work, args)
        del work
        torch.cuda.empty_cache()
        if env.world == 1:
            extras["lm_head"] = guarded(lm_head_leg, env, args)
            extras["prefill"] = guarded(prefill_leg, env, args)
            extras["decode"] = guarded(decode_leg, args)
        else:
            extras["tp"] = {mode: tp_stack(env, args, mode, 64, 4) for mode in ("single", "fused")}

    if env.rank == 0:
        cpu_baseline = None            # timed at N = 1 only (rank 0's host cores)
        if env.world == 1:
            one_pass, cpu_alg, cores, reps, dt = cpu_sample(M, 10.0)
            t0 = time.perf_counter()
            for _ in range(reps):
                one_pass()
            cpu_dt = time.perf_counter() - t0
            cpu_baseline = {"value": cpu_alg * reps / cpu_dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                            "sample": f"{reps} passes over one layer (4 linears) at {M} tokens, dense int8 ternary "
                                      f"weights, {cpu_dt:.1f} s"}
        line = {
            "metric": "ternaspmm_algorithmic_GBps", "value": head["value"], "unit": "GB/s", "n_gpus": env.world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8xternary->int32->bf16", "data": "synthetic",
            "config": sweep_config(args, env.world),
            "launch": "one CUDA graph replay per step", "compressed_weight_bytes_per_rank": wbytes_total,
            "roofline": head["roofline"], "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": head["gpu_launches"], "clocks": clocks,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    _finish(env.world)


# ----------------------------------------------------------------------------
# Tensor-parallel arm (the scaled ternary model): hidden 8192, 64/8 heads,
# ffn 28672, batch 64.  Per layer: QKV and gate-up column-parallel, O and down
# row-parallel with ONE all-reduce each; the attention itself is not part of
# the path and is skipped (its output is a fixed synthetic tensor).  Strong
# scaling: the model is fixed, each rank holds 1/N of every weight.
# ----------------------------------------------------------------------------

def tp_stack(env, args, mode, M, L):
    """`L` layers of the 8192-wide model's four linears at `M` tokens, sharded over all ranks (see the
    comment above).  Returns the timing of one step (all layers) as a dict."""
    torch, dist = env.torch, env.dist
    from ternainfer_b200 import tp
    from ternainfer_b200.convert import compress_weight, compressed_nbytes
    world, rank, device = env.world, env.rank, env.device
    dim, H, Hkv, D, ffn = 8192, 64, 8, 128, 28672
    gen = torch.Generator(device=device)

    def tern(n, k, seed):
        gen.manual_seed(seed)
        r = torch.rand((n, k), generator=gen, device=device)
        sign = torch.randint(0, 2, (n, k), generator=gen, device=device, dtype=torch.int8) * 2 - 1
        return torch.where(r < P_ZERO, torch.zeros((), dtype=torch.int8, device=device), sign)

    layers, wbytes, dense0 = [], 0, {}
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
            ws[:len(segs) if segs else 1] = torch.tensor([0.02, 0.03, 0.025][:len(segs) if segs else 1], device=device)
            dic[name + ".weight_scale"] = ws.to(torch.bfloat16)
            if segs:
                dic[name + ".weight_segments"] = torch.tensor(segs)
            if li == 0 and rank == 0:
                dense0[name] = (w.cpu().numpy(), [dic[name + sfx] for sfx in (".weight_compressed_val", ".weight_TileOffsets_global",
                                                                           ".weight_TileOffsets_median", ".weight_bitmap")],
                                dic[name + ".weight_scale"], segs)
            del w
        ones_d = torch.ones(dim // world, device=device)
        ones_f = torch.ones(ffn // world, device=device)
        layers.append((tp.ColumnParallelSpBitLinear(dim, specs[0][2], dic, "wqkv"),
                       tp.RowParallelSpBitLinear(dim // world, dim, dic, "wo", None, ones_d, 1e-5, mode, max_tokens=M),
                       tp.ColumnParallelSpBitLinear(dim, specs[2][2], dic, "w13"),
                       tp.RowParallelSpBitLinear(ffn // world, dim, dic, "w2", None, ones_f, 1e-5, mode,
                                                 gated=True, max_tokens=M)))
    gen.manual_seed(args.seed)
    x0 = torch.randn((M, dim), generator=gen, device=device).to(torch.bfloat16)
    attn = torch.randn((M, dim // world), generator=gen, device=device).to(torch.bfloat16)
    if world > 1:
        dist.broadcast(x0, 0)

    # Sanity check outside the timed region (rank 0, layer 0): every shard's packed weight and the
    # kernels that multiply it, against the CPU oracle - int32 accumulators of all four linears
    # bit-exact, and the column-parallel QKV (explicit scale segments) bf16-identical.
    if rank == 0:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import ternaspmm_oracle as o
        import c_oracle
        c_oracle.load().oracle_set_num_threads(max(1, (os.cpu_count() or 1) // world))   # torchrun exports OMP_NUM_THREADS=1
        one = np.full(M, 0x3F80, np.uint16)
        for name, (wd, packed, ws, segs) in dense0.items():
            n, k = wd.shape
            xq = torch.randint(-128, 128, (M, k), dtype=torch.int8, device=device)
            got = tp._accumulate_i32(xq, packed, n).cpu().numpy()
            acc, _ = c_oracle.ternaspmm(xq.cpu().numpy(), wd, one, np.full(4, 0x3F80, np.uint16), 1)
            if not (got == acc).all():
                raise SystemExit(f"tp bench sanity check failed: int32 accumulators of {name} differ from the oracle")
        wd, packed, ws, segs = dense0["wqkv"]
        xq, s = tp._quant_fused(x0)
        bounds = [sum(segs[:i + 1]) for i in range(2)]
        got = tp._linear_segments(xq, s, packed, ws, bounds, wd.shape[0]).view(torch.int16).cpu().numpy().view(np.uint16)
        acc = o.gemm_i32(xq.cpu().numpy(), wd) if wd.size < (1 << 26) else \
            c_oracle.ternaspmm(xq.cpu().numpy(), wd, one, np.full(4, 0x3F80, np.uint16), 1)[0]
        g = (np.arange(wd.shape[0]) >= bounds[0]).astype(np.int64) + (np.arange(wd.shape[0]) >= bounds[1])
        v = (acc.astype(np.float32) / s.float().cpu().numpy().reshape(-1, 1)).astype(np.float32) * \
            ws.float().cpu().numpy()[g][None, :]
        if not (got == o.f32_to_bf16_bits(v)).all():
            raise SystemExit("tp bench sanity check failed: sharded QKV output differs from the oracle")
    dense0.clear()
    # rank 0 has just spent seconds on the host-side check: meet here, or the other ranks' first fused
    # calls would wait for it on the device beyond the library's bounded-wait limit
    env.barrier()

    def step():
        x = x0
        for qkv, wo, w13, w2 in layers:
            qkv(x)
            h = wo(attn, residual=x)
            x = w2(w13(h), residual=h)
        return x

    class _Eager:
        def replay(self):
            step()

    with torch.cuda.stream(env.stream):
        for _ in range(2):
            step()
        env.stream.synchronize()
        if args.no_graph:
            graph = _Eager()
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=env.stream):
                y = step()
    ms = env.time_replays(graph.replay, args.steps, args.warmup, min_load_s=0.3)
    tp.check_status()     # a device-side wait that ran out would have poisoned the outputs
    if not torch.isfinite(step().float()).all():
        raise SystemExit("tp bench: non-finite outputs")
    wb = torch.tensor([float(wbytes)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(wb)
    peak, kind = measured_peak()
    val = float(wb.item()) * args.steps / (ms * 1e-3) / 1e9
    res = {"mode": mode, "ms_per_step": ms / args.steps, "layers": L, "tokens": M, "tp": world,
           "compressed_weight_GBps": val, "per_gpu_frac": val / world / peak, "peak_kind": "of " + kind,
           "collective": {"single": "one NCCL all-reduce per row-parallel linear",
                          "fused": "reduce-scatter + all-gather inside the finish kernel over peer memory (plain NVLink "
                                   "loads and stores)",
                          "exact": "three all-reduces per row-parallel linear (bit-exact mode)"}[mode],
           "gpu_launches": (6 if mode == "exact" else 10) * L * args.steps}
    del layers, graph
    torch.cuda.empty_cache()
    return res


def run_tp_arm(args):
    env = Env()
    M = args.tokens if args.tokens != 8 else 64
    L = args.layers if args.layers != 30 else 4
    sampler = ClockSampler(env.local_rank)
    if env.rank == 0:
        sampler.start()
    res = tp_stack(env, args, args.tp_mode, M, L)
    clocks = sampler.stop() if env.rank == 0 else None
    if env.rank == 0:
        peak, kind = measured_peak()
        line = {"metric": "ternaspmm_tp_compressed_weight_GBps", "value": res["compressed_weight_GBps"], "unit": "GB/s",
                "n_gpus": env.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int8xternary->int32->bf16", "data": "synthetic",
                "config": {"workload": f"tp_linear_stack_8192x28672_bs{M}", "layers": L, "tokens": M, "tp": env.world,
                           "row_parallel_mode": args.tp_mode, "collective": res["collective"],
                           "l2_policy": "inputs larger than L2: every step streams all layers' weight shards"},
                "roofline": {"bound": "hbm", "achieved": res["compressed_weight_GBps"] / env.world, "peak": peak,
                             "unit": "GB/s", "frac": res["per_gpu_frac"], "peak_kind": "of " + kind, "traffic": None,
                             "note": "per-GPU compressed-weight bytes per second"},
                "gpu_launches": res["gpu_launches"], "clocks": clocks}
        print(json.dumps(line), flush=True)
    _finish(env.world)


# ----------------------------------------------------------------------------
# End-to-end decode arm: the 30-layer BitNet-2B architecture
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
    torch.set_num_threads(os.cpu_count() or 1)    # launchers export OMP_NUM_THREADS=1; use the host's cores
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


def decode_run(args, bsz, fused, reps):
    """Greedy generation of 128 tokens after a 512-token prompt at batch `bsz`; best of `reps` runs."""
    import torch
    from ternainfer_b200.generate import FastGen, GenArgs, build_random_model
    from ternainfer_b200.model import ModelArgs
    margs = ModelArgs(n_layers=args.layers, fused_glue=fused)
    model, _ = build_random_model(margs, 512 + 128, args.seed)
    gen = FastGen(model, GenArgs(128, bsz, 512, True))
    g = torch.Generator(device="cuda").manual_seed(args.seed + 1)
    prompt = torch.randint(0, margs.vocab_size, (bsz, 512), generator=g, device="cuda")
    gen.generate(prompt)            # captures the graphs
    best, first = None, None
    for _ in range(reps):
        toks, st = gen.generate(prompt)
        first = toks[0, :8].tolist()
        if best is None or st["decode_tokens_per_s"] > best["decode_tokens_per_s"]:
            best = st
    del gen, model
    torch.cuda.empty_cache()
    return best, first


def decode_leg(args):
    """Decode tokens/s of the 30-layer model (prompt 512, 128 generated tokens) at batch 1 and 8, with
    the fused front-ends and with plain torch glue between the linears, plus the PyTorch-CPU decode step."""
    out = {"layers": args.layers, "prompt": 512, "generate": 128,
           "note": "random-init weights give near-tied logits over 128256 words, so the two glue variants (another "
                   "fp32 summation order in RMSNorm, another attention kernel) choose different tokens; with the norm's "
                   "summation order held equal the fused path returns the eager model's logits and tokens exactly "
                   "(tests/test_gpu_model.py, 30 layers, batch 1 and 8)"}
    for bsz in (1, 8):
        entry = {}
        for fused in (True, False):
            st, first = decode_run(args, bsz, fused, 2)
            entry["fused_glue" if fused else "torch_glue"] = {
                "decode_tokens_per_s": st["decode_tokens_per_s"], "prefill_tokens_per_s": st["prefill_tokens_per_s"],
                "first_tokens": first}
        cpu_tps, cores, sample = cpu_decode_sample(bsz, args.layers, seconds_budget=6.0)
        entry["cpu_baseline"] = {"value": cpu_tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        out[f"bs{bsz}"] = entry
    return out


def run_decode_arm(args):
    import torch
    torch.cuda.set_device(0)
    bsz = args.tokens if args.tokens in (1, 8) else 1
    sampler = ClockSampler(0)
    sampler.start()
    best, _ = decode_run(args, bsz, not args.unfused, max(1, args.steps // 10))
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
    ap.add_argument("--workload", default="sweep", choices=["sweep", "tp", "decode", "list", "head", "prefill"])
    ap.add_argument("--unfused", action="store_true", help="decode workload: plain torch glue between the linears")
    ap.add_argument("--tp_mode", default="single", choices=["single", "fused", "exact"])
    ap.add_argument("--no_graph", action="store_true", help="tp workload: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--headline_only", action="store_true",
                    help="sweep workload: only the headline and end-to-end legs (short runs for profiling)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "tp":
        run_tp_arm(args)
    elif args.workload == "decode":
        run_decode_arm(args)
    elif args.workload in ("list", "head", "prefill"):
        run_single_leg(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
