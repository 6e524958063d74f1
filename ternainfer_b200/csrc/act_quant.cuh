// Fused activation front-ends of the ternary linears for sm_100a: the work the
// reference does between two TernaSpMM calls with a chain of small library
// kernels (xformers RMSNorm, the Triton-compiled `quant_input`, `squared_relu`;
// model.py:120-123, 235-243, 277-282, 323-335 of Gu-J/TernaInfer) as ONE kernel
// per linear input:
//   norm_quant       x -> RMSNorm(x) * w -> per-token absmax int8 + scale
//   gated_norm_quant [x1 | x3] -> relu(x1)^2 * x3 -> RMSNorm * w -> int8 + scale
// One CTA per token row; the row is staged once in shared memory as bf16, so
// HBM traffic is one read of the activations and one write of int8 + scale.
// Rounding points follow the eager PyTorch evaluation of the same expressions
// (bf16 after the norm, bf16(1/amax) * 127 for the scale, bf16(x*s) before the
// round-half-even).  The fp32 sum of squares has a FIXED order, so the result is
// reproducible bit for bit by any implementation that follows it: with T
// threads, thread t adds f*f (product rounded, then sum rounded: no fused
// multiply-add) over elements (j*T + t)*8 + 0..7 for j = 0, 1, ...; the 32
// lanes of a warp combine by the xor butterfly 16, 8, 4, 2, 1; warp sums are
// added in warp order.  The RMS factor is 1 / sqrt(ss / K + eps) with IEEE
// division and square root.  T = min(1024, max(64, K/8 rounded up to 32)).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

namespace tsp {

constexpr int kActMaxThreads = 1024;   // one 8-element vector per thread up to K = 8192; longer rows loop

__device__ __forceinline__ float bf16_round_f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float block_reduce(float v, float* scratch, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, v, d);
        v = is_max ? fmaxf(v, o) : v + o;
    }
    __syncthreads();   // scratch may still be read from the previous reduction
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) r = is_max ? fmaxf(r, scratch[i]) : r + scratch[i];
    return r;
}

// MODE 0: y = RMSNorm(v) * w.  MODE 1: y = v * w without the normalisation, and the row's sum
// of squares of v is written to ss_out (tensor-parallel row shards: the RMS factor needs the sum
// over all shards and is applied after the all-reduce).  MODE 2: y = v (plain quantiser).
// MODE 3: y = RMSNorm(v) * w written out as bf16 to `q` (read as bf16 [M][K]), no quantiser: the
// model's final norm in the same fixed summation order.
enum ActMode : int { ACT_RMSNORM = 0, ACT_SCALE_SUMSQ = 1, ACT_PLAIN = 2, ACT_NORM_ONLY = 3 };

// x: [M][ld] bf16 (GATED: the row holds [x1 (K) | x3 (K)], ld = 2K), w: [K] bf16 norm weight,
// q: [M][K] int8, s_out: [M] bf16, ss_out: [M] fp32 (MODE 1).  Dynamic shared memory: K bf16.
template <bool GATED, int MODE>
__global__ void __launch_bounds__(kActMaxThreads) norm_quant_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ w, float eps,
                                                                  int K, int8_t* __restrict__ q,
                                                                  __nv_bfloat16* __restrict__ s_out,
                                                                  float* __restrict__ ss_out) {
    extern __shared__ __align__(16) uint8_t act_smem[];
    __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(act_smem);
    __shared__ float scratch[kActMaxThreads / 32];
    griddep_launch_dependents();
    griddep_wait();   // the activations come from the previous kernel
    const int t = blockIdx.x, tid = threadIdx.x;
    const __nv_bfloat16* xr = x + (size_t)t * (GATED ? 2 * K : K);

    // pass 1: stage the row (after the gate, if any) and its sum of squares
    float ss = 0.f;
    for (int k0 = tid * 8; k0 < K; k0 += blockDim.x * 8) {
        const uint4 a = *reinterpret_cast<const uint4*>(xr + k0);
        const __nv_bfloat16* av = reinterpret_cast<const __nv_bfloat16*>(&a);
        __align__(16) __nv_bfloat16 v[8];
        if (GATED) {
            const uint4 b = *reinterpret_cast<const uint4*>(xr + K + k0);
            const __nv_bfloat16* bv = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float r = fmaxf(__bfloat162float(av[i]), 0.f);
                const float sq = bf16_round_f(r * r);                       // relu(x1) ** 2, bf16
                v[i] = __float2bfloat16_rn(sq * __bfloat162float(bv[i]));   // * x3, bf16
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = av[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float f = __bfloat162float(v[i]);
            ss = __fadd_rn(ss, __fmul_rn(f, f));
        }
        *reinterpret_cast<uint4*>(row + k0) = *reinterpret_cast<const uint4*>(v);
    }
    float rstd = 1.f;
    if (MODE != ACT_PLAIN) {
        ss = block_reduce(ss, scratch, false);
        if (MODE == ACT_RMSNORM || MODE == ACT_NORM_ONLY) rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), eps)));
        if (MODE == ACT_SCALE_SUMSQ && tid == 0) ss_out[t] = ss;
    }

    // pass 2: normalise, apply the weight, round to bf16, absmax
    float amax = 0.f;
    for (int k0 = tid * 8; k0 < K; k0 += blockDim.x * 8) {
        uint4 a = *reinterpret_cast<const uint4*>(row + k0);
        __nv_bfloat16* av = reinterpret_cast<__nv_bfloat16*>(&a);
        if (MODE != ACT_PLAIN) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + k0);
            const __nv_bfloat16* ww = reinterpret_cast<const __nv_bfloat16*>(&wv);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float y = __fmul_rn((MODE == ACT_RMSNORM || MODE == ACT_NORM_ONLY) ? __fmul_rn(__bfloat162float(av[i]), rstd) : __bfloat162float(av[i]),
                                          __bfloat162float(ww[i]));
                av[i] = __float2bfloat16_rn(y);
            }
            if (MODE == ACT_NORM_ONLY) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(q) + (size_t)t * K + k0) = a;
            else *reinterpret_cast<uint4*>(row + k0) = a;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(__bfloat162float(av[i])));
    }
    if (MODE == ACT_NORM_ONLY) return;
    amax = block_reduce(amax, scratch, true);
    amax = bf16_round_f(fmaxf(amax, 1e-5f));
    const float s = bf16_round_f(bf16_round_f(1.0f / amax) * 127.0f);   // 127 / amax as reciprocal * 127, in bf16
    if (tid == 0) s_out[t] = __float2bfloat16_rn(s);

    // pass 3: quantise
    for (int k0 = tid * 16; k0 < K; k0 += blockDim.x * 16) {
        __align__(16) int8_t o[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float p = bf16_round_f(__bfloat162float(row[k0 + i]) * s);
            o[i] = (int8_t)fminf(fmaxf(rintf(p), -128.f), 127.f);
        }
        *reinterpret_cast<uint4*>(q + (size_t)t * K + k0) = *reinterpret_cast<const uint4*>(o);
    }
}

// Tail of a row-parallel linear after the all-reduce: buf holds the summed fp32 partial outputs
// [M][N] followed by the summed per-token sums of squares [M];
// out = bf16(buf[t][n] * rsqrt(ss[t] / full_width + eps) * ws) (+ residual, rounded again).
__global__ void __launch_bounds__(256) tp_finish_kernel(const float* __restrict__ buf, const __nv_bfloat16* ws,
                                                        float eps, int full_width, int M, int N,
                                                        const __nv_bfloat16* residual, __nv_bfloat16* out) {
    griddep_launch_dependents();
    griddep_wait();
    const float w = __bfloat162float(ws[0]);
    const long long total = (long long)M * N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / N);
        const float rstd = rsqrtf(buf[total + t] / (float)full_width + eps);
        __nv_bfloat16 v = __float2bfloat16_rn((buf[i] * rstd) * w);
        if (residual) v = __float2bfloat16_rn(__bfloat162float(residual[i]) + __bfloat162float(v));
        out[i] = v;
    }
}


// ---------------------------------------------------------------------------------------------
// Row-parallel tail with the all-reduce fused in (one process per GPU, peer memory over NVLink),
// as a reduce-scatter followed by an all-gather inside ONE launch per rank.
// Every rank's fp32 partial outputs [M*N] and partial sums of squares [M] sit in a buffer that
// all ranks have mapped (symmetric memory), and so does every rank's bf16 output [M*N].
//   1. block 0 tells every peer "my partials of this call are complete" by a system-scope atomic
//      increment of this rank's counter in the peer's flag array (the partials were written by
//      the previous kernel of the stream, so they are complete when this kernel starts);
//   2. every block waits until all peers' counters in the LOCAL flag array have reached this
//      call's number (runs so far + 1) - a spin bounded by `limit_ns` of the global timer;
//   3. rank r owns the r-th slice of the M*N outputs: its blocks pull that slice of all ranks'
//      partials with plain 16-byte loads (own from local memory, the others over NVLink; no
//      multicast), add them in rank order, apply rsqrt(sum_sq/width + eps) * ws (+ residual) and
//      push the finished bf16 values into EVERY rank's output buffer with plain peer stores.
//      Per rank (T-1)/T * (4 + 2) * M*N bytes cross NVLink instead of (T-1) * 4 * M*N for
//      "every rank pulls everything"; each output element is computed once, so all ranks hold
//      bit-identical activations;
//   4. the last block of the rank to finish signals "my slice has been pushed and I have read
//      your partials" to every peer (second counter set), waits (bounded) for the same signal
//      from all peers and advances the local run counter.  When the kernel ends, this rank's
//      output is complete AND no peer still reads this rank's partial buffer, so the buffers of
//      a call site may be reused by the very next call: no ordering rule is left to the caller.
// When a wait runs out the kernel reports ST_WAIT_TIMEOUT through `status`, fills its own output
// with bf16 NaN (a missed peer shows up downstream instead of as stale data) and returns.
struct TpPeers {
    const float* buf[8];      // partial buffers of ranks 0..world-1 (this rank's own pointer included)
    unsigned int* flag[8];    // flag arrays of ranks 0..world-1: flag[r][j] = "partials ready" calls signalled by
                              // rank j, flag[r][8 + j] = "slice pushed" calls signalled by rank j
    __nv_bfloat16* out[8];    // output buffers of ranks 0..world-1
};

// Bounded wait until *f (system scope) has reached `expected`.
__device__ __forceinline__ bool wait_counter_sys(const volatile unsigned int* f, unsigned int expected,
                                                 unsigned long long limit_ns) {
    const unsigned long long t_start = global_timer_ns();
    for (unsigned int it = 0; it < (1u << 26); ++it) {   // wall-time limit below; the count is a second fence
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if ((int)(v - expected) >= 0) return true;
        if (it > 64) {
            __nanosleep(200);
            if (global_timer_ns() - t_start > limit_ns) return false;
        }
    }
    return false;
}

__global__ void __launch_bounds__(256) tp_allreduce_finish_kernel(const TpPeers peers, int rank, int world,
                                                                  unsigned int* runs, unsigned int* done_blocks,
                                                                  const __nv_bfloat16* ws, float eps, int full_width,
                                                                  int M, int N, const __nv_bfloat16* residual,
                                                                  int* status, unsigned long long limit_ns) {
    __shared__ unsigned int expected_s;
    __shared__ int failed_s;
    __shared__ int last_s;
    griddep_launch_dependents();
    griddep_wait();            // the partials come from the previous kernel of the stream
    const int tid = threadIdx.x;
    if (tid == 0) {
        expected_s = *reinterpret_cast<volatile unsigned int*>(runs) + 1u;
        failed_s = 0;
    }
    if (blockIdx.x == 0 && tid < world && tid != rank) {
        __threadfence_system();
        atomicAdd_system(peers.flag[tid] + rank, 1u);
    }
    __syncthreads();
    const unsigned int expected = expected_s;
    if (tid < world && tid != rank && !wait_counter_sys(peers.flag[rank] + tid, expected, limit_ns)) failed_s = 1;
    __syncthreads();
    const bool failed = failed_s != 0;
    __nv_bfloat16* out = peers.out[rank];
    const long long total = (long long)M * N;          // N is a multiple of 4
    const long long vecs = total >> 2;

    if (!failed) {
        const float w = __bfloat162float(ws[0]);
        const long long v0 = vecs * rank / world, v1 = vecs * (rank + 1) / world;   // this rank's slice
        for (long long vi = v0 + (long long)blockIdx.x * blockDim.x + tid; vi < v1; vi += (long long)gridDim.x * blockDim.x) {
            const long long i = vi << 2;
            const int t = (int)(i / N);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float ss = 0.f;
            for (int r = 0; r < world; ++r) {
                float4 v;
                float q;
                asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                             : "l"(peers.buf[r] + i));
                asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(q) : "l"(peers.buf[r] + total + t));
                acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
                ss += q;
            }
            const float rstd = rsqrtf(ss / (float)full_width + eps);
            const float y[4] = {acc.x, acc.y, acc.z, acc.w};
            __align__(8) __nv_bfloat16 o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[e] = __float2bfloat16_rn((y[e] * rstd) * w);
                if (residual) o[e] = __float2bfloat16_rn(__bfloat162float(residual[i + e]) + __bfloat162float(o[e]));
            }
            const uint2 packed = *reinterpret_cast<const uint2*>(o);
            for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(peers.out[r] + i) = packed;   // all-gather by push
        }
    } else {
        if (tid == 0) atomicExch(status, 4 /* ST_WAIT_TIMEOUT */);
        for (long long vi = (long long)blockIdx.x * blockDim.x + tid; vi < vecs; vi += (long long)gridDim.x * blockDim.x)
            *reinterpret_cast<uint2*>(out + (vi << 2)) = make_uint2(0x7FC07FC0u, 0x7FC07FC0u);
    }

    // the last block of this rank to get here closes the call
    __threadfence_system();    // this thread's pushes are visible system-wide before the block is counted
    __syncthreads();
    if (tid == 0) {
        const unsigned int prev = atomicAdd(done_blocks, 1u);
        last_s = prev == gridDim.x - 1;
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence_system();
    if (tid < world && tid != rank) {
        bool ok = true;
        if (!failed) {
            atomicAdd_system(peers.flag[tid] + 8 + rank, 1u);       // my slice sits in your output; I am done with your partials
            ok = wait_counter_sys(peers.flag[rank] + 8 + tid, expected, limit_ns);
        }
        if (!ok) failed_s = 2;
    }
    __syncthreads();
    if (failed_s == 2) {
        // a peer's slice never arrived: the whole output is suspect
        if (tid == 0) atomicExch(status, 4 /* ST_WAIT_TIMEOUT */);
        for (long long vi = tid; vi < vecs; vi += blockDim.x)
            *reinterpret_cast<uint2*>(out + (vi << 2)) = make_uint2(0x7FC07FC0u, 0x7FC07FC0u);
    }
    if (tid == 0) {
        *done_blocks = 0u;
        *reinterpret_cast<volatile unsigned int*>(runs) = expected;
        __threadfence();
    }
}

}  // namespace tsp
