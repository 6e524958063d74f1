// Output head of the decoder for decode-sized batches on sm_100a: logits of up
// to 8 tokens over the whole vocabulary plus the greedy token, in one launch.
//
// Replaces, for M <= 8 rows, the dense bf16 GEMM `logits = self.output(self.norm(h))`
// over the tied embedding (model.py:367, :385 of Gu-J/TernaInfer; 128256 x 2560
// bf16 = 657 MB per decoded token, more than all ternary layers together) and the
// separate `torch.argmax` of the generation loop (generate.py:283, :305).
//
// HBM-bound: the embedding is read exactly once.  Persistent CTAs, one per SM,
// each owning a contiguous range of 16-row groups of the embedding; the warps of
// a CTA take groups from that range through a shared-memory counter.  A warp
// streams its 16 rows with one 128-bit load per lane and row (lane (g, q) reads 8
// consecutive k of rows g and g+8; k is only a summation index, so the tensor-core
// fragments are filled straight from those registers with the hidden states
// permuted the same way), multiplies with mma.sync m16n8k16 bf16 (tokens are the
// MMA's N = 8) and accumulates in fp32.  The hidden states [8][K] sit in shared
// memory (row stride padded by 64 bytes: conflict-free 128-bit reads).
//
// Outputs: optional fp32 logits [M][V] - by default float(bf16(acc)), the value
// the reference's bf16 linear would return - and the arg-max per token over those
// values (ties: smallest index, as torch.argmax), found in two stages: lane ->
// warp -> CTA in registers / shared memory, then per-CTA candidates in a small
// global scratch area and a reduction by the last CTA to arrive.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

namespace tsp {

constexpr int kHeadWarps = 16;
constexpr int kHeadMaxCtas = 1024;              // scratch holds this many candidate slots
constexpr int kHeadUnroll = 8;                  // k-steps of 32 in flight per warp (16 x 128-bit loads per lane)

struct HeadCandidate {
    float v;
    int idx;
};
// scratch layout: [0] arrival counter (uint32, zero between calls), then kHeadMaxCtas * 8 candidates
constexpr size_t kHeadScratchBytes = 16 + sizeof(HeadCandidate) * 8 * kHeadMaxCtas;

struct HeadParams {
    const __nv_bfloat16* h;      // [M][K]
    const __nv_bfloat16* emb;    // [V][K]
    float* logits;               // [M][V] or null
    long long* argmax;           // [M] or null
    unsigned int* counter;       // scratch: arrival counter
    HeadCandidate* cand;         // scratch: [ctas][8]
    int M, V, K, round_bf16;
};

__device__ __forceinline__ uint4 ldg_stream_128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ bool head_better(float v, int i, float bv, int bi) {
    return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(kHeadWarps * 32, 1) lm_head_kernel(const HeadParams p) {
    extern __shared__ __align__(16) uint8_t head_smem[];
    __shared__ int next_group;
    __shared__ HeadCandidate warp_best[kHeadWarps][8];
    __shared__ int is_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int K = p.K, V = p.V;
    const int hs = K * 2 + 64;                                    // bytes per token row in shared memory
    const int groups = (V + 15) >> 4;
    const int g0 = (int)(((long long)groups * blockIdx.x) / gridDim.x);
    const int g1 = (int)(((long long)groups * (blockIdx.x + 1)) / gridDim.x);

    griddep_launch_dependents();
    if (tid == 0) next_group = g0;
    griddep_wait();                                               // the hidden states come from the previous kernel
    // stage the hidden states (rows beyond M are zero)
    for (int i = tid; i < 8 * (K >> 3); i += blockDim.x) {
        const int t = i / (K >> 3), c = i - t * (K >> 3);
        const uint4 v = t < p.M ? ld_cg_128(p.h + (size_t)t * K + c * 8) : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(head_smem + t * hs + c * 16) = v;
    }
    __syncthreads();

    float best_v[2] = {-INFINITY, -INFINITY};
    int best_i[2] = {0x7FFFFFFF, 0x7FFFFFFF};
    const uint8_t* hrow = head_smem + g * hs + q * 16;

    for (;;) {
        int grp = 0;
        if (lane == 0) grp = atomicAdd(&next_group, 1);
        grp = __shfl_sync(0xffffffffu, grp, 0);
        if (grp >= g1) break;
        const int r0 = grp * 16 + g, r1 = r0 + 8;
        const bool ok0 = r0 < V, ok1 = r1 < V;
        const __nv_bfloat16* e0 = p.emb + (size_t)(ok0 ? r0 : 0) * K + q * 8;
        const __nv_bfloat16* e1 = p.emb + (size_t)(ok1 ? r1 : 0) * K + q * 8;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        int k0 = 0;
        for (; k0 + 32 * kHeadUnroll <= K; k0 += 32 * kHeadUnroll) {
            uint4 a[kHeadUnroll], b[kHeadUnroll];
#pragma unroll
            for (int u = 0; u < kHeadUnroll; ++u) {
                a[u] = ldg_stream_128(e0 + k0 + 32 * u);
                b[u] = ldg_stream_128(e1 + k0 + 32 * u);
            }
#pragma unroll
            for (int u = 0; u < kHeadUnroll; ++u) {
                const uint4 x = *reinterpret_cast<const uint4*>(hrow + (k0 + 32 * u) * 2);
                mma_bf16_16x8x16(acc, a[u].x, b[u].x, a[u].y, b[u].y, x.x, x.y);
                mma_bf16_16x8x16(acc, a[u].z, b[u].z, a[u].w, b[u].w, x.z, x.w);
            }
        }
        for (; k0 < K; k0 += 32) {
            const uint4 a = ldg_stream_128(e0 + k0), b = ldg_stream_128(e1 + k0);
            const uint4 x = *reinterpret_cast<const uint4*>(hrow + k0 * 2);
            mma_bf16_16x8x16(acc, a.x, b.x, a.y, b.y, x.x, x.y);
            mma_bf16_16x8x16(acc, a.z, b.z, a.w, b.w, x.z, x.w);
        }
        // acc[0], acc[1]: row r0, tokens 2q, 2q+1;  acc[2], acc[3]: row r1
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int row = c < 2 ? r0 : r1, tok = 2 * q + (c & 1);
            const bool ok = c < 2 ? ok0 : ok1;
            const float v = p.round_bf16 ? __bfloat162float(__float2bfloat16_rn(acc[c])) : acc[c];
            if (ok && tok < p.M) {
                if (p.logits) p.logits[(size_t)tok * V + row] = v;
                if (head_better(v, row, best_v[c & 1], best_i[c & 1])) best_v[c & 1] = v, best_i[c & 1] = row;
            }
        }
    }
    if (!p.argmax) return;

    // ---- arg-max, stage 1: lanes with the same q (the same two tokens) -> warp -> CTA
#pragma unroll
    for (int d = 4; d < 32; d <<= 1)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v[j], d);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i[j], d);
            if (head_better(ov, oi, best_v[j], best_i[j])) best_v[j] = ov, best_i[j] = oi;
        }
    if (g == 0) {
        warp_best[warp][2 * q] = {best_v[0], best_i[0]};
        warp_best[warp][2 * q + 1] = {best_v[1], best_i[1]};
    }
    __syncthreads();
    if (tid < 8) {
        HeadCandidate b = warp_best[0][tid];
        for (int w = 1; w < kHeadWarps; ++w) {
            const HeadCandidate c = warp_best[w][tid];
            if (head_better(c.v, c.idx, b.v, b.idx)) b = c;
        }
        p.cand[blockIdx.x * 8 + tid] = b;
        __threadfence();
    }
    __syncthreads();
    // ---- stage 2: the last CTA to arrive reduces the per-CTA candidates
    if (tid == 0) {
        const unsigned int prev = atomicAdd(p.counter, 1u);
        is_last = prev == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (warp < 8 && warp < p.M) {
        HeadCandidate b = {-INFINITY, 0x7FFFFFFF};
        for (int c = lane; c < (int)gridDim.x; c += 32) {
            const volatile HeadCandidate* src = p.cand + c * 8 + warp;
            const float v = src->v;
            const int i = src->idx;
            if (head_better(v, i, b.v, b.idx)) b = {v, i};
        }
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b.v, d);
            const int oi = __shfl_xor_sync(0xffffffffu, b.idx, d);
            if (head_better(ov, oi, b.v, b.idx)) b = {ov, oi};
        }
        if (lane == 0) p.argmax[warp] = b.idx == 0x7FFFFFFF ? 0 : b.idx;
    }
    if (tid == 0) *p.counter = 0u;                               // ready for the next call
}

}  // namespace tsp
