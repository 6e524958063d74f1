// Dense int8 GEMM on CTA pairs for sm_100a: out = epilogue(W[N][K] x x[M][K]^T) with the dense
// weight matrix that decompress_kernel (dense_prefill.cuh) has written to the workspace.
//
// Second stage of the large-batch path through the reference-sized workspace: it stands where the
// reference runs its CUTLASS 2.x int8 GEMM with the scale epilogue visitor on the decompressed
// weight (kernels/src/TernaSpMM_API.cuh:262-285, kernels/src/GEMM/gemm_scale_ws.h of
// Gu-J/TernaInfer).
//
// Why pairs.  With both operands arriving by TMA the single-CTA kernel (spmm_large_m_kernel<256, dense>)
// is bound by the operand traffic from L2 into the SMs: a 128 x 256 tile needs 48 KB per 128 k, and
// halving the token tile to 128 raises the time in proportion to the bytes (measured).  Two CTAs of a
// cluster, on the two SMs of one TPC, share a 256 x 256 tile with tcgen05.mma.cta_group::2: CTA r
// holds weight rows [128 r, 128 r + 128) and tokens [128 r, 128 r + 128) of the tile in its shared
// memory (32 KB per 128 k) and the accumulators of its 128 weight rows x 256 tokens in its tensor
// memory - two thirds of the bytes per operation.
//
// Roles per CTA (18 warps): warp 0 - one thread issues this CTA's two TMA loads per stage (no
// multicast), completing on the LEADER's (cluster rank 0) full barrier; warp 1 - allocates tensor
// memory (both CTAs), and in the leader one thread issues the MMAs for the pair and commits stage
// releases / accumulator-complete signals to both CTAs; warps 2-17 - epilogue of this CTA's 128
// weight rows, handing the accumulator buffer back to the leader's MMA thread.  Six stages, two
// accumulator buffers of 256 columns.  Every wait is bounded (status 4).
#pragma once
#include "spmm_large_m.cuh"

namespace tsp {

constexpr int kPairNT = 256;                 // tokens per tile (the MMA's N)
constexpr int kPairRows = 256;               // weight rows per tile (the MMA's M over both CTAs)
constexpr int kPairStages = 6;
constexpr int kPairHalf = 128 * kLgKStep;    // bytes of one operand half per stage: 128 rows x 128 k
constexpr int kPairEpiWarps = 16;            // four per 32-lane quarter of tensor memory, a quarter of the token columns each:
                                             // the epilogue of a slice is a chain of latencies, so more warps hide more of it

#ifdef TSP_PAIR_ABLATE   // tuning builds, compile-time: 1 = no epilogue work, 2 = no weight loads, 4 = no activation loads, 8 = no MMAs
#define PAIR_ABLATE(bit) ((TSP_PAIR_ABLATE) & (bit))
#else
#define PAIR_ABLATE(bit) 0
#endif

struct PairSmem {
    static constexpr int threads = (kLgFirstEpi + kPairEpiWarps) * 32;
    static constexpr int bar_full = 0;       // [6]   leader: both CTAs' TMA bytes of a stage have landed
    static constexpr int bar_empty = 48;     // [6]   each CTA: the MMAs have read the stage
    static constexpr int bar_acc_full = 96;  // [2]   each CTA: a tile's accumulators are complete
    static constexpr int bar_acc_empty = 112;   // [2] leader: both CTAs' epilogues have read the buffer
    static constexpr int tmem_slot = 136;
    static constexpr int abort_flag = 140;
    static constexpr int scl = 256;          // float[64] per epilogue warp
    static constexpr int ostage = scl + kPairEpiWarps * (kPairNT / 4) * 4;   // 1 KB per epilogue warp (output staging)
    static constexpr int a = (ostage + kPairEpiWarps * kOutStageBytes + 1023) / 1024 * 1024;
    static constexpr int b = a + kPairStages * kPairHalf;
    static constexpr int rest = b + kPairStages * kPairHalf;
    static constexpr int total = 1024 + rest;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of both CTAs] * B[smem of both CTAs]; M = 256, N and K = 32 from the descriptors
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive (once the MMAs issued so far are complete) on the barrier at this offset in BOTH CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
// 2-D TMA tile load into this CTA's shared memory whose completion bytes go to a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

__global__ void __launch_bounds__(PairSmem::threads, 1)
    spmm_dense_pair_kernel(const SpmmParams p, const __grid_constant__ CUtensorMap tmap_x,
                           const __grid_constant__ CUtensorMap tmap_w) {
    using L = PairSmem;
    constexpr int ST = kPairStages, NT = kPairNT;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t dyn = smem_u32(smem);
    const uint32_t sbase = (dyn + 1023u) & ~1023u;       // the same offset in both CTAs of the pair
    uint8_t* rest = smem + (sbase - dyn);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(rest + L::abort_flag);
    float* s_s = reinterpret_cast<float*>(rest + L::scl);
    auto bar_full = [&](int s) { return sbase + L::bar_full + 8 * s; };
    auto bar_empty = [&](int s) { return sbase + L::bar_empty + 8 * s; };
    auto bar_acc_full = [&](int b) { return sbase + L::bar_acc_full + 8 * b; };
    auto bar_acc_empty = [&](int b) { return sbase + L::bar_acc_empty + 8 * b; };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = p.N, K = p.K, M = p.M;
    const uint32_t crank = cluster_ctarank();            // 0 = leader
    const int pair = (int)blockIdx.x >> 1, npairs = (int)gridDim.x >> 1;
    const int KS = (K + kLgKStep - 1) / kLgKStep;
    const int RB = (N + kPairRows - 1) / kPairRows;      // row block fastest: pairs that run side by side share the activation tile in L2
    const int n_tiles = RB * ((M + NT - 1) / NT);
    const int my_tiles = pair < n_tiles ? (n_tiles - 1 - pair) / npairs + 1 : 0;

    griddep_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < ST; ++s) {
            mbar_init(bar_full(s), 1);       // the leader's loader thread (+ the TMA bytes of both CTAs)
            mbar_init(bar_empty(s), 1);      // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full(b), 1);                   // tcgen05.commit after a tile's last MMA
            mbar_init(bar_acc_empty(b), 2 * kPairEpiWarps);  // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(sbase + L::tmem_slot, 2 * NT);
    tc_fence_before();
    __syncthreads();
    cluster_arrive();                        // the peer's barriers exist before anything is sent to them
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(rest + L::tmem_slot);
    bool ok = true;

    if (warp == 0) {
        // ------------------------------------------------ operand loader (both CTAs)
        if (lane == 0) {
            griddep_wait();   // the dense weights and the activations come from earlier kernels of the stream
            int gs = 0;
            for (int ti = 0; ti < my_tiles && ok; ++ti) {
                const int tile = pair + ti * npairs;
                const int w0 = (tile % RB) * kPairRows + (int)crank * 128;   // this CTA's weight rows
                const int t0 = (tile / RB) * NT + (int)crank * 128;          // this CTA's tokens
                for (int ks = 0; ks < KS; ++ks, ++gs) {
                    const int s = gs % ST, it = gs / ST;
                    if (it > 0) ok = wait_or_abort(bar_empty(s), (it - 1) & 1, abort_flag);
                    if (!ok) break;
                    const uint32_t full = map_to_rank(bar_full(s), 0);
                    if (crank == 0) mbar_arrive_expect_tx(bar_full(s), (PAIR_ABLATE(2) ? 0 : 2 * kPairHalf) + (PAIR_ABLATE(4) ? 0 : 2 * kPairHalf));
                    if (!PAIR_ABLATE(2)) tma_load_2d_pair(sbase + L::a + s * kPairHalf, &tmap_w, ks * kLgKStep, w0, full);
                    if (!PAIR_ABLATE(4)) tma_load_2d_pair(sbase + L::b + s * kPairHalf, &tmap_x, ks * kLgKStep, t0, full);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && crank == 0) {
            // int8 x int8 -> int32, K-major A and B, M = 256 over the pair, N = 256
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(kPairRows >> 4) << 24);
            int gs = 0;
            for (int ti = 0; ti < my_tiles && ok; ++ti) {
                const int buf = ti & 1, use = ti >> 1;
                if (use > 0) {   // both CTAs' epilogues must have drained this accumulator buffer
                    ok = wait_or_abort(bar_acc_empty(buf), (use - 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * NT);
                for (int ks = 0; ks < KS; ++ks, ++gs) {
                    const int s = gs % ST, it = gs / ST;
                    ok = wait_or_abort(bar_full(s), it & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = sbase + L::a + s * kPairHalf, b_addr = sbase + L::b + s * kPairHalf;
#pragma unroll
                    for (int j = 0; j < 4; ++j)   // four K=32 slices inside the 128-byte swizzle row
                        if (!PAIR_ABLATE(8)) umma_i8_pair(d_tmem, umma_desc_sw128(a_addr + 32 * j), umma_desc_sw128(b_addr + 32 * j), idesc,
                                     (ks | j) != 0);
                    umma_commit_pair(bar_empty(s));     // frees the stage in both CTAs
                }
                if (ok) umma_commit_pair(bar_acc_full(buf));   // this tile's accumulators are complete in both CTAs
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue (both CTAs, own 128 weight rows)
        griddep_wait();  // scales, residual and the output buffer may belong to the previous kernel
        const int quarter = warp & 3;          // the tensor-memory lanes a warp may read: 32 * (warp % 4)
        constexpr int CW = NT / (kPairEpiWarps / 4);   // token columns per epilogue warp
        const int cb = ((warp - kLgFirstEpi) >> 2) * CW;
        float* s_w = s_s + (warp - kLgFirstEpi) * CW;
        const uint32_t ostage = sbase + L::ostage + (uint32_t)((warp - kLgFirstEpi) * kOutStageBytes);
        const bool wide = (p.epilogue == EPI_DECODE || p.epilogue == EPI_PREFILL) &&
                          ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.residual)) & 15) == 0;
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int tile = pair + ti * npairs;
            const int rb = tile % RB, t0 = (tile / RB) * NT + cb;
            const int buf = ti & 1, use = ti >> 1;
            const int n = rb * kPairRows + (int)crank * 128 + 32 * quarter + lane;
            const bool n_ok = n < N;
            const bool scaled = p.epilogue == EPI_DECODE || p.epilogue == EPI_PREFILL;
            const int gsel = (scaled && n_ok) ? ws_group(n, p) : -1;
            const float ws_el = gsel >= 0 ? __bfloat162float(p.ws[gsel]) : 0.f;
            const int g0 = __shfl_sync(0xffffffffu, gsel, 0);
            const bool fast = p.epilogue == EPI_PREFILL && __all_sync(0xffffffffu, gsel == g0 || gsel < 0);
            const float ws0 = __shfl_sync(0xffffffffu, ws_el, 0);
            __syncwarp();                          // the previous tile's scales are no longer read
            if (p.epilogue != EPI_RAW_I32)
                for (int i = lane; i < CW; i += 32) {
                    const float sv = (t0 + i < M) ? __bfloat162float(p.s[t0 + i]) : 1.f;
                    s_w[i] = fast ? ((sv != 0.f) ? __fdiv_rn(ws0, sv) : 0.f) : sv;
                }
            __syncwarp();
            if (ok) ok = wait_or_abort(bar_acc_full(buf), use & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);   // the tensor-memory loads below are warp-collective
            if (!ok) break;
            tc_fence_after();
            const int cols = min(CW, M - t0);
#pragma unroll 1
            for (int c0 = 0; c0 < (PAIR_ABLATE(1) ? 0 : cols); c0 += 16) {
                int v[16];
                tmem_ld16(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(buf * NT + cb + c0), v);
                const long long o0 = (long long)(t0 + c0) * N + n;
                const int live = n_ok ? min(16, M - t0 - c0) : 0;   // (n_ok is uniform over the warp: N is a multiple of 64)
                if (wide) {
                    store_slice16_wide(p, v, s_w + c0, o0 - lane, live, fast, ws_el, ostage, lane);
                } else {
                    float sc[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) sc[j] = s_w[c0 + j];
                    store_slice16(p, v, sc, o0, live, fast, ws_el);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(bar_acc_empty(buf), 0));   // the leader may overwrite this buffer
        }
    }
    if (*abort_flag && tid == 0) atomicExch(p.status, ST_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    cluster_arrive();        // neither CTA frees tensor memory or leaves while the other may still signal it
    cluster_wait();
    if (warp == 1) tmem_dealloc_pair(tmem_base, 2 * NT);
}

}  // namespace tsp
