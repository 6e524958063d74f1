// Large-batch TernaSpMM kernel for sm_100a: compressed ternary weights are
// decoded on chip straight into the tensor-core operand layout and multiplied
// with tcgen05.mma (int8 x int8 -> int32 accumulators in tensor memory).
//
// One launch replaces the reference's prefill pair - the decompress kernel
// that writes a dense int8 copy of W to a global workspace
// (kernels/src/SpMM/SpMM_Kernel.cuh:165-295 of Gu-J/TernaInfer) followed by the
// CUTLASS 2.x int8 GEMM with the scale epilogue visitor
// (kernels/src/GEMM/gemm_scale_ws.h, epilogue_visitor_scale_ws.h:175-211).
// No dense copy of the weights ever reaches HBM.
//
// Persistent CTAs (one per SM) walk over output tiles of 128 weight rows (the
// MMA's M) x NT tokens (the MMA's N); a tile runs over all of K in pipeline
// steps of 128 k.  Tensor memory holds TWO accumulator buffers of NT columns,
// so the epilogue of tile i overlaps the K loop of tile i+1.  Warp roles:
//   warp 0     activation loader: one thread issues 2-D TMA tile loads of
//              x[NT tokens][128 k] (128-byte swizzle, no multicast).
//   warp 1     one thread issues tcgen05.mma (four K=32 steps per stage) and
//              commits stage releases / the accumulator-full barrier.
//   warps 2-9  epilogue: tcgen05.ld of one 32-lane quarter and one half of
//              the token columns each -> scale -> bf16 (or int32 / fp32)
//              stores, then hand the buffer back.
//   warps 10.. decoders, four per pipeline stage: decoder group g owns stage g
//              and handles every k-step gs with gs % stages == g; each of its
//              warps takes one 64x64 tile of the packed format (row half, k
//              half).  They read bitmaps, offsets and sign words from global
//              memory through a register pipeline that runs ahead across tile
//              boundaries, decode with the same table lookup as the
//              small-batch kernel and store int8 rows of 128 k in the
//              128-byte-swizzled K-major layout.
// All hand-offs are mbarriers; every wait has an iteration limit and a CTA-wide
// abort flag so that a lost signal ends the kernel with a status word.
//
// K split.  A launch with fewer output tiles than half the SMs (narrow layers
// at a few hundred tokens, the K-sharded linears of a big model) would leave
// most of the chip idle while each CTA walks through all of K.  Such launches
// run as thread-block clusters of S = 2, 4 or 8 CTAs per tile: CTA r takes the
// r-th slice of K, and the partial accumulators are reduce-scattered through
// distributed shared memory - every CTA owns NT/S token columns, receives the
// other CTAs' partials for them as 16-byte st.shared::cluster stores into one
// slot per sender of the (by then idle) pipeline stage memory, adds them to
// its own accumulators and runs the epilogue for its columns.  (Remote
// atomics were measured at 1-2 per clock per SM and are not used here.)
#pragma once
#include <cuda.h>

#include "spmm_small_m.cuh"

namespace tsp {

constexpr int kLgEpiWarps = 8;           // two per 32-lane quarter of tensor memory, half of the token columns each
constexpr int kLgFirstEpi = 2;           // warp 0 loads activations, warp 1 issues the MMAs
constexpr int kLgFirstDecoder = kLgFirstEpi + kLgEpiWarps;
constexpr int kLgKStep = 128;            // k per pipeline stage = one 128-byte swizzle row
constexpr int kLgAStage = 128 * 128;     // bytes: 128 rows x 128 k int8
constexpr int kOutStageBytes = 16 * 32 * 2;   // output staging per epilogue warp

// DENSE: the weight operand is a dense int8 matrix W[N][K] in global memory (decompressed beforehand,
// see dense_prefill.cuh) and arrives by TMA like the activations: no decoder warps, no lookup tables.
template <int NT, bool DENSE = false>
struct LargeMSmem {
    static constexpr int stages = (NT > 128 && !DENSE) ? 3 : 4;   // dense: no tables in shared memory, room for a fourth stage
    static constexpr int threads = DENSE ? kLgFirstDecoder * 32 : (kLgFirstDecoder + 4 * stages) * 32;   // four decoder warps per stage
    static constexpr int bars = 0;                         // full_a[4] full_b[4] empty[4] acc_full[2] acc_empty[2]
    static constexpr int tmem_slot = 136;
    static constexpr int abort_flag = 140;
    static constexpr int scl = 256;                        // float s[NT / 2] per epilogue warp
    static constexpr int ostage = scl + kLgEpiWarps * (NT / 2) * 4;   // 1 KB per epilogue warp: a slice of 16 tokens x 32 columns, bf16
    static constexpr int a = (ostage + kLgEpiWarps * kOutStageBytes + 1023) / 1024 * 1024;
    static constexpr int b = a + stages * kLgAStage;
    static constexpr int rest = b + stages * NT * kLgKStep;
    static constexpr int tables = DENSE ? 0 : (NT <= 64 ? 2 : 1);   // the two-table decode where shared memory allows it
    static constexpr int align = DENSE ? 1024 : kLutBytes;          // the stage buffers need 1024 bytes, the tables 32 KB
    static constexpr int total = tables * kLutBytes + align + rest;   // tables first (aligned), the rest behind them
};

// ---- tcgen05 wrappers ------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; int8 operands, int32 accumulators, M=128, N and K=32 from the descriptors
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 2-D TMA tile load, completion in bytes on an mbarrier (no multicast)
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// K-major operand with 128-byte swizzle: rows of 128 bytes, groups of 8 rows
// 1024 bytes apart; descriptor version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Bounded wait for a phase of an mbarrier.  mbarrier.try_wait suspends the thread in hardware for a short,
// system-dependent time and wakes it when the phase completes, so a poll is cheap; after a first burst the
// thread also looks at the CTA's abort flag and sleeps briefly between polls.  The limit is TIME on the
// global timer (the duration of a poll is not specified, so an iteration count alone bounds nothing): when
// it runs out the CTA-wide abort flag is raised, every role leaves its loop and the kernel ends with status 4.
constexpr unsigned long long kLgWaitLimitNs = 2000ull * 1000ull * 1000ull;
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < (1u << 28); ++it) {
        if (mbar_test(bar, parity)) return true;
        if (it >= 32) {
            if (*abort_flag) return false;
            if ((it & 63u) == 32u) {
                const unsigned long long now = global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > kLgWaitLimitNs) break;
            }
            __nanosleep(64);
        }
    }
    *abort_flag = 1;
    return false;
}

// Epilogue of one 16-token slice of one output column: v = the 16 accumulators, sc = the tokens' scales
// (or prefill coefficients ws/s), o0 = index of the first output element, live = tokens to store.
// All loads (residual) are issued before the first store.
__device__ __forceinline__ void store_slice16(const SpmmParams& p, const int (&v)[16], const float (&sc)[16],
                                              long long o0, int live, bool fast, float ws_el) {
    const int N = p.N;
    if (p.epilogue == EPI_RAW_I32) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < live) stg_b32(reinterpret_cast<int*>(p.out) + o0 + (long long)j * N, (uint32_t)v[j]);
    } else if (p.epilogue == EPI_F32_DIV) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < live)
                stg_b32(reinterpret_cast<float*>(p.out) + o0 + (long long)j * N, __float_as_uint(__fdiv_rn(__int2float_rn(v[j]), sc[j])));
    } else {
        __nv_bfloat16 r[16];
#pragma unroll
        for (int j = 0; j < 16; ++j)
            r[j] = fast ? __float2bfloat16_rn(__fmul_rn(__int2float_rn(v[j]), sc[j]))
                        : scale_epilogue(v[j], sc[j], ws_el, p.epilogue);
        if (p.residual) {
            __nv_bfloat16 res[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) res[j] = j < live ? __ushort_as_bfloat16(ldg_b16(p.residual + o0 + (long long)j * N)) : r[j];
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = __float2bfloat16_rn(__bfloat162float(res[j]) + __bfloat162float(r[j]));
        }
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < live) stg_b16(reinterpret_cast<__nv_bfloat16*>(p.out) + o0 + (long long)j * N, __bfloat16_as_ushort(r[j]));
    }
}

// The bf16 epilogues of a 16-token slice with wide stores.  A lane holds 16 tokens of ONE output column,
// but the output is [token][column]: stored straight from registers a warp instruction covers 64 bytes,
// and the store path is bound by the number of such requests (measured: 28 M two-byte stores took longer
// than the whole contraction).  So the warp transposes the slice through 1 KB of shared memory -
// [16 tokens][32 columns] - and stores 16 bytes per lane: two instructions of 8 rows x 64 bytes instead of
// sixteen of one row.  The residual, if any, is read the same way (16 bytes per lane) and added after the
// first rounding, as in add_residual().  `o_row0` = index of (first token, the warp's first column);
// needs a 16-byte aligned output (and residual).
__device__ __forceinline__ void store_slice16_wide(const SpmmParams& p, const int (&v)[16], const float* sc,
                                                   long long o_row0, int live, bool fast, float ws_el, uint32_t stage,
                                                   int lane) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float scj = sc[j];   // the tokens' scales (or prefill coefficients), in shared memory
        const __nv_bfloat16 r = fast ? __float2bfloat16_rn(__fmul_rn(__int2float_rn(v[j]), scj))
                                     : scale_epilogue(v[j], scj, ws_el, p.epilogue);
        sts_b16(stage + (uint32_t)(j * 64 + lane * 2), __bfloat16_as_ushort(r));
    }
    __syncwarp();
    const int part = lane & 3;
    uint4 d[2], res[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = (lane >> 2) + 8 * i;
        d[i] = lds128(stage + (uint32_t)(row * 64 + part * 16));
        if (p.residual && row < live) res[i] = ldg_128(p.residual + o_row0 + (long long)row * p.N + part * 8);
    }
    if (p.residual) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t* dv = reinterpret_cast<uint32_t*>(&d[i]);
            const uint32_t* rv = reinterpret_cast<const uint32_t*>(&res[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(rv[e] << 16) + __uint_as_float(dv[e] << 16);
                const float hi = __uint_as_float(rv[e] & 0xFFFF0000u) + __uint_as_float(dv[e] & 0xFFFF0000u);
                dv[e] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) |
                        ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = (lane >> 2) + 8 * i;
        if (row < live) stg_128(reinterpret_cast<__nv_bfloat16*>(p.out) + o_row0 + (long long)row * p.N + part * 8, d[i]);
    }
    __syncwarp();   // the staging area is free for the next slice
}

template <int NT, bool DENSE = false>
__global__ void __launch_bounds__(LargeMSmem<NT, DENSE>::threads, 1)
    spmm_large_m_kernel(const SpmmParams p, const __grid_constant__ CUtensorMap tmap_x,
                        const __grid_constant__ CUtensorMap tmap_w) {
    using L = LargeMSmem<NT, DENSE>;
    constexpr int ST = L::stages;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t dyn = smem_u32(smem);
    const uint32_t lut_base = (dyn + (uint32_t)L::align - 1u) & ~((uint32_t)L::align - 1u);
    const uint32_t sbase = lut_base + L::tables * kLutBytes;  // the stage buffers are 1024-byte aligned
    uint8_t* rest = smem + (sbase - dyn);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(rest + L::abort_flag);
    float* s_s = reinterpret_cast<float*>(rest + L::scl);
    auto bar_full_a = [&](int s) { return sbase + L::bars + 8 * s; };
    auto bar_full_b = [&](int s) { return sbase + L::bars + 32 + 8 * s; };
    auto bar_empty = [&](int s) { return sbase + L::bars + 64 + 8 * s; };
    auto bar_acc_full = [&](int b) { return sbase + L::bars + 96 + 8 * b; };
    auto bar_acc_empty = [&](int b) { return sbase + L::bars + 112 + 8 * b; };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = p.N, K = p.K, M = p.M;
    const int KT = K >> 6;                 // 64-wide k-tiles of the packed format
    const int KS = (K + kLgKStep - 1) / kLgKStep;   // pipeline steps of 128 k
    // Output tiles of this CTA: blockIdx.x, + gridDim.x, ...; row block fastest, so CTAs that run
    // side by side share the activation tile in L2.
    const int RB = (N + 127) / 128;
    const int n_tiles = RB * ((M + NT - 1) / NT);
    // K split: the S CTAs of a cluster share a tile; CTA `crank` takes k-steps [ks0, ks0 + KSl).
    // Without a split the "cluster" is the CTA itself.
    const int S = p.splits;
    const int cid = (int)blockIdx.x / S, ncl = (int)gridDim.x / S, crank = (int)blockIdx.x - cid * S;
    const int ks0 = (int)(((long long)KS * crank) / S);
    const int KSl = (int)(((long long)KS * (crank + 1)) / S) - ks0;
    const int my_tiles = (cid < n_tiles) ? (n_tiles - 1 - cid) / ncl + 1 : 0;   // exactly 1 when S > 1
    const int G = my_tiles * KSl;          // pipeline steps of this CTA over all its tiles

    phase_mark(0);
    griddep_launch_dependents();

    // ---- set-up
    if (tid == 0) {
        for (int s = 0; s < 4; ++s) {
            mbar_init(bar_full_a(s), DENSE ? 1 : 4);   // the four decoder warps of a stage (dense: the loader thread + TMA bytes)
            mbar_init(bar_full_b(s), 1);   // the loader thread (+ TMA bytes)
            mbar_init(bar_empty(s), 1);    // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full(b), 1);              // tcgen05.commit after a tile's last MMA
            mbar_init(bar_acc_empty(b), kLgEpiWarps);   // the epilogue warps have read the buffer
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    // (the one-copy tables are staged in the first pipeline stage, which is idle until the loop starts)
    uint32_t* lut1 = reinterpret_cast<uint32_t*>(rest + L::a);
    for (int e = tid; e < 256 * L::tables; e += L::threads) lut1[e] = e < 256 ? lut_entry(e) : lut_entry_upper(e - 256);
    __syncthreads();
    for (int i = tid; i < 256 * 8 * L::tables; i += L::threads) sts128(lut_base + i * 16, make_uint4(lut1[i >> 3], lut1[i >> 3], lut1[i >> 3], lut1[i >> 3]));
    if (DENSE) griddep_wait();   // the dense weights were written by the previous kernel of the stream
    if (warp == 1) tmem_alloc(sbase + L::tmem_slot, 2 * NT);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(rest + L::tmem_slot);
    bool ok = true;
    phase_mark(1);

    if (warp == 0) {
        // ------------------------------------------------ activation loader
        if (lane == 0) {
            griddep_wait();  // the activations may come from the previous kernel
            int gs = 0;
            for (int ti = 0; ti < my_tiles && ok; ++ti) {
                const int tile = cid + ti * ncl;
                const int t0 = (tile / RB) * NT;
                for (int ks = ks0; ks < ks0 + KSl; ++ks, ++gs) {
                    const int s = gs % ST, it = gs / ST;
                    if (it > 0) ok = wait_or_abort(bar_empty(s), (it - 1) & 1, abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar_full_b(s), NT * kLgKStep);
                    tma_load_2d(sbase + L::b + s * (NT * kLgKStep), &tmap_x, ks * kLgKStep, t0, bar_full_b(s));
                    if (DENSE) {   // 128 weight rows x 128 k of the dense matrix (rows beyond N read as zero)
                        mbar_arrive_expect_tx(bar_full_a(s), kLgAStage);
                        tma_load_2d(sbase + L::a + s * kLgAStage, &tmap_w, ks * kLgKStep, (tile % RB) * 128, bar_full_a(s));
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // int8 x int8 -> int32, K-major A and B, M = 128, N = NT
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | (8u << 24);
            int gs = 0;
            for (int ti = 0; ti < my_tiles && ok; ++ti) {
                const int buf = ti & 1, use = ti >> 1;
                if (use > 0) {   // the epilogue must have drained this accumulator buffer
                    ok = wait_or_abort(bar_acc_empty(buf), (use - 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * NT);
                for (int ks = 0; ks < KSl; ++ks, ++gs) {
                    const int s = gs % ST, it = gs / ST;
                    ok = wait_or_abort(bar_full_a(s), it & 1, abort_flag) &&
                         wait_or_abort(bar_full_b(s), it & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    if (gs == 0) phase_mark_here(2);
                    const uint32_t a_addr = sbase + L::a + s * kLgAStage, b_addr = sbase + L::b + s * (NT * kLgKStep);
#pragma unroll
                    for (int j = 0; j < 4; ++j)   // four K=32 slices inside the 128-byte swizzle row
                        umma_i8(d_tmem, umma_desc_sw128(a_addr + 32 * j), umma_desc_sw128(b_addr + 32 * j), idesc,
                                (ks | j) != 0);
                    umma_commit(bar_empty(s));     // frees the stage when these MMAs have read it
                }
                if (ok) umma_commit(bar_acc_full(buf));   // this tile's accumulators are complete
            }
            phase_mark_here(3);
        }
    } else if (!DENSE && warp >= kLgFirstDecoder) {
        // ---------------------------------------------------------- decoders
        const int dw = warp - kLgFirstDecoder;
        const int half = dw & 1, kk = (dw >> 1) & 1, grp = dw >> 2;   // grp = the pipeline stage this group owns
        const int g = lane >> 2, q = lane & 3;
        const uint32_t lut_lane = lut_base | (uint32_t)(lane * 4);
        const int steps = G > grp ? (G - grp + ST - 1) / ST : 0;      // this group's pipeline steps grp, grp+ST, ...
        // Register pipeline over those steps (it runs ahead across tile boundaries):
        //   stage A  bitmap words + offsets of the step two ahead
        //   stage B  sign-stream position and the sign words of the next step
        //   stage C  decode the current step and store it
        // so the three dependent global round trips of a tile overlap the decoding of the
        // two tiles before it.  (row block, k-step) of the step whose head is loaded next
        // advance incrementally - no division in the loop.
        int f_ks = grp, f_rb = cid % RB, f_left = my_tiles;
        const int rb_step = ncl % RB;
        bool f_valid;
        auto next_head = [&]() {
            while (f_left > 0 && f_ks >= KSl) {
                f_ks -= KSl, --f_left;
                f_rb += rb_step;
                if (f_rb >= RB) f_rb -= RB;
            }
            const int rt = f_rb * 2 + half, kt = (ks0 + f_ks) * 2 + kk;
            f_valid = f_left > 0 && rt * 64 < N && kt < KT;
            f_ks += ST;
            return load_head(p, (long long)rt * KT + kt, f_valid, lane);
        };
        TileHead h_cur = next_head();
        bool v_cur = f_valid;
        TileHead h_nxt = next_head();
        bool v_nxt = f_valid;
        TileSigns s_cur = load_signs(p, h_cur, v_cur, lane);
        const uint32_t a_stage = sbase + L::a + grp * kLgAStage;
        // row = 64*half + 16*r + 8*h + g (row & 7 == g), 16-byte chunk (4*kk + q) ^ g: 128-byte swizzle
        const uint32_t a_lane = a_stage + (uint32_t)((64 * half + g) * 128) + (((uint32_t)(4 * kk + q) ^ (uint32_t)g) << 4);
        for (int i = 0; i < steps && ok; ++i) {
            const TileHead h_far = next_head();                       // stage A
            const bool v_far = f_valid;
            const TileSigns s_nxt = load_signs(p, h_nxt, v_nxt, lane);   // stage B
            if (i > 0) ok = wait_or_abort(bar_empty(grp), (i - 1) & 1, abort_flag);
            if (!ok) break;
            if (v_cur) {                                              // stage C
                const uint32_t w[4] = {h_cur.bw.x, h_cur.bw.y, h_cur.bw.z, h_cur.bw.w};
                int pos = s_cur.pos;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    uint32_t a[8];
                    const int c = __popc(w[r]);
                    if (L::tables == 2) decode_word2(w[r], __funnelshift_r(s_cur.lo[r], s_cur.hi[r], (uint32_t)pos), c, lut_lane, 0u, a);
                    else decode_word(w[r], __funnelshift_r(s_cur.lo[r], s_cur.hi[r], (uint32_t)pos), lut_lane, a);
                    pos += c;
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        sts128(a_lane + (uint32_t)((16 * r + 8 * h) * 128), make_uint4(a[h], a[2 + h], a[4 + h], a[6 + h]));
                }
            }
            fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full_a(grp));
            h_cur = h_nxt, v_cur = v_nxt, h_nxt = h_far, v_nxt = v_far, s_cur = s_nxt;
        }
    } else {
        // ---------------------------------------------------------- epilogue
        griddep_wait();  // scales, residual and the output buffer may belong to the previous kernel
        const int quarter = warp & 3;          // the tensor-memory lanes a warp may read: 32 * (warp % 4)
        constexpr int CW = NT / 2;             // token columns per epilogue warp
        const int cb = ((warp - kLgFirstEpi) >> 2) * CW;
        float* s_w = s_s + (warp - kLgFirstEpi) * CW;   // this warp's scales (or coefficients) of the tile
        const uint32_t ostage = sbase + L::ostage + (uint32_t)((warp - kLgFirstEpi) * kOutStageBytes);
        const bool wide = (p.epilogue == EPI_DECODE || p.epilogue == EPI_PREFILL) &&
                          ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.residual)) & 15) == 0;
        for (int ti = 0; ti < (S == 1 ? my_tiles : 0); ++ti) {
            const int tile = cid + ti * ncl;
            const int rb = tile % RB, t0 = (tile / RB) * NT + cb;
            const int buf = ti & 1, use = ti >> 1;
            const int n = rb * 128 + 32 * quarter + lane;
            const bool n_ok = n < N;
            const bool scaled = p.epilogue == EPI_DECODE || p.epilogue == EPI_PREFILL;
            const int gsel = (scaled && n_ok) ? ws_group(n, p) : -1;
            const float ws_el = gsel >= 0 ? __bfloat162float(p.ws[gsel]) : 0.f;
            // Prefill form with one scale segment for all 32 rows of the warp (always, under the
            // reference's per-128-column rule): the coefficient ws/s[t] is formed once per token
            // and the per-element work is one multiply.
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
            const int cols = min(CW, M - t0);   // live tokens of this warp's columns
#pragma unroll 1
            for (int c0 = 0; c0 < cols; c0 += 16) {
                // All loads of a 16-token slice (tensor memory, scales, residual) are issued before
                // its first store: the output pointer is generic, so a store in between would order
                // every later load behind it and serialise the slice.
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
            if (lane == 0) mbar_arrive(bar_acc_empty(buf));   // the MMA warp may overwrite this buffer
        }
    }
    if (S > 1) {
        // K split: reduce-scatter of the partial accumulators over the cluster.  Everything else of the
        // CTA is idle by now, so 16 warps take part (the eight epilogue warps and the first eight decoder
        // warps: four per 32-lane quarter of tensor memory); all threads pass the two cluster barriers.
        const bool helper = warp >= kLgFirstEpi && warp < kLgFirstEpi + 16 && my_tiles > 0;
        const int quarter = warp & 3, part = (warp - kLgFirstEpi) >> 2;   // part 0..3 of the columns
        const int row = 32 * quarter + lane;
        const int CWo = NT / S;                            // token columns per owner, a power of two >= 16
        const int lg = 31 - __clz(CWo);
        const int SLOT = CWo * 128 * 4;                    // bytes per sender: [CWo/4 column groups][128 rows][4 columns]
        const int rb = cid % RB, t0 = (cid / RB) * NT;
        const uint32_t buf = sbase + L::a;                 // S-1 slots, one per sending CTA
        const int per = CWo / 4;                           // owned columns finished by this warp (>= 4)
        const int tb = t0 + crank * CWo + part * per;      // its first token
        const int n = rb * 128 + row;
        const bool n_ok = n < N;
        float* s_w = s_s + (warp - kLgFirstEpi) * (NT / 8);
        bool fast = false;
        float ws_el = 0.f;
        if (helper) {
            // step 1: scales (or prefill coefficients ws/s) of the columns this warp will finish, then wait
            // until this CTA's accumulators are complete - its stage memory is idle from then on
            griddep_wait();
            const bool scaled = p.epilogue == EPI_DECODE || p.epilogue == EPI_PREFILL;
            const int gsel = (scaled && n_ok) ? ws_group(n, p) : -1;
            ws_el = gsel >= 0 ? __bfloat162float(p.ws[gsel]) : 0.f;
            const int g0 = __shfl_sync(0xffffffffu, gsel, 0);
            fast = p.epilogue == EPI_PREFILL && __all_sync(0xffffffffu, gsel == g0 || gsel < 0);
            const float ws0 = __shfl_sync(0xffffffffu, ws_el, 0);
            if (p.epilogue != EPI_RAW_I32)
                for (int i = lane; i < per; i += 32) {
                    const float sv = (tb + i < M) ? __bfloat162float(p.s[tb + i]) : 1.f;
                    s_w[i] = fast ? ((sv != 0.f) ? __fdiv_rn(ws0, sv) : 0.f) : sv;
                }
            __syncwarp();
            if (ok) ok = wait_or_abort(bar_acc_full(0), 0, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            if (tid == kLgFirstEpi * 32) phase_mark_here(4);
        }
        __syncwarp();
        cluster_arrive();
        cluster_wait();                                    // every CTA of the cluster is done with its stage memory
        phase_mark(5);
        if (helper && ok) {
            // step 2: send the partial accumulators of foreign columns to their owners, 4 columns per store
            const int live = min(NT, M - t0);
            for (int c0 = part * (NT / 4); c0 < min((part + 1) * (NT / 4), live); c0 += 16) {
                const int owner = c0 >> lg;                // a 16-column slice has one owner
                if (owner == crank) continue;
                int v[16];
                tmem_ld16(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)c0, v);
                const int slot = crank < owner ? crank : crank - 1;
                // a warp's 32 rows of one column group are 512 contiguous bytes
                const uint32_t dst = map_to_rank(buf + (uint32_t)(slot * SLOT + ((((c0 & (CWo - 1)) >> 2) * 128 + row) << 4)),
                                                 (uint32_t)owner);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (c0 + 4 * i < live) st_cluster_v4(dst + 2048 * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            }
        }
        __syncwarp();
        cluster_arrive();
        cluster_wait();                                    // all partials have landed
        phase_mark(6);
        if (helper && ok) {
            // step 3: own accumulators + the S-1 received slots -> epilogue for the owned columns
            for (int cc0 = 0; cc0 < per && tb + cc0 < M; cc0 += 16) {
                const int ncol = min(min(16, per - cc0), M - tb - cc0);
                const int col = part * per + cc0;          // column inside the owned range
                int v[16];
                tmem_ld16(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(crank * CWo + col), v);
                for (int sl = 0; sl < S - 1; ++sl) {
                    const uint32_t src = buf + (uint32_t)(sl * SLOT + (((col >> 2) * 128 + row) << 4));
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (4 * i < ncol) {
                            const uint4 w = lds128(src + 2048 * i);
                            v[4 * i] += (int)w.x, v[4 * i + 1] += (int)w.y, v[4 * i + 2] += (int)w.z, v[4 * i + 3] += (int)w.w;
                        }
                }
#pragma unroll
                for (int h = 0; h < 16; h += 8) {          // two halves: loads of a half before its stores
                    float sc[8];
                    __nv_bfloat16 res[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const bool live = h + j < ncol;
                        sc[j] = (live && p.epilogue != EPI_RAW_I32) ? s_w[cc0 + h + j] : 1.f;
                        res[j] = (live && n_ok && p.residual) ? __ushort_as_bfloat16(ldg_b16(p.residual + (long long)(tb + cc0 + h + j) * N + n))
                                                              : __float2bfloat16_rn(0.f);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (h + j < ncol && n_ok) {
                            const long long o = (long long)(tb + cc0 + h + j) * N + n;
                            if (p.epilogue == EPI_RAW_I32) stg_b32(reinterpret_cast<int*>(p.out) + o, (uint32_t)v[h + j]);
                            else if (p.epilogue == EPI_F32_DIV)
                                stg_b32(reinterpret_cast<float*>(p.out) + o, __float_as_uint(__fdiv_rn(__int2float_rn(v[h + j]), sc[j])));
                            else {
                                __nv_bfloat16 r = fast ? __float2bfloat16_rn(__fmul_rn(__int2float_rn(v[h + j]), sc[j]))
                                                       : scale_epilogue(v[h + j], sc[j], ws_el, p.epilogue);
                                if (p.residual) r = __float2bfloat16_rn(__bfloat162float(res[j]) + __bfloat162float(r));
                                stg_b16(reinterpret_cast<__nv_bfloat16*>(p.out) + o, __bfloat16_as_ushort(r));
                            }
                        }
                    }
                }
            }
        }
    }
    if (tid == kLgFirstEpi * 32) phase_mark_here(7);
    if (*abort_flag && tid == 0) atomicExch(p.status, ST_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    phase_mark(8);
    if (warp == 1) tmem_dealloc(tmem_base, 2 * NT);
}

}  // namespace tsp
