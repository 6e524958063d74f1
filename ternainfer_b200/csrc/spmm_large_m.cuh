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
// CTA tile: 128 weight rows (the MMA's M) x NT tokens (the MMA's N) x all of
// K, 128 k per pipeline stage.  Warp roles:
//   warps 0-15 decoders: two warps share the 64x64 weight tile (row half,
//              k half) of every second k-step, each taking two of the four
//              16-row groups; they read bitmaps,
//              offsets and sign words from global memory, decodes with the
//              same table lookup as the small-batch kernel and stores int8
//              rows of 128 k in the 128-byte-swizzled K-major layout.  After
//              the K loop the same warps are the epilogue (tcgen05.ld ->
//              scale -> bf16 store).
//   warp 16    activation loader: one thread issues 2-D TMA tile loads of
//              x[NT tokens][128 k] (128-byte swizzle, no multicast).
//   warp 17    one thread issues tcgen05.mma (four K=32 steps per stage) and
//              commits stage releases / the final accumulator barrier.
// All hand-offs are mbarriers; every wait has an iteration limit and a CTA-wide
// abort flag so that a lost signal ends the kernel with a status word.
#pragma once
#include <cuda.h>

#include "spmm_small_m.cuh"

namespace tsp {

constexpr int kLgDecoders = 16;          // two warps per 64x64 tile, two k-steps in flight
constexpr int kLgThreads = (kLgDecoders + 2) * 32;
constexpr int kLgKStep = 128;            // k per pipeline stage = one 128-byte swizzle row
constexpr int kLgAStage = 128 * 128;     // bytes: 128 rows x 128 k int8

template <int NT>
struct LargeMSmem {
    static constexpr int stages = NT > 128 ? 3 : 4;
    static constexpr int bars = 0;                         // full_a[4] full_b[4] empty[4] acc : 13 x 8 bytes
    static constexpr int tmem_slot = 112;
    static constexpr int abort_flag = 116;
    static constexpr int scl = 128;                        // float s[NT]
    static constexpr int lut1 = scl + NT * 4;              // the 256 table entries, one copy
    static constexpr int a = (lut1 + 1024 + 1023) / 1024 * 1024;
    static constexpr int b = a + stages * kLgAStage;
    static constexpr int rest = b + stages * NT * kLgKStep;
    static constexpr int total = 2 * kLutBytes + rest;     // table aligned to 32 KB, the rest behind it
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

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        if (mbar_test(bar, parity)) return true;
        if (it > 32) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    *abort_flag = 1;
    return false;
}

template <int NT>
__global__ void __launch_bounds__(kLgThreads, 1)
    spmm_large_m_kernel(const SpmmParams p, const __grid_constant__ CUtensorMap tmap_x) {
    using L = LargeMSmem<NT>;
    constexpr int ST = L::stages;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t dyn = smem_u32(smem);
    const uint32_t lut_base = (dyn + (uint32_t)kLutBytes - 1u) & ~((uint32_t)kLutBytes - 1u);
    const uint32_t sbase = lut_base + kLutBytes;  // 32 KB aligned, so the stage buffers are 1024-byte aligned
    uint8_t* rest = smem + (sbase - dyn);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(rest + L::abort_flag);
    float* s_s = reinterpret_cast<float*>(rest + L::scl);
    auto bar_full_a = [&](int s) { return sbase + L::bars + 8 * s; };
    auto bar_full_b = [&](int s) { return sbase + L::bars + 32 + 8 * s; };
    auto bar_empty = [&](int s) { return sbase + L::bars + 64 + 8 * s; };
    const uint32_t bar_acc = sbase + L::bars + 96;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rb = blockIdx.x, t0 = blockIdx.y * NT;
    const int N = p.N, K = p.K, M = p.M;
    const int KT = K >> 6;                 // 64-wide k-tiles of the packed format
    const int KS = (K + kLgKStep - 1) / kLgKStep;   // pipeline steps of 128 k

    griddep_launch_dependents();

    // ---- set-up
    if (tid == 0) {
        for (int s = 0; s < 4; ++s) {
            mbar_init(bar_full_a(s), 8);   // the eight decoder warps of a stage
            mbar_init(bar_full_b(s), 1);   // the loader thread (+ TMA bytes)
            mbar_init(bar_empty(s), 1);    // tcgen05.commit
        }
        mbar_init(bar_acc, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    for (int e = tid; e < 256; e += kLgThreads) reinterpret_cast<uint32_t*>(rest + L::lut1)[e] = lut_entry(e);
    __syncthreads();
    for (int i = tid; i < 256 * 8; i += kLgThreads) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(rest + L::lut1)[i >> 3];
        sts128(lut_base + i * 16, make_uint4(v, v, v, v));
    }
    if (warp == kLgDecoders + 1) tmem_alloc(sbase + L::tmem_slot, NT);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(rest + L::tmem_slot);
    bool ok = true;

    if (warp == kLgDecoders) {
        // ------------------------------------------------ activation loader
        if (lane == 0) {
            griddep_wait();  // the activations may come from the previous kernel
            for (int ks = 0; ks < KS && ok; ++ks) {
                const int s = ks % ST, it = ks / ST;
                if (it > 0) ok = wait_or_abort(bar_empty(s), (it - 1) & 1, abort_flag);
                if (!ok) break;
                mbar_arrive_expect_tx(bar_full_b(s), NT * kLgKStep);
                tma_load_2d(sbase + L::b + s * (NT * kLgKStep), &tmap_x, ks * kLgKStep, t0, bar_full_b(s));
            }
        }
    } else if (warp == kLgDecoders + 1) {
        // ------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // int8 x int8 -> int32, K-major A and B, M = 128, N = NT
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | (8u << 24);
            for (int ks = 0; ks < KS && ok; ++ks) {
                const int s = ks % ST, it = ks / ST;
                ok = wait_or_abort(bar_full_a(s), it & 1, abort_flag) && wait_or_abort(bar_full_b(s), it & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = sbase + L::a + s * kLgAStage, b_addr = sbase + L::b + s * (NT * kLgKStep);
#pragma unroll
                for (int j = 0; j < 4; ++j)   // four K=32 slices inside the 128-byte swizzle row
                    umma_i8(tmem_base, umma_desc_sw128(a_addr + 32 * j), umma_desc_sw128(b_addr + 32 * j), idesc,
                            (ks | j) != 0);
                umma_commit(bar_empty(s));     // frees the stage when these MMAs have read it
            }
            umma_commit(bar_acc);              // accumulators complete
        }
    } else {
        // ---------------------------------------------------------- decoders
        const int sub = warp & 1, half = (warp >> 1) & 1, kk = (warp >> 2) & 1, grp = warp >> 3;
        const int g = lane >> 2, q = lane & 3;
        const int rt = rb * 2 + half;
        const bool have_rows = rt * 64 < N;
        const uint32_t lut_lane = lut_base | (uint32_t)(lane * 4);
        // Register pipeline over this warp's tiles (k-steps grp, grp+2, ...):
        //   stage A  bitmap words + offsets of the tile two steps ahead
        //   stage B  sign-stream position and the eight sign words of the next tile
        //   stage C  decode the current tile and store it
        // so the three dependent global round trips of a tile overlap the
        // decoding of the two tiles before it.
        struct Head { uint4 bw; int toff, qbase; bool valid; };
        struct Signs { uint32_t lo[2], hi[2], sh[2]; };   // this warp's two bitmap words: 2*sub, 2*sub+1
        auto load_head = [&](int ks) {
            Head h;
            const int kt = ks * 2 + kk;
            h.valid = have_rows && ks < KS && kt < KT;
            h.bw = make_uint4(0, 0, 0, 0), h.toff = 0, h.qbase = 0;
            if (h.valid) {
                const long long T = (long long)rt * KT + kt;
                h.bw = __ldg(reinterpret_cast<const uint4*>(p.bitmap + T * 128) + lane);
                h.toff = __ldg(p.tile_off + T);
                const int qd = lane >> 3;
                h.qbase = qd ? (int)__ldg(p.quarter_off + 3 * T + qd - 1) : 0;
            }
            return h;
        };
        auto load_signs = [&](const Head& h) {
            Signs sg;
            const uint32_t w[4] = {h.bw.x, h.bw.y, h.bw.z, h.bw.w};
            int cnt[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) cnt[r] = __popc(w[r]);
            const int tot = cnt[0] + cnt[1] + cnt[2] + cnt[3];
            int incl = tot;
#pragma unroll
            for (int d = 1; d < 8; d <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, d, 8);
                if ((lane & 7) >= d) incl += t;
            }
            long long pos = (long long)h.toff + h.qbase + incl - tot + (sub ? cnt[0] + cnt[1] : 0);
            const int mine[2] = {sub ? cnt[2] : cnt[0], sub ? cnt[3] : cnt[1]};
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint32_t* sw = p.signs + (pos >> 5);
                sg.lo[r] = h.valid ? __ldg(sw) : 0u;
                sg.hi[r] = h.valid ? __ldg(sw + 1) : 0u;
                sg.sh[r] = (uint32_t)pos & 31u;
                pos += mine[r];
            }
            return sg;
        };
        Head h_cur = load_head(grp), h_nxt = load_head(grp + 2);
        Signs s_cur = load_signs(h_cur);
        for (int ks = grp; ks < KS && ok; ks += 2) {
            const int s = ks % ST, it = ks / ST;
            const Head h_far = load_head(ks + 4);      // stage A
            const Signs s_nxt = load_signs(h_nxt);     // stage B
            if (it > 0) ok = wait_or_abort(bar_empty(s), (it - 1) & 1, abort_flag);
            if (!ok) break;
            if (h_cur.valid) {                         // stage C
                const uint32_t w[2] = {sub ? h_cur.bw.z : h_cur.bw.x, sub ? h_cur.bw.w : h_cur.bw.y};
                const uint32_t a_stage = sbase + L::a + s * kLgAStage;
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int r = 2 * sub + rr;
                    uint32_t a[8];
                    decode_word(w[rr], __funnelshift_r(s_cur.lo[rr], s_cur.hi[rr], s_cur.sh[rr]), lut_lane, a);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = 64 * half + 16 * r + 8 * h + g;          // row & 7 == g
                        const uint32_t chunk = (uint32_t)((4 * kk + q) ^ g);     // 128-byte swizzle
                        sts128(a_stage + row * 128 + chunk * 16, make_uint4(a[h], a[2 + h], a[4 + h], a[6 + h]));
                    }
                }
            }
            fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full_a(s));
            h_cur = h_nxt, h_nxt = h_far, s_cur = s_nxt;
        }

        // ---------------------------------------------------------- epilogue
        griddep_wait();  // scales and the output buffer may belong to the previous kernel
        const int dtid = tid;  // 0..255
        if (p.epilogue != EPI_RAW_I32)
            for (int i = dtid; i < NT; i += kLgDecoders * 32) s_s[i] = (t0 + i < M) ? __bfloat162float(p.s[t0 + i]) : 1.f;
        asm volatile("bar.sync 1, %0;" ::"n"(kLgDecoders * 32) : "memory");
        if (ok) ok = wait_or_abort(bar_acc, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);   // the tensor-memory loads below are warp-collective
        tc_fence_after();
        const int quarter = warp & 3, cpart = warp >> 2;   // TMEM lane quarter (= warp % 4) and column quarter
        const int n = rb * 128 + 32 * quarter + lane;
        const bool n_ok = n < N;
        float ws_el = 0.f;
        if (p.epilogue != EPI_RAW_I32 && p.epilogue != EPI_F32_DIV && n_ok)
            ws_el = __bfloat162float(p.ws[ws_group(n, p)]);
        if (ok) {
#pragma unroll 1
            for (int c0 = cpart * (NT / 4); c0 < (cpart + 1) * (NT / 4); c0 += 16) {
                int v[16];
                tmem_ld16(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)c0, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int t = t0 + c0 + j;
                    if (n_ok && t < M) {
                        const long long o = (long long)t * N + n;
                        if (p.epilogue == EPI_RAW_I32) reinterpret_cast<int*>(p.out)[o] = v[j];
                        else if (p.epilogue == EPI_F32_DIV) reinterpret_cast<float*>(p.out)[o] = __fdiv_rn(__int2float_rn(v[j]), s_s[c0 + j]);
                        else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = add_residual(scale_epilogue(v[j], s_s[c0 + j], ws_el, p.epilogue), p.residual, o);
                    }
                }
            }
        }
    }
    if (*abort_flag && tid == 0) atomicExch(p.status, ST_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == kLgDecoders + 1) tmem_dealloc(tmem_base, NT);
}

}  // namespace tsp
