// Small-batch TernaSpMM kernel (up to 32 tokens per pass) for sm_100a.
//
// One launch replaces the reference's decode SpMM kernel plus its split-K
// reduction/scale kernel (kernels/src/SpMM/SpMM_Kernel.cuh:16-163 and
// kernels/src/SpMM/Reduction_Kernel.cuh:23-63 in Gu-J/TernaInfer).
//
// Work split: blockIdx.y = 64-row tile of the weight, blockIdx.x = K split
// (the CTAs of one row tile form a thread-block cluster), blockIdx.z = block
// of MT*8 tokens.  Each CTA streams its compressed k-tiles into shared memory
// with 1-D bulk async copies completing on an mbarrier, each warp decodes
// whole 64x64 tiles (bitmap popcount prefix -> sign window -> 256-entry
// lookup of 4 int8 weights) straight into int8 MMA A fragments and multiplies
// them with the activation fragments, partial sums are combined across warps
// in shared memory and across the cluster through distributed shared memory,
// and the cluster's first CTA applies the scale epilogue and stores bf16.
// The int32 workspace of the reference is not needed.
#pragma once
#include <cuda_bf16.h>

#include "ptx_sm100.cuh"

namespace tsp {

enum Epilogue : int { EPI_DECODE = 0, EPI_PREFILL = 1, EPI_RAW_I32 = 2 };
enum Status : int { ST_OK = 0, ST_BAD_SHAPE = 1, ST_BAD_POINTER = 2, ST_LAUNCH = 3, ST_WAIT_TIMEOUT = 4 };

struct SpmmParams {
    const int8_t* x;             // [M][K] int8
    const uint32_t* bitmap;      // tiles * 128 words
    const int* tile_off;         // tiles + 1, in values (bits), multiples of 32
    const uint16_t* quarter_off; // 3 per tile: non-zeros after lanes 7, 15, 23
    const uint32_t* signs;       // packed sign bits
    void* out;                   // bf16 [M][N] or int32 [M][N]
    const __nv_bfloat16* s;      // [M]
    const __nv_bfloat16* ws;     // [4]
    int ws_num, M, N, K, epilogue, splits;
    int seg_b[3];   // first output column of scale segments 1, 2, 3 (INT_MAX when absent)
    int seg_gran;   // 1, or the reference's granularity: 8 (decode form) / 128 (prefill form)
    int* status;
};

constexpr int kChunkTiles = 16;                    // k-tiles resident in shared memory at once
constexpr int kLutBytes = 256 * 32 * 4;            // one copy of the table per lane (bank = lane)
constexpr int kSignBufBytes = kChunkTiles * 512 + 64;
constexpr int kPreTiles = 1;                       // tiles per warp decoded into registers before the dependency wait

// Phase timestamps for tuning builds (-DTSP_PHASE_TIMERS): thread 0 of every
// CTA records the global timer at a few points; compiled out otherwise.
#ifdef TSP_PHASE_TIMERS
constexpr int kPhaseSlots = 12;
__device__ unsigned long long g_phase_log[4096 * kPhaseSlots];
__device__ __forceinline__ void phase_mark(int k) {
    if (threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        if (cta < 4096) g_phase_log[cta * kPhaseSlots + k] = t;
    }
}
#else
__device__ __forceinline__ void phase_mark(int) {}
#endif

constexpr int kRedStride = 68;                     // ints per token row of the reduction buffer (conflict-free)

// Shared-memory plan.  The lookup table must start on a 32 KB boundary of the
// shared window (its entry index is OR-ed into the address), which the
// dynamic segment's base does not guarantee; the other buffers ("rest") go
// into the gap in front of the table when it is large enough, else behind it.
template <int MT>
struct SmallMSmem {
    static constexpr int lut1 = 0;                                // the 256 entries, one copy
    static constexpr int red = lut1 + 1024;                       // int32 [MT*8][kRedStride]
    static constexpr int toff = red + MT * 8 * kRedStride * 4;    // int [kChunkTiles+1]
    static constexpr int qoff = toff + 80;                        // u16 [3*kChunkTiles]
    static constexpr int scl = qoff + 96;                         // float s[MT*8], ws[4]
    static constexpr int flag = scl + (MT * 8 + 4) * 4;           // int: bulk copies arrived
    static constexpr int bar = flag + 8;                          // mbarrier
    static constexpr int bm = (bar + 16 + 127) / 128 * 128;       // bitmap chunk
    static constexpr int sg = bm + kChunkTiles * 512;             // sign chunk
    static constexpr int rest = (sg + kSignBufBytes + 127) / 128 * 128;
    static constexpr int total = kLutBytes + 2 * rest + 128;      // worst case of the run-time placement
    static_assert(2 * rest >= kLutBytes, "placement bound assumes the gap never exceeds twice the rest region");
};

// Four int8 weights of one bitmap nibble: bit j of `nib` set -> weight j is
// +1, or -1 when the next unused sign bit is set; sign bits are consumed in
// ascending j.
__device__ __forceinline__ uint32_t lut_entry(uint32_t e) {
    const uint32_t nib = e & 15u, sg = e >> 4;
    uint32_t v = 0, r = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if ((nib >> j) & 1u) {
            v |= (((sg >> r) & 1u) ? 0xFFu : 0x01u) << (8 * j);
            ++r;
        }
    return v;
}

// Scale-segment index of output column n.  The host turns the reference's
// rules into three boundaries and a granularity: the decode form decides per
// group of 8 outputs, equal widths N/ws_num or the 2560/640/640 split when
// ws_num == 3 and N == 3840 (Reduction_Kernel.cuh:42-54); the prefill form
// decides per 128 columns, N == 3840 alone selects the split, and the index is
// clamped to ws_num-1 (epilogue_visitor_scale_ws.h:135-145).  Explicit
// boundaries (sharded layers) use granularity 1.
__device__ __forceinline__ int ws_group(int n, const SpmmParams& p) {
    const int col = n & ~(p.seg_gran - 1);
    const int g = (col >= p.seg_b[0]) + (col >= p.seg_b[1]) + (col >= p.seg_b[2]);
    const int limit = (p.epilogue == EPI_PREFILL || p.seg_gran == 1) ? p.ws_num - 1 : 3;
    return max(min(g, limit), 0);
}

__device__ __forceinline__ __nv_bfloat16 scale_epilogue(int acc, float s_el, float ws_el, int epilogue) {
    float v;
    if (epilogue == EPI_PREFILL) {
        const float coeff = (s_el != 0.f) ? __fdiv_rn(ws_el, s_el) : 0.f;
        v = __fmul_rn(__int2float_rn(acc), coeff);
    } else {
        v = __fmul_rn(__fdiv_rn(__int2float_rn(acc), s_el), ws_el);
    }
    return __float2bfloat16_rn(v);
}

// Sign-stream position (in bits, relative to the chunk's first loaded word) of
// this lane's first non-zero of tile i, plus the lane's four bitmap words.
struct TileHead {
    uint32_t w[4];
    int cnt[4];
    int pos;
};

__device__ __forceinline__ TileHead tile_head(uint32_t bm_tile, const int* toff_s, const uint16_t* qoff_s, int i,
                                              int w_first, int lane) {
    TileHead h;
    const uint4 bw = lds128(bm_tile + lane * 16);
    h.w[0] = bw.x, h.w[1] = bw.y, h.w[2] = bw.z, h.w[3] = bw.w;
#pragma unroll
    for (int r = 0; r < 4; ++r) h.cnt[r] = __popc(h.w[r]);
    const int tot = h.cnt[0] + h.cnt[1] + h.cnt[2] + h.cnt[3];
    int incl = tot;  // inclusive prefix over the 8 lanes of this quarter
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, d, 8);
        if ((lane & 7) >= d) incl += t;
    }
    const int qd = lane >> 3;
    const int qbase = qd ? (int)qoff_s[3 * i + qd - 1] : 0;
    h.pos = toff_s[i] - w_first * 32 + qbase + incl - tot;
    return h;
}

// One bitmap word (32 weights: rows g and g+8 of one 16-row group, 16 k) and
// its sign window -> the 8 A-fragment registers of two k32 MMA steps.
// All eight sign offsets come from one bit-parallel prefix (nibble popcounts
// -> byte fields -> multiply), so the eight table reads are independent.
// `lut_lane` = table base (32 KB aligned) | lane*4; entry index = bitmap
// nibble | sign nibble << 4 sits in address bits 7..14.
__device__ __forceinline__ void decode_word(uint32_t bmw, uint32_t sgn, uint32_t lut_lane, uint32_t (&a)[8]) {
    const uint32_t t1 = bmw - ((bmw >> 1) & 0x55555555u);
    const uint32_t y = (t1 & 0x33333333u) + ((t1 >> 2) & 0x33333333u);  // popcount of each nibble
    const uint32_t ye = y & 0x0F0F0F0Fu;                                // nibbles 0,2,4,6 in bytes 0..3
    const uint32_t yo = (y >> 4) & 0x0F0F0F0Fu;                         // nibbles 1,3,5,7
    const uint32_t pe = (ye + yo) * 0x01010100u;                        // byte b: non-zeros before nibble 2b
    const uint32_t po = pe + ye;                                        // byte b: non-zeros before nibble 2b+1
    const uint32_t glo = sgn << 11, ghi = sgn >> 21;                    // sign window pre-shifted to bits 11..
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t amt = ((j & 1) ? po : pe) >> (8 * (j >> 1));     // the funnel shift uses amt mod 32
        const uint32_t gs = __funnelshift_r(glo, ghi, amt);
        const uint32_t bj = (4 * j <= 7) ? (bmw << (7 - 4 * j)) : (bmw >> (4 * j - 7));
        a[j] = lds32((bj & 0x780u) | ((gs & 0x7800u) | lut_lane));
    }
}

__device__ __forceinline__ uint32_t sign_window(uint32_t sg_base, int pos) {
    const uint32_t sw = sg_base + (uint32_t)(pos >> 5) * 4u;
    return __funnelshift_r(lds32(sw), lds32(sw + 4), pos & 31);
}

template <int MT>
__device__ __forceinline__ void load_x_frags(uint4 (&bx)[MT], const int8_t* x, int K, int m0, int mrows, int ktile,
                                             int g, int q) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int t = mt * 8 + g;
        bx[mt] = t < mrows ? __ldg(reinterpret_cast<const uint4*>(x + (long long)(m0 + t) * K + ktile * 64 + q * 16))
                           : make_uint4(0, 0, 0, 0);
    }
}

template <int MT, int MAXW, int MINB>
__global__ void __launch_bounds__(MAXW * 32, MINB) spmm_small_m_kernel(const SpmmParams p) {
    using L = SmallMSmem<MT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t dyn = (smem_u32(smem) + 127u) & ~127u;
    const uint32_t lut_base = (dyn + (uint32_t)kLutBytes - 1u) & ~((uint32_t)kLutBytes - 1u);
    const uint32_t sbase = (lut_base - dyn >= (uint32_t)L::rest) ? dyn : lut_base + kLutBytes;  // "rest" region
    uint8_t* rest = smem + (sbase - smem_u32(smem));
    int* red = reinterpret_cast<int*>(rest + L::red);
    int* toff_s = reinterpret_cast<int*>(rest + L::toff);
    uint16_t* qoff_s = reinterpret_cast<uint16_t*>(rest + L::qoff);
    float* scl_s = reinterpret_cast<float*>(rest + L::scl);
    const uint32_t bar = sbase + L::bar;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int rank = blockIdx.x, S = p.splits;
    const int rt = blockIdx.y;
    const int m0 = blockIdx.z * (MT * 8);
    const int mrows = min(p.M - m0, MT * 8);
    const int KT = p.K >> 6;
    const int kt0 = (int)(((long long)KT * rank) / S), kt1 = (int)(((long long)KT * (rank + 1)) / S);

    phase_mark(0);
    // Let the next kernel in the stream start its own weight prefetch now
    // (programmatic dependent launch; a no-op for ordinary launches).
    griddep_launch_dependents();

    // ---- prologue: everything here touches only immutable weight data, so it
    // may run while the previous kernel of the stream is still executing.
    const int n0 = min(kChunkTiles, kt1 - kt0);
    const long long tbase0 = (long long)rt * KT + kt0;
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
        mbar_expect_tx(bar, (uint32_t)(n0 * 512));
        bulk_g2s(sbase + L::bm, p.bitmap + tbase0 * 128, (uint32_t)(n0 * 512), bar);
    }
    int toff_v = 0, qoff_v = 0;
    if (tid <= n0) toff_v = p.tile_off[tbase0 + tid];
    if (tid < 3 * n0) qoff_v = p.quarter_off[3 * tbase0 + tid];
    // lookup table: the 256 entries once, then 32 copies (lane l reads bank l)
    for (int e = tid; e < 256; e += blockDim.x) reinterpret_cast<uint32_t*>(rest + L::lut1)[e] = lut_entry(e);
    for (int i = tid; i < MT * 8 * kRedStride; i += blockDim.x) red[i] = 0;
    if (tid <= n0) toff_s[tid] = toff_v;
    if (tid < 3 * n0) qoff_s[tid] = (uint16_t)qoff_v;
    __syncthreads();
    int w_first = (toff_s[0] >> 5) & ~3;  // first sign word of the chunk, rounded down to 16 bytes
    if (tid == 0) {
        const int w_end = ((toff_s[n0] >> 5) + 3) & ~3;
        const uint32_t bytes = (uint32_t)(w_end - w_first) * 4u;
        if (bytes) {
            mbar_expect_tx(bar, bytes);
            bulk_g2s(sbase + L::sg, p.signs + w_first, bytes, bar);
        }
        mbar_arrive(bar);
    }
    for (int i = tid; i < 256 * 8; i += blockDim.x) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(rest + L::lut1)[i >> 3];
        sts128(lut_base + i * 16, make_uint4(v, v, v, v));
    }
    __syncthreads();
    cluster_arrive();  // this CTA's reduction buffer is zeroed
    phase_mark(1);

    int acc[4][MT][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][mt][c] = 0;

    const uint32_t lut_lane = lut_base | (uint32_t)(lane * 4);
    // One warp polls the copy barrier; the others sleep at the CTA barrier
    // instead of spending issue slots on polling.
    volatile int* ok_flag = reinterpret_cast<volatile int*>(rest + L::flag);
    uint32_t phase = 0;
    if (warp == 0) {
        const bool arrived = mbar_wait_bounded(bar, phase);
        if (lane == 0) *ok_flag = arrived;
    }
    __syncthreads();
    bool ok = *ok_flag != 0;
    phase ^= 1u;
    phase_mark(2);

    // ---- decode this warp's first tile(s) into registers before the wait
    uint32_t pre[kPreTiles][4][8];
    if (ok) {
#pragma unroll
        for (int tp = 0; tp < kPreTiles; ++tp) {
            const int i = warp + tp * nwarps;
            if (i < n0) {
                TileHead h = tile_head(sbase + L::bm + i * 512, toff_s, qoff_s, i, w_first, lane);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    decode_word(h.w[r], sign_window(sbase + L::sg, h.pos), lut_lane, pre[tp][r]);
                    h.pos += h.cnt[r];
                }
            }
        }
    }
    phase_mark(3);

    // ---- activations, scales and the output may belong to the previous kernel
    griddep_wait();
    phase_mark(4);
    if (tid < mrows && p.epilogue != EPI_RAW_I32) scl_s[tid] = __bfloat162float(p.s[m0 + tid]);
    if (tid >= 32 && tid < 36 && p.epilogue != EPI_RAW_I32) scl_s[MT * 8 + tid - 32] = __bfloat162float(p.ws[tid - 32]);

    if (ok) {
#pragma unroll
        for (int tp = 0; tp < kPreTiles; ++tp) {
            const int i = warp + tp * nwarps;
            if (i < n0) {
                uint4 bx[MT];
                load_x_frags<MT>(bx, p.x, p.K, m0, mrows, kt0 + i, g, q);
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma_s8_16x8x32(acc[r][mt], pre[tp][r][0], pre[tp][r][1], pre[tp][r][2], pre[tp][r][3],
                                       bx[mt].x, bx[mt].y);
                        mma_s8_16x8x32(acc[r][mt], pre[tp][r][4], pre[tp][r][5], pre[tp][r][6], pre[tp][r][7],
                                       bx[mt].z, bx[mt].w);
                    }
            }
        }
    }

    // ---- remaining tiles: streamed (decode + multiply), chunk by chunk
    for (int c0 = kt0; c0 < kt1 && ok; c0 += kChunkTiles) {
        const int n = min(kChunkTiles, kt1 - c0);
        if (c0 != kt0) {
            const long long tbase = (long long)rt * KT + c0;
            __syncthreads();  // every warp is done with the previous chunk
            if (tid == 0) {
                mbar_expect_tx(bar, (uint32_t)(n * 512));
                bulk_g2s(sbase + L::bm, p.bitmap + tbase * 128, (uint32_t)(n * 512), bar);
            }
            if (tid <= n) toff_s[tid] = p.tile_off[tbase + tid];
            if (tid < 3 * n) qoff_s[tid] = p.quarter_off[3 * tbase + tid];
            __syncthreads();
            w_first = (toff_s[0] >> 5) & ~3;
            if (tid == 0) {
                const int w_end = ((toff_s[n] >> 5) + 3) & ~3;
                const uint32_t bytes = (uint32_t)(w_end - w_first) * 4u;
                if (bytes) {
                    mbar_expect_tx(bar, bytes);
                    bulk_g2s(sbase + L::sg, p.signs + w_first, bytes, bar);
                }
                mbar_arrive(bar);
            }
            if (warp == 0) {
                const bool arrived = mbar_wait_bounded(bar, phase);
                if (lane == 0) *ok_flag = arrived;
            }
            __syncthreads();
            ok = *ok_flag != 0;
            phase ^= 1u;
            if (!ok) break;
        }
        for (int i = warp + (c0 == kt0 ? kPreTiles * nwarps : 0); i < n; i += nwarps) {
            TileHead h = tile_head(sbase + L::bm + i * 512, toff_s, qoff_s, i, w_first, lane);
            uint4 bx[MT];
            load_x_frags<MT>(bx, p.x, p.K, m0, mrows, c0 + i, g, q);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                uint32_t a[8];
                decode_word(h.w[r], sign_window(sbase + L::sg, h.pos), lut_lane, a);
                h.pos += h.cnt[r];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_s8_16x8x32(acc[r][mt], a[0], a[1], a[2], a[3], bx[mt].x, bx[mt].y);
                    mma_s8_16x8x32(acc[r][mt], a[4], a[5], a[6], a[7], bx[mt].z, bx[mt].w);
                }
            }
        }
    }
    if (!ok && tid == 0) atomicExch(p.status, ST_WAIT_TIMEOUT);
    phase_mark(5);

    // ---- combine: warps -> CTA buffer -> cluster rank 0
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int v = acc[r][mt][c];
                if (v != 0) atomicAdd(&red[(mt * 8 + 2 * q + (c & 1)) * kRedStride + 16 * r + g + 8 * (c >> 1)], v);
            }
    __syncthreads();
    phase_mark(6);
    cluster_wait();  // every CTA of the cluster has zeroed its buffer
    phase_mark(7);
    if (rank != 0) {
        const uint32_t remote = map_to_rank(sbase + L::red, 0);
        for (int i = tid; i < MT * 8 * kRedStride; i += blockDim.x) {
            const int v = red[i];
            if (v != 0) red_add_cluster(remote + i * 4, v);
        }
    }
    cluster_arrive();
    cluster_wait();  // all partial sums have landed in rank 0
    phase_mark(8);
    if (rank != 0) return;

    // ---- epilogue (rank 0): scale and store
    const int N = p.N;
    for (int i = tid; i < mrows * 64; i += blockDim.x) {
        const int t = i >> 6, nl = i & 63;
        const int n = rt * 64 + nl;
        const int v = red[t * kRedStride + nl];
        const long long o = (long long)(m0 + t) * N + n;
        if (p.epilogue == EPI_RAW_I32) {
            reinterpret_cast<int*>(p.out)[o] = v;
        } else {
            const float s_el = scl_s[t];
            const float ws_el = scl_s[MT * 8 + ws_group(n, p)];
            reinterpret_cast<__nv_bfloat16*>(p.out)[o] = scale_epilogue(v, s_el, ws_el, p.epilogue);
        }
    }
    phase_mark(9);
}

}  // namespace tsp
