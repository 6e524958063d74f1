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
    int* status;
};

constexpr int kChunkTiles = 16;                    // k-tiles resident in shared memory at once
constexpr int kXStride = kChunkTiles * 64 + 64;    // bytes per token row: == 64 (mod 128), conflict-free 128-bit reads
constexpr int kLutBytes = 256 * 32 * 4;            // one copy of the table per lane (bank = lane)
constexpr int kSignBufBytes = kChunkTiles * 512 + 64;

template <int MT>
struct SmallMSmem {
    static constexpr int lut = 0;
    static constexpr int red = lut + kLutBytes;                   // int32 [MT*8][64]
    static constexpr int toff = red + MT * 8 * 64 * 4;            // int [kChunkTiles+1]
    static constexpr int qoff = toff + 80;                        // u16 [3*kChunkTiles]
    static constexpr int bar = qoff + 96;                         // mbarrier
    static constexpr int bm = bar + 16;                           // bitmap chunk
    static constexpr int sg = bm + kChunkTiles * 512;             // sign chunk
    static constexpr int xs = sg + kSignBufBytes;                 // activations
    static constexpr int total = xs + MT * 8 * kXStride;
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

// Scale-segment index of output column n.  Decode form: one group per 8
// consecutive outputs, the 2560/640/640 split when ws_num == 3 and N == 3840
// (Reduction_Kernel.cuh:42-54).  Prefill form: one group per 128 columns,
// N == 3840 alone selects the split, clamped (epilogue_visitor_scale_ws.h:
// 135-145).
__device__ __forceinline__ int ws_group(int n, int N, int ws_num, int epilogue) {
    int g;
    if (epilogue == EPI_PREFILL) {
        const int col = n & ~127;
        if (N == 3840) g = col < 2560 ? 0 : (col < 3200 ? 1 : 2);
        else g = col / (N / ws_num);
        g = min(g, ws_num - 1);
    } else {
        const int col = n & ~7;
        if (ws_num == 3 && N == 3840) g = col < 2560 ? 0 : (col < 3200 ? 1 : 2);
        else g = col / (N / ws_num);
    }
    return min(max(g, 0), 3);
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

template <int MT, int MAXW>
__global__ void __launch_bounds__(MAXW * 32, 1) spmm_small_m_kernel(const SpmmParams p) {
    using L = SmallMSmem<MT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    uint32_t* lut_w = reinterpret_cast<uint32_t*>(smem + L::lut);
    int* red = reinterpret_cast<int*>(smem + L::red);
    int* toff_s = reinterpret_cast<int*>(smem + L::toff);
    uint16_t* qoff_s = reinterpret_cast<uint16_t*>(smem + L::qoff);
    const uint32_t bar = sbase + L::bar;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int rank = blockIdx.x, S = p.splits;
    const int rt = blockIdx.y;
    const int m0 = blockIdx.z * (MT * 8);
    const int mrows = min(p.M - m0, MT * 8);
    const int KT = p.K >> 6;
    const int kt0 = (int)(((long long)KT * rank) / S), kt1 = (int)(((long long)KT * (rank + 1)) / S);

    // ---- set-up: lookup table, zeroed reduction buffer and padding rows
    for (int i = tid; i < 256 * 32; i += blockDim.x) lut_w[i] = lut_entry(i >> 5);
    for (int i = tid; i < MT * 8 * 64; i += blockDim.x) red[i] = 0;
    for (int i = tid; i < (MT * 8 - mrows) * (kXStride / 16); i += blockDim.x)
        reinterpret_cast<uint4*>(smem + L::xs + mrows * kXStride)[i] = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    cluster_arrive();  // this CTA's reduction buffer is zeroed

    int acc[4][MT][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][mt][c] = 0;

    const uint32_t lut_lane = sbase + L::lut + lane * 4;
    uint32_t phase = 0;
    bool ok = true;

    for (int c0 = kt0; c0 < kt1 && ok; c0 += kChunkTiles) {
        const int n = min(kChunkTiles, kt1 - c0);
        const long long tbase = (long long)rt * KT + c0;
        if (c0 != kt0) __syncthreads();  // every warp is done with the previous chunk
        if (tid == 0) {
            mbar_expect_tx(bar, (uint32_t)(n * 512 + mrows * n * 64));
            bulk_g2s(sbase + L::bm, p.bitmap + tbase * 128, (uint32_t)(n * 512), bar);
        }
        if (warp == 0)
            for (int t = lane; t < mrows; t += 32)
                bulk_g2s(sbase + L::xs + t * kXStride, p.x + (long long)(m0 + t) * p.K + c0 * 64, (uint32_t)(n * 64),
                         bar);
        if (tid <= n) toff_s[tid] = p.tile_off[tbase + tid];
        if (tid < 3 * n) qoff_s[tid] = p.quarter_off[3 * tbase + tid];
        __syncthreads();
        const int w_first = (toff_s[0] >> 5) & ~3;  // first sign word of the chunk, rounded down to 16 bytes
        if (tid == 0) {
            const int w_end = ((toff_s[n] >> 5) + 3) & ~3;
            const uint32_t bytes = (uint32_t)(w_end - w_first) * 4u;
            if (bytes) {
                mbar_expect_tx(bar, bytes);
                bulk_g2s(sbase + L::sg, p.signs + w_first, bytes, bar);
            }
            mbar_arrive(bar);
        }
        ok = mbar_wait_bounded(bar, phase);
        phase ^= 1u;
        if (!ok) break;

        for (int i = warp; i < n; i += nwarps) {
            const uint4 bw = lds128(sbase + L::bm + i * 512 + lane * 16);
            const uint32_t w[4] = {bw.x, bw.y, bw.z, bw.w};
            int cnt[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) cnt[r] = __popc(w[r]);
            const int tot = cnt[0] + cnt[1] + cnt[2] + cnt[3];
            int incl = tot;  // inclusive prefix over the 8 lanes of this quarter
#pragma unroll
            for (int d = 1; d < 8; d <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, d, 8);
                if ((lane & 7) >= d) incl += t;
            }
            const int qd = lane >> 3;
            const int qbase = qd ? (int)qoff_s[3 * i + qd - 1] : 0;
            int pos = toff_s[i] - w_first * 32 + qbase + incl - tot;  // bit position in the sign buffer

            uint4 bx[MT];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) bx[mt] = lds128(sbase + L::xs + (mt * 8 + g) * kXStride + i * 64 + q * 16);

#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const uint32_t sw = sbase + L::sg + (uint32_t)(pos >> 5) * 4u;
                uint32_t sgn = __funnelshift_r(lds32(sw), lds32(sw + 4), pos & 31);
                pos += cnt[r];
                uint32_t a[8];
                uint32_t bmw = w[r];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t nib = bmw & 15u;
                    a[j] = lds32(lut_lane + ((nib | ((sgn & 15u) << 4)) << 7));
                    sgn >>= __popc(nib);
                    bmw >>= 4;
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_s8_16x8x32(acc[r][mt], a[0], a[1], a[2], a[3], bx[mt].x, bx[mt].y);
                    mma_s8_16x8x32(acc[r][mt], a[4], a[5], a[6], a[7], bx[mt].z, bx[mt].w);
                }
            }
        }
    }
    if (!ok && tid == 0) atomicExch(p.status, ST_WAIT_TIMEOUT);

    // ---- combine: warps -> CTA buffer -> cluster rank 0
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int v = acc[r][mt][c];
                if (v != 0) atomicAdd(&red[(mt * 8 + 2 * q + (c & 1)) * 64 + 16 * r + g + 8 * (c >> 1)], v);
            }
    __syncthreads();
    cluster_wait();  // every CTA of the cluster has zeroed its buffer
    if (rank != 0) {
        const uint32_t remote = map_to_rank(sbase + L::red, 0);
        for (int i = tid; i < MT * 8 * 64; i += blockDim.x) {
            const int v = red[i];
            if (v != 0) red_add_cluster(remote + i * 4, v);
        }
    }
    cluster_arrive();
    cluster_wait();  // all partial sums have landed in rank 0
    if (rank != 0) return;

    // ---- epilogue (rank 0): scale and store
    const int N = p.N;
    for (int i = tid; i < mrows * 64; i += blockDim.x) {
        const int t = i >> 6, nl = i & 63;
        const int n = rt * 64 + nl;
        const int v = red[t * 64 + nl];
        const long long o = (long long)(m0 + t) * N + n;
        if (p.epilogue == EPI_RAW_I32) {
            reinterpret_cast<int*>(p.out)[o] = v;
        } else {
            const float s_el = __bfloat162float(p.s[m0 + t]);
            const float ws_el = __bfloat162float(p.ws[ws_group(n, N, p.ws_num, p.epilogue)]);
            reinterpret_cast<__nv_bfloat16*>(p.out)[o] = scale_epilogue(v, s_el, ws_el, p.epilogue);
        }
    }
}

}  // namespace tsp
