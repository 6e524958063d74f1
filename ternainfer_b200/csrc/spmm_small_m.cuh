// Small-batch TernaSpMM kernel (up to 32 tokens per pass) for sm_100a.
//
// One launch replaces the reference's decode SpMM kernel plus its split-K
// reduction/scale kernel (kernels/src/SpMM/SpMM_Kernel.cuh:16-163 and
// kernels/src/SpMM/Reduction_Kernel.cuh:23-63 in Gu-J/TernaInfer).
//
// Work split: blockIdx.y = 64-row tile of the weight (or a pair of them, each
// with half of the warps: fat CTAs for weights with more row tiles than SMs),
// blockIdx.x = K split (the CTAs of one row tile form a thread-block
// cluster), blockIdx.z = block of MT*8 tokens.  Every warp owns whole 64x64
// tiles and runs decoupled from the other warps: it streams its tiles' bitmap
// words (one coalesced 128-bit load per lane), offsets and sign words from
// global memory through a register pipeline (bitmaps two tiles ahead, sign
// words one tile ahead), decodes them (bitmap popcount prefix -> sign windows
// -> two 256-entry lookup tables of 4 int8 weights) straight into int8 MMA A
// fragments and multiplies them with activation fragments read from L2.  The
// first tile of every warp is decoded into registers before the
// programmatic-dependency wait, since weights never depend on the previous
// kernel - and the second one into a per-warp shared-memory slot where the
// launch has one CTA per SM.  Partial sums are combined across warps in
// shared memory and across the cluster through distributed shared memory; the
// cluster's first CTA applies the scale epilogue and stores bf16.  The int32
// workspace of the reference is not needed.
//
// Template parameters: MT = token groups of 8 per pass, MAXW / MINB = launch
// bounds (warps per CTA, CTAs per SM): <1,14,2> <2,10,2> <4,8,2> are the thin
// variants (two CTAs per SM), <1,28,1> <2,20,1> <4,16,1> the fat ones.
#pragma once
#include <cuda_bf16.h>

#include "ptx_sm100.cuh"

namespace tsp {

enum Epilogue : int { EPI_DECODE = 0, EPI_PREFILL = 1, EPI_RAW_I32 = 2, EPI_F32_DIV = 3 };   // 3: fp32 acc / s[t]
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
    const __nv_bfloat16* residual;  // optional bf16 [M][N] added to the rounded result (residual stream), or null
    int ws_num, M, N, K, epilogue, splits;
    int stage_second;            // small-batch kernel: every warp has a 4 KB shared-memory slot for its second tile
    int rpc;                     // small-batch kernel: row tiles per CTA (1 or 2), each with blockDim/32/rpc warps
    int seg_b[3];   // first output column of scale segments 1, 2, 3 (INT_MAX when absent)
    int seg_gran;   // 1, or the reference's granularity: 8 (decode form) / 128 (prefill form)
    int* status;
};

constexpr int kLutBytes = 256 * 32 * 4;            // one copy of a table per lane (bank = lane)
constexpr int kLut2Bytes = 2 * kLutBytes;          // lower-nibble table + upper-nibble table
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
// the calling thread records (for kernels whose roles live in different warps)
__device__ __forceinline__ void phase_mark_here(int k) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta < 4096) g_phase_log[cta * kPhaseSlots + k] = t;
}
#else
__device__ __forceinline__ void phase_mark(int) {}
__device__ __forceinline__ void phase_mark_here(int) {}
#endif

constexpr int kRedStride = 68;                     // ints per token row of the reduction buffer (conflict-free)

// Shared-memory plan.  The lookup tables must start on a 32 KB boundary of the
// shared window (the entry index is OR-ed into the address), which the
// dynamic segment's base does not guarantee; the small buffers ("rest") go
// into the gap in front of the tables when it is large enough, else behind.
template <int MT, int RPC = 1>   // RPC: row tiles a CTA may cover (2 for the one-CTA-per-SM variants)
struct SmallMSmem {
    static constexpr int lut1 = 0;                                // the 2 x 256 entries, one copy
    static constexpr int red = lut1 + 2048;                       // int32 [RPC row tiles][MT*8][kRedStride]
    static constexpr int scl = red + RPC * MT * 8 * kRedStride * 4;   // float s[MT*8], ws[4]
    static constexpr int rest = (scl + (MT * 8 + 4) * 4 + 127) / 128 * 128;
    static constexpr int total = kLut2Bytes + kLutBytes + rest;   // worst case of the run-time placement
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

// out = linear(x) or, with a residual, bf16(residual + bf16(linear(x))): the
// two roundings of `h = x + wo(...)` in model.py:323-335 of the reference.
__device__ __forceinline__ __nv_bfloat16 add_residual(__nv_bfloat16 v, const __nv_bfloat16* residual, long long o) {
    return residual ? __float2bfloat16_rn(__bfloat162float(residual[o]) + __bfloat162float(v)) : v;
}

// One 64x64 tile as a warp sees it while it is in flight: the lane's four
// bitmap words and the tile's offsets (TileHead, loaded two tiles ahead), then
// the lane's eight sign words (TileSigns, loaded one tile ahead).
struct TileHead {
    uint4 bw;
    int toff, qbase;
};
struct TileSigns {
    uint32_t lo[4], hi[4];
    int pos;      // bit position of the lane's first sign in the stream (its low 5 bits are the first shift)
};

__device__ __forceinline__ TileHead load_head(const SpmmParams& p, long long tile, bool valid, int lane) {
    TileHead h;
    h.bw = make_uint4(0, 0, 0, 0), h.toff = 0, h.qbase = 0;
    if (valid) {
        h.bw = __ldg(reinterpret_cast<const uint4*>(p.bitmap + tile * 128) + lane);
        h.toff = __ldg(p.tile_off + tile);
        const int qd = lane >> 3;
        h.qbase = qd ? (int)__ldg(p.quarter_off + 3 * tile + qd - 1) : 0;
    }
    return h;
}

// popcounts -> 8-lane prefix (the three stored counts give the quarter bases)
// -> this lane's position in the tile's sign stream -> its sign words.
__device__ __forceinline__ TileSigns load_signs(const SpmmParams& p, const TileHead& h, bool valid, int lane) {
    TileSigns sg;
    const int c0 = __popc(h.bw.x), c1 = __popc(h.bw.y), c2 = __popc(h.bw.z), c3 = __popc(h.bw.w);
    const int tot = c0 + c1 + c2 + c3;
    int incl = tot;
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, d, 8);
        if ((lane & 7) >= d) incl += t;
    }
    int pos = h.toff + h.qbase + incl - tot;
    sg.pos = pos;
    const int cn[4] = {c0, c1, c2, c3};
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t* sw = p.signs + (pos >> 5);
        sg.lo[r] = valid ? __ldg(sw) : 0u;
        sg.hi[r] = valid ? __ldg(sw + 1) : 0u;
        pos += cn[r];
    }
    return sg;
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

// Entry of the second table, used for the upper nibble of a byte of bitmap:
// index bits 0-3 = the four sign bits just BELOW the end of the byte's sign
// run, bits 4-7 = the bitmap nibble.  The nibble's c non-zeros own the top c
// of those four bits, in ascending order.
__device__ __forceinline__ uint32_t lut_entry_upper(uint32_t e) {
    const uint32_t x4 = e & 15u, nib = e >> 4;
    const uint32_t c = __popc(nib);
    uint32_t v = 0, r = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if ((nib >> j) & 1u) {
            v |= (((x4 >> (4 - c + r)) & 1u) ? 0xFFu : 0x01u) << (8 * j);
            ++r;
        }
    return v;
}

// Same result as decode_word with 40 % fewer integer instructions, using two
// tables.  Per byte of bitmap (two nibbles) ONE shift positions both nibbles
// (lower at address bits 7-10, upper at 11-14) and per byte boundary ONE
// funnel shift positions both neighbouring sign windows: with the window
// pre-shifted by 11, shifting right by the number of non-zeros before the
// boundary puts the four sign bits above it at bits 11-14 (they belong to the
// lower nibble of the next byte, table `lut_lo`) and the four bits below it at
// bits 7-10 (they end the sign run of the upper nibble of the previous byte,
// table `lut_hi`, whose entries take their signs from the top of that field).
__device__ __forceinline__ void decode_word2(uint32_t bmw, uint32_t sgn, int total, uint32_t lut_lo, uint32_t /*lut_hi*/,
                                             uint32_t (&a)[8]) {
    const uint32_t t1 = bmw - ((bmw >> 1) & 0x55555555u);
    const uint32_t y = (t1 & 0x33333333u) + ((t1 >> 2) & 0x33333333u);  // popcount of each nibble
    const uint32_t z = (y + (y >> 4)) & 0x0F0F0F0Fu;                    // popcount of each byte
    const uint32_t pb = z * 0x01010100u;                                // byte b: non-zeros before byte b
    const uint32_t glo = sgn << 11, ghi = sgn >> 21;
    uint32_t yb[5];
    yb[0] = glo;
#pragma unroll
    for (int b = 1; b < 4; ++b) yb[b] = __funnelshift_r(glo, ghi, pb >> (8 * b));   // shift amount is taken mod 32
    yb[4] = __funnelshift_rc(glo, ghi, (uint32_t)total);   // total may be 32: clamp form, not wrap
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const uint32_t bs = b == 0 ? (bmw << 7) : (bmw >> (8 * b - 7));  // nibble 2b at bits 7-10, nibble 2b+1 at 11-14
        const uint32_t base = (bs & 0x7F80u) | lut_lo;                    // both nibbles + table base + lane, once per byte
        // one bit-select per lookup: the sign field replaces the other nibble's field
        a[2 * b] = lds32((yb[b] & 0x7800u) | (base & ~0x7800u));
        a[2 * b + 1] = lds32_plus<kLutBytes>((yb[b + 1] & 0x780u) | (base & ~0x780u));   // second table, 32 KB further
    }
}

// Decode one tile (four bitmap words) into 4 x 8 A-fragment registers.
__device__ __forceinline__ void decode_tile(const TileHead& h, const TileSigns& sg, uint32_t lut_lo, uint32_t lut_hi,
                                            uint32_t (&a)[4][8]) {
    const uint32_t w[4] = {h.bw.x, h.bw.y, h.bw.z, h.bw.w};
    int pos = sg.pos;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int c = __popc(w[r]);
        decode_word2(w[r], __funnelshift_r(sg.lo[r], sg.hi[r], (uint32_t)pos), c, lut_lo, lut_hi, a[r]);
        pos += c;
    }
}

// Decode one tile into a warp's 4 KB shared-memory slot: word r -> two 16-byte stores per lane
// ([2r + half][lane], 512 contiguous bytes per store instruction).
__device__ __forceinline__ void decode_tile_to_smem(const TileHead& h, const TileSigns& sg, uint32_t lut_lo, uint32_t lut_hi,
                                                    uint32_t slot_lane) {
    const uint32_t w[4] = {h.bw.x, h.bw.y, h.bw.z, h.bw.w};
    int pos = sg.pos;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int c = __popc(w[r]);
        uint32_t a[8];
        decode_word2(w[r], __funnelshift_r(sg.lo[r], sg.hi[r], (uint32_t)pos), c, lut_lo, lut_hi, a);
        sts128(slot_lane + (2 * r) * 512, make_uint4(a[0], a[1], a[2], a[3]));
        sts128(slot_lane + (2 * r + 1) * 512, make_uint4(a[4], a[5], a[6], a[7]));
        pos += c;
    }
}

template <int MT>
__device__ __forceinline__ void load_x_frags(uint4 (&bx)[MT], const int8_t* x, int K, int m0, int mrows, int ktile,
                                             int g, int q) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int t = mt * 8 + g;
        // produced by the previous kernel of the stream: coherent load through L2, not the read-only path
        bx[mt] = t < mrows ? ld_cg_128(x + (long long)(m0 + t) * K + ktile * 64 + q * 16) : make_uint4(0, 0, 0, 0);
    }
}

template <int MT, int MAXW, int MINB>
__global__ void __launch_bounds__(MAXW * 32, MINB) spmm_small_m_kernel(const SpmmParams p) {
    using L = SmallMSmem<MT, MINB == 1 ? 2 : 1>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t dyn = (smem_u32(smem) + 127u) & ~127u;
    const uint32_t lut_base = (dyn + (uint32_t)kLutBytes - 1u) & ~((uint32_t)kLutBytes - 1u);
    const uint32_t sbase = (lut_base - dyn >= (uint32_t)L::rest) ? dyn : lut_base + kLut2Bytes;  // "rest" region
    uint8_t* rest = smem + (sbase - smem_u32(smem));
    int* red = reinterpret_cast<int*>(rest + L::red);
    float* scl_s = reinterpret_cast<float*>(rest + L::scl);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = (blockDim.x >> 5) / p.rpc;
    const int g = lane >> 2, q = lane & 3;
    const int rank = blockIdx.x, S = p.splits;
    // Row tiles of this CTA: one, or two with half of the warps each (a fat CTA that covers 128 rows,
    // for weights with more row tiles than SMs).  `nwarps` below = the warps that share a row tile.
    const int rpc = p.rpc, sub = rpc == 2 ? warp / ((blockDim.x >> 5) >> 1) : 0;
    const int rt = blockIdx.y * rpc + sub;
    const bool rt_ok = rt * 64 < p.N;
    const int m0 = blockIdx.z * (MT * 8);
    const int mrows = min(p.M - m0, MT * 8);
    const int KT = p.K >> 6;
    const int kt0 = (int)(((long long)KT * rank) / S), kt1 = rt_ok ? (int)(((long long)KT * (rank + 1)) / S) : kt0;
    const long long tile0 = (long long)rt * KT;

    phase_mark(0);
    // Let the next kernel in the stream start its own weight prefetch now
    // (programmatic dependent launch; a no-op for ordinary launches).
    griddep_launch_dependents();

    // ---- prologue: everything up to the dependency wait touches only
    // immutable weight data, so it may overlap the previous kernel.
    // First loads of this warp's pipeline (tiles kt0+warp, +nwarps, ...):
    int kt = kt0 + (warp - sub * nwarps);
    int* red_w = red + sub * (MT * 8 * kRedStride);   // this row tile's reduction buffer
    TileHead h_cur = load_head(p, tile0 + kt, kt < kt1, lane);
    TileHead h_nxt = load_head(p, tile0 + kt + nwarps, kt + nwarps < kt1, lane);
    // lookup tables: the 2 x 256 entries once, then 32 copies (lane l reads bank l)
    for (int e = tid; e < 512; e += blockDim.x)
        reinterpret_cast<uint32_t*>(rest + L::lut1)[e] = e < 256 ? lut_entry(e) : lut_entry_upper(e - 256);
    for (int i = tid; i < rpc * MT * 8 * kRedStride; i += blockDim.x) red[i] = 0;
    __syncthreads();
    for (int i = tid; i < 512 * 8; i += blockDim.x) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(rest + L::lut1)[i >> 3];
        sts128(lut_base + i * 16, make_uint4(v, v, v, v));
    }
    TileSigns s_cur = load_signs(p, h_cur, kt < kt1, lane);
    __syncthreads();
    if (S > 1) cluster_arrive();  // this CTA's reduction buffer is zeroed
    phase_mark(1);

    int acc[4][MT][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][mt][c] = 0;

    const uint32_t lut_lo = lut_base | (uint32_t)(lane * 4), lut_hi = lut_lo + kLutBytes;

    // ---- decode this warp's first tile into registers before the wait
    uint32_t pre[4][8];
    const bool have_first = kt < kt1;
    if (have_first) decode_tile(h_cur, s_cur, lut_lo, lut_hi, pre);
    TileSigns s_nxt = load_signs(p, h_nxt, kt + nwarps < kt1, lane);
    TileHead h_far = load_head(p, tile0 + kt + 2 * nwarps, kt + 2 * nwarps < kt1, lane);
    // ---- and, where the launch gives every warp a shared-memory slot (one fat CTA per SM), the
    // second tile too: after the wait only the activation loads and the MMAs are left for it
    const bool staged = p.stage_second && kt + nwarps < kt1;
    const uint32_t slot_lane = lut_base + kLut2Bytes + (uint32_t)L::rest + (uint32_t)(warp * 4096 + lane * 16);
    if (staged) {
        decode_tile_to_smem(h_nxt, s_nxt, lut_lo, lut_hi, slot_lane);
        h_nxt = h_far;
        s_nxt = load_signs(p, h_nxt, kt + 2 * nwarps < kt1, lane);
        h_far = load_head(p, tile0 + kt + 3 * nwarps, kt + 3 * nwarps < kt1, lane);
    }
    phase_mark(3);

    // ---- activations, scales and the output may belong to the previous kernel
    griddep_wait();
    phase_mark(4);
    if (tid < mrows && p.epilogue != EPI_RAW_I32) scl_s[tid] = __bfloat162float(p.s[m0 + tid]);
    if (tid >= 32 && tid < 36 && p.epilogue != EPI_RAW_I32 && p.epilogue != EPI_F32_DIV) scl_s[MT * 8 + tid - 32] = __bfloat162float(p.ws[tid - 32]);

    if (have_first) {
        uint4 bx[MT];
        load_x_frags<MT>(bx, p.x, p.K, m0, mrows, kt, g, q);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_s8_16x8x32(acc[r][mt], pre[r][0], pre[r][1], pre[r][2], pre[r][3], bx[mt].x, bx[mt].y);
                mma_s8_16x8x32(acc[r][mt], pre[r][4], pre[r][5], pre[r][6], pre[r][7], bx[mt].z, bx[mt].w);
            }
    }

    if (staged) {
        kt += nwarps;
        uint4 bx[MT];
        load_x_frags<MT>(bx, p.x, p.K, m0, mrows, kt, g, q);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint4 lo = lds128(slot_lane + (2 * r) * 512), hi = lds128(slot_lane + (2 * r + 1) * 512);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_s8_16x8x32(acc[r][mt], lo.x, lo.y, lo.z, lo.w, bx[mt].x, bx[mt].y);
                mma_s8_16x8x32(acc[r][mt], hi.x, hi.y, hi.z, hi.w, bx[mt].z, bx[mt].w);
            }
        }
    }

    // ---- remaining tiles of this warp: streamed through the register pipeline
    for (kt += nwarps; kt < kt1; kt += nwarps) {
        h_cur = h_nxt, s_cur = s_nxt, h_nxt = h_far;
        uint4 bx[MT];
        load_x_frags<MT>(bx, p.x, p.K, m0, mrows, kt, g, q);
        s_nxt = load_signs(p, h_nxt, kt + nwarps < kt1, lane);
        h_far = load_head(p, tile0 + kt + 2 * nwarps, kt + 2 * nwarps < kt1, lane);
        uint32_t a[4][8];
        decode_tile(h_cur, s_cur, lut_lo, lut_hi, a);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_s8_16x8x32(acc[r][mt], a[r][0], a[r][1], a[r][2], a[r][3], bx[mt].x, bx[mt].y);
                mma_s8_16x8x32(acc[r][mt], a[r][4], a[r][5], a[r][6], a[r][7], bx[mt].z, bx[mt].w);
            }
    }
    phase_mark(5);

    // ---- combine: warps -> CTA buffer -> cluster rank 0
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int v = acc[r][mt][c];
                if (v != 0) atomicAdd(&red_w[(mt * 8 + 2 * q + (c & 1)) * kRedStride + 16 * r + g + 8 * (c >> 1)], v);
            }
    __syncthreads();
    phase_mark(6);
    if (S > 1) {
        cluster_wait();  // every CTA of the cluster has zeroed its buffer
        phase_mark(7);
        if (rank != 0) {
            const uint32_t remote = map_to_rank(sbase + L::red, 0);
            for (int i = tid; i < rpc * MT * 8 * kRedStride; i += blockDim.x) {
                const int v = red[i];
                if (v != 0) red_add_cluster(remote + i * 4, v);
            }
        }
        cluster_arrive();
        cluster_wait();  // all partial sums have landed in rank 0
        phase_mark(8);
        if (rank != 0) return;
    }

    // ---- epilogue (rank 0): scale and store
    const int N = p.N;
    for (int i = tid; i < rpc * mrows * 64; i += blockDim.x) {
        const int j = i >= mrows * 64 ? 1 : 0, r = i - j * mrows * 64;   // row tile of the CTA, index inside it
        const int t = r >> 6, nl = r & 63;
        const int n = ((int)blockIdx.y * rpc + j) * 64 + nl;
        if (n >= N) continue;
        const int v = red[j * (MT * 8 * kRedStride) + t * kRedStride + nl];
        const long long o = (long long)(m0 + t) * N + n;
        if (p.epilogue == EPI_RAW_I32) {
            reinterpret_cast<int*>(p.out)[o] = v;
        } else if (p.epilogue == EPI_F32_DIV) {
            reinterpret_cast<float*>(p.out)[o] = __fdiv_rn(__int2float_rn(v), scl_s[t]);
        } else {
            const float s_el = scl_s[t];
            const float ws_el = scl_s[MT * 8 + ws_group(n, p)];
            reinterpret_cast<__nv_bfloat16*>(p.out)[o] = add_residual(scale_epilogue(v, s_el, ws_el, p.epilogue), p.residual, o);
        }
    }
    phase_mark(9);
}

}  // namespace tsp
