// Work-list TernaSpMM kernel for sm_100a: MANY independent small-batch linears
// (up to 16 tokens each) in ONE persistent launch.
//
// A call of bitlinear_TernaSpMM on a BitNet-2B layer streams 1.3 - 7 MB of
// compressed weights: 0.2 - 1.1 us at HBM speed, well below what a launch costs
// even with programmatic dependent launch (table build, dependency wait, grid
// completion).  This kernel takes a table of linears - each what one call of
// the reference's entry point would compute (kernels/TernaSpMM.cu:25-71 of
// Gu-J/TernaInfer: decode SpMM + split-K reduction + scale epilogue) - and runs
// them back to back without any of that: one CTA per SM stays resident, builds
// the two decode tables once, and every warp walks the whole list with ONE
// register pipeline (bitmap words two tiles ahead, sign words one tile ahead)
// that keeps running across item boundaries, so the HBM stream never drains.
//
// Work split per item: its row tiles x k-tiles, in that order, are cut into
// one contiguous chunk per CTA (balanced to a tile), a chunk is dealt to the
// CTA's warps round robin.  Partial sums meet in three steps, none of which
// stops the decode of later tiles:
//   warp   registers, across the k-tiles of one row tile;
//   CTA    shared-memory atomics into one of 4 x 4 slots (4 items in flight x
//          up to 4 row tiles of an item per CTA); the last warp to contribute
//          to a slot pushes it on;
//   chip   red.global.add into an int32 accumulator ring in the scratch area
//          (4 items deep); the last CTA to arrive for a row tile reads the sums
//          back, applies the scale epilogue (and optional residual), stores
//          bf16 and re-zeroes what it used.
// Every wait in here is a bounded spin that ends the launch with status 4.
// The items of a list must be independent of each other: an item may not read
// what another item of the same list writes.
#pragma once
#include <cuda_bf16.h>

#include "spmm_small_m.cuh"

namespace tsp {

constexpr int kListMaxItems = 256;     // items per launch (the table is staged in shared memory)
constexpr int kListRing = 4;           // items whose chip-wide accumulators may be in flight
constexpr int kListSlots = 4;          // row tiles of one item that one CTA's chunk may touch
constexpr int kListMaxRT = 296;        // row tiles per item (wider layers are split into several items by the host)
constexpr int kListSpin = 1 << 22;     // iteration limit of the (rare) waits

struct ListItem {                      // 128 bytes, device memory
    const int8_t* x;
    const uint32_t* bitmap;
    const int* tile_off;
    const uint16_t* quarter_off;
    const uint32_t* signs;
    __nv_bfloat16* out;                // first column of this item's rows: out[t * ld_out + n]
    const __nv_bfloat16* s;
    const __nv_bfloat16* ws;
    const __nv_bfloat16* residual;     // same indexing as out, or null
    int M, N, K, ld_out;               // N = output rows of this item (a multiple of 64)
    int n0;                            // column of the full layer where this item starts (scale segments use layer columns)
    int ws_num, epilogue, seg_gran;
    int seg_b[3];
    int layer_n;                       // output width of the full layer (unused by the kernel)
    int pad[2];
};
static_assert(sizeof(ListItem) == 128, "ListItem is staged as eight 16-byte words");

struct ListScratch {                   // head of the scratch area; the accumulator ring follows
    unsigned int abort;
    unsigned int ctas_done;
    unsigned int pad[2];
    unsigned int item_done[kListMaxItems];               // row tiles of item i whose outputs are stored
    unsigned int rt_count[kListRing][kListMaxRT];        // CTAs that have pushed their share of a row tile
};

struct ItemAux {                       // per item and CTA, derived once
    int t0, n, rtA, need;              // first tile and tile count of this CTA's chunk, its first row tile,
};                                     // slots of earlier items that share this item's slot set

template <int MT>
struct ListSmem {
    static constexpr int lut1 = 0;                                      // the 2 x 256 table entries, one copy
    static constexpr int items = 2048;
    static constexpr int aux = items + kListMaxItems * 128;
    static constexpr int slots = aux + kListMaxItems * 16;              // int32 [4 sets][4 slots][MT*8][kRedStride]
    static constexpr int slot_ints = MT * 8 * kRedStride;
    static constexpr int counts = slots + kListRing * kListSlots * slot_ints * 4;   // uint [4][4] warps arrived
    static constexpr int flushed = counts + 64;                         // uint [4] slots flushed per set (cumulative)
    static constexpr int rest = (flushed + 16 + 127) / 128 * 128;
    static constexpr int total = kLut2Bytes + kLutBytes + rest;
};

// A tile of a warp's sequence, packed into one register: item << 24 | row tile << 12 | k-tile
// (at most 256 items, 296 row tiles, 4095 k-tiles); all ones: the sequence is exhausted.
struct TileRef {
    uint32_t v;
    __device__ __forceinline__ bool valid() const { return v != 0xFFFFFFFFu; }
    __device__ __forceinline__ int item() const { return (int)(v >> 24); }
    __device__ __forceinline__ int rt() const { return (int)((v >> 12) & 0xFFFu); }
    __device__ __forceinline__ int kt() const { return (int)(v & 0xFFFu); }
    __device__ __forceinline__ uint32_t item_rt() const { return v >> 12; }
};

struct ListCursor {
    int item, j, n, rt, kt, KT;
};

// Next tile of this warp: tiles warp, warp + W, ... of the CTA's chunk of the current item, then on
// to the next item with a non-empty share.
template <int W>
__device__ __forceinline__ TileRef list_next(ListCursor& c, const ListItem* items, const ItemAux* aux, int n_items, int warp) {
    c.j += W;
    c.kt += W;
    while (c.j >= c.n) {
        if (++c.item >= n_items) {
            c.item = n_items, c.j = 0, c.n = 0;
            return {0xFFFFFFFFu};
        }
        const ItemAux ax = aux[c.item];
        c.n = ax.n, c.j = warp;
        if (warp < ax.n) {
            c.KT = items[c.item].K >> 6;
            const int tile = ax.t0 + warp;
            c.rt = tile / c.KT, c.kt = tile - c.rt * c.KT;
        }
    }
    while (c.kt >= c.KT) c.kt -= c.KT, ++c.rt;
    return {((uint32_t)c.item << 24) | ((uint32_t)c.rt << 12) | (uint32_t)c.kt};
}

__device__ __forceinline__ TileHead list_load_head(const ListItem* items, const TileRef& r, int lane) {
    TileHead h;
    h.bw = make_uint4(0, 0, 0, 0), h.toff = 0, h.qbase = 0;
    if (r.valid()) {
        const ListItem& it = items[r.item()];
        const long long tile = (long long)r.rt() * (it.K >> 6) + r.kt();
        h.bw = __ldg(reinterpret_cast<const uint4*>(it.bitmap + tile * 128) + lane);
        h.toff = __ldg(it.tile_off + tile);
        const int qd = lane >> 3;
        h.qbase = qd ? (int)__ldg(it.quarter_off + 3 * tile + qd - 1) : 0;
    }
    return h;
}

__device__ __forceinline__ TileSigns list_load_signs(const ListItem* items, const TileRef& r, const TileHead& h, int lane) {
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
    const bool valid = r.valid();
    const uint32_t* signs = valid ? items[r.item()].signs : nullptr;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        sg.lo[i] = valid ? __ldg(signs + (pos >> 5)) : 0u;
        sg.hi[i] = valid ? __ldg(signs + (pos >> 5) + 1) : 0u;
        pos += cn[i];
    }
    return sg;
}

__device__ __forceinline__ int list_ws_group(int col, const ListItem& it) {
    const int c = col & ~(it.seg_gran - 1);
    const int g = (c >= it.seg_b[0]) + (c >= it.seg_b[1]) + (c >= it.seg_b[2]);
    const int limit = (it.epilogue == EPI_PREFILL || it.seg_gran == 1) ? it.ws_num - 1 : 3;
    return max(min(g, limit), 0);
}

// Bounded wait until *p >= want; gives up early when another warp has already given up.
__device__ __forceinline__ bool list_wait_ge(const volatile unsigned int* p, unsigned int want,
                                             const volatile unsigned int* abort_flag) {
    for (int i = 0; i < kListSpin; ++i) {
        if (*p >= want) return true;
        if ((i & 1023) == 1023 && *abort_flag) return false;
        __nanosleep(64);
    }
    return false;
}

template <int MT, int W>
__global__ void __launch_bounds__(W * 32, 1) spmm_list_kernel(const ListItem* __restrict__ items_g, int n_items,
                                                             uint8_t* __restrict__ scratch, int acc_ld, int* status) {
    using L = ListSmem<MT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t dyn = (smem_u32(smem) + 127u) & ~127u;
    const uint32_t lut_base = (dyn + (uint32_t)kLutBytes - 1u) & ~((uint32_t)kLutBytes - 1u);
    const uint32_t sbase = (lut_base - dyn >= (uint32_t)L::rest) ? dyn : lut_base + kLut2Bytes;
    uint8_t* rest = smem + (sbase - smem_u32(smem));
    ListItem* items = reinterpret_cast<ListItem*>(rest + L::items);
    ItemAux* aux = reinterpret_cast<ItemAux*>(rest + L::aux);
    int* slots = reinterpret_cast<int*>(rest + L::slots);
    unsigned int* counts = reinterpret_cast<unsigned int*>(rest + L::counts);
    volatile unsigned int* flushed = reinterpret_cast<volatile unsigned int*>(rest + L::flushed);
    ListScratch* sc = reinterpret_cast<ListScratch*>(scratch);
    int* acc_g = reinterpret_cast<int*>(scratch + sizeof(ListScratch));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int cta = blockIdx.x, G = gridDim.x;

    griddep_launch_dependents();
    // ---- set-up, once per launch: item table, per-item shares of this CTA, decode tables, slots
    for (int i = tid; i < n_items * 8; i += W * 32)
        reinterpret_cast<uint4*>(items)[i] = __ldg(reinterpret_cast<const uint4*>(items_g) + i);
    for (int e = tid; e < 512; e += W * 32)
        reinterpret_cast<uint32_t*>(rest + L::lut1)[e] = e < 256 ? lut_entry(e) : lut_entry_upper(e - 256);
    for (int i = tid; i < kListRing * kListSlots * L::slot_ints; i += W * 32) slots[i] = 0;
    if (tid < 16) counts[tid] = 0;
    if (tid < 4) flushed[tid] = 0;
    __syncthreads();
    for (int i = tid; i < 512 * 8; i += W * 32) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(rest + L::lut1)[i >> 3];
        sts128(lut_base + i * 16, make_uint4(v, v, v, v));
    }
    for (int i = tid; i < n_items; i += W * 32) {
        const int KT = items[i].K >> 6;
        const long long T = (long long)(items[i].N >> 6) * KT;
        const int Gi = (int)(T < G ? T : G);
        ItemAux ax = {0, 0, 0, 0};
        if (cta < Gi) {
            ax.t0 = (int)(T * cta / Gi);
            ax.n = (int)(T * (cta + 1) / Gi) - ax.t0;
            ax.rtA = ax.t0 / KT;
        }
        aux[i] = ax;
    }
    __syncthreads();
    if (tid == 0) {   // slots of earlier items in the same slot set (cumulative, per set)
        int cum[kListRing] = {0, 0, 0, 0};
        for (int i = 0; i < n_items; ++i) {
            const int KT = items[i].K >> 6;
            aux[i].need = cum[i & 3];
            if (aux[i].n > 0) cum[i & 3] += (aux[i].t0 + aux[i].n - 1) / KT - aux[i].rtA + 1;
        }
    }
    __syncthreads();

    const uint32_t lut_lo = lut_base | (uint32_t)(lane * 4), lut_hi = lut_lo + kLutBytes;
    ListCursor cur = {-1, 0, 0, 0, 0, 1};
    TileRef r0 = list_next<W>(cur, items, aux, n_items, warp);
    TileHead h0 = list_load_head(items, r0, lane);
    TileRef r1 = list_next<W>(cur, items, aux, n_items, warp);
    TileHead h1 = list_load_head(items, r1, lane);
    TileSigns s0 = list_load_signs(items, r0, h0, lane);

    int acc[4][MT][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][mt][c] = 0;

    griddep_wait();   // activations, scales, residuals and outputs may belong to the previous kernel
    bool ok = true;

    while (r0.valid() && ok) {
        const TileRef r2 = list_next<W>(cur, items, aux, n_items, warp);
        const TileHead h2 = list_load_head(items, r2, lane);
        const TileSigns s1 = list_load_signs(items, r1, h1, lane);
        const int item = r0.item(), rt = r0.rt();
        const ListItem& it = items[item];
        uint4 bx[MT];
        load_x_frags<MT>(bx, it.x, it.K, 0, it.M, r0.kt(), g, q);
        uint32_t a[4][8];
        decode_tile(h0, s0, lut_lo, lut_hi, a);
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_s8_16x8x32(acc[r][mt], a[r][0], a[r][1], a[r][2], a[r][3], bx[mt].x, bx[mt].y);
                mma_s8_16x8x32(acc[r][mt], a[r][4], a[r][5], a[r][6], a[r][7], bx[mt].z, bx[mt].w);
            }

        if (r1.item_rt() != r0.item_rt()) {
            // ---- this warp leaves row tile rt of this item: hand its partial sums on
            const ItemAux ax = aux[item];
            const int set = item & 3, slot = rt - ax.rtA;
            const int KT = it.K >> 6;
            int* sl = slots + (set * kListSlots + slot) * L::slot_ints;
            if (flushed[set] < (unsigned int)ax.need) ok = list_wait_ge(flushed + set, (unsigned int)ax.need, &sc->abort);
            __threadfence_block();
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int v = acc[r][mt][c];
                        if (v != 0) atomicAdd(&sl[(mt * 8 + 2 * q + (c & 1)) * kRedStride + 16 * r + g + 8 * (c >> 1)], v);
                        acc[r][mt][c] = 0;
                    }
            __syncwarp();
            // warps of this CTA with tiles in this row tile: the chunk's tiles ja .. jb-1, dealt round robin
            const int ja = max(0, rt * KT - ax.t0), jb = min(ax.n, (rt + 1) * KT - ax.t0);
            unsigned int prev = 0;
            if (lane == 0) {
                __threadfence_block();
                prev = atomicAdd(&counts[set * kListSlots + slot], 1u);
            }
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if ((int)prev == min(W, jb - ja) - 1 && ok) {
                // ---- last warp of the CTA for this slot: push it to the chip-wide accumulators
                __threadfence_block();
                const int ring = item & (kListRing - 1);
                if (item >= kListRing) {   // the ring entry's previous user must be completely stored
                    const unsigned int want = (unsigned int)(items[item - kListRing].N >> 6);
                    if (*(volatile unsigned int*)&sc->item_done[item - kListRing] < want)
                        ok = list_wait_ge(&sc->item_done[item - kListRing], want, &sc->abort);
                    __threadfence();
                }
                int* ag = acc_g + (size_t)ring * 16 * acc_ld + rt * 64;
                if (ok) {
#pragma unroll 4
                    for (int i = lane; i < MT * 8 * 64; i += 32) {
                        const int t = i >> 6, c = i & 63;
                        const int v = sl[t * kRedStride + c];
                        if (v != 0) {
                            atomicAdd(ag + (size_t)t * acc_ld + c, v);
                            sl[t * kRedStride + c] = 0;
                        }
                    }
                }
                __threadfence();
                __syncwarp();
                // CTAs whose chunks reach into this row tile
                const long long T = (long long)(it.N >> 6) * KT;
                const int Gi = (int)(T < G ? T : G);
                const long long lo = (long long)rt * KT, hi = lo + KT;
                const int cA = (int)(((lo + 1) * Gi + T - 1) / T) - 1, cB = (int)((hi * Gi + T - 1) / T) - 1;
                unsigned int prevg = 0;
                if (lane == 0) {
                    counts[set * kListSlots + slot] = 0;
                    __threadfence_block();
                    atomicAdd((unsigned int*)&flushed[set], 1u);
                    prevg = atomicAdd(&sc->rt_count[ring][rt], 1u);
                }
                prevg = __shfl_sync(0xffffffffu, prevg, 0);
                if ((int)prevg == cB - cA && ok) {
                    // ---- last CTA for this row tile: scale epilogue, store, re-zero
                    __threadfence();
                    const int n_base = rt * 64;
#pragma unroll 2
                    for (int i = lane; i < it.M * 64; i += 32) {
                        const int t = i >> 6, c = i & 63;
                        int* src = ag + (size_t)t * acc_ld + c;
                        int v;
                        asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
                        *src = 0;
                        const float s_el = __bfloat162float(it.s[t]);
                        const float ws_el = __bfloat162float(it.ws[list_ws_group(it.n0 + n_base + c, it)]);
                        const long long o = (long long)t * it.ld_out + n_base + c;
                        it.out[o] = add_residual(scale_epilogue(v, s_el, ws_el, it.epilogue), it.residual, o);
                    }
                    // rows of the ring entry beyond M were never touched; those below M are zero again
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) {
                        sc->rt_count[ring][rt] = 0;
                        __threadfence();
                        atomicAdd(&sc->item_done[item], 1u);
                    }
                }
            }
            ok = __all_sync(0xffffffffu, ok);
        }
        r0 = r1, h0 = h1, s0 = s1;
        r1 = r2, h1 = h2;
    }
    if (!ok) {
        if (lane == 0) {
            atomicExch(&sc->abort, 1u);
            atomicExch(status, ST_WAIT_TIMEOUT);
        }
    }
    // ---- the last CTA to finish re-arms the scratch area for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned int prev = atomicAdd(&sc->ctas_done, 1u);
        if (prev == (unsigned int)G - 1) {
            __threadfence();
            for (int i = 0; i < n_items; ++i) sc->item_done[i] = 0;
            sc->ctas_done = 0;
            __threadfence();
        }
    }
}

}  // namespace tsp
