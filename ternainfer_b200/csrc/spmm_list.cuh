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
// the two decode tables once, and every warp walks its share of the whole list
// with ONE register pipeline (bitmap words two tiles ahead, sign words one tile
// ahead) that keeps running across row tiles and items, so the HBM stream never
// drains.
//
// Work split.  All 64x64 tiles of the list form one sequence (item by item, row
// tile by row tile, k-tile by k-tile); every CTA takes one contiguous share of
// it, equal to a tile, and deals its share to its warps round robin, so every
// warp of the chip decodes the same number of tiles (+-1).  A row tile that lies
// inside one CTA's share - all of them except at most two per CTA - never leaves
// the SM: warps add their partial sums into one of eight shared-memory slots
// (row tiles in flight); the last decoder warp to arrive only marks the slot
// complete, and a dedicated EPILOGUE WARP (one per CTA, it decodes nothing) turns
// complete slots into bf16 stores.  Were the last arriver to run the epilogue,
// the slowest warp would collect every epilogue, fall further behind and pace
// the whole CTA (measured: a third of the warps asleep in the slot-reuse wait,
// 660 GB/s instead of 1140); letting decoder warps pick epilogues up at their
// own row-tile ends needs calls in the decode loop that cost it its registers.  A row tile cut by a share boundary is summed
// across the CTAs that hold its pieces through a small int32 area in the scratch
// memory (red.global.add); the last CTA to arrive reads the sums back, runs the
// epilogue and re-zeroes what it used.  Nothing in the kernel is a barrier
// between items: warps run on into the next row tile or item at once.
// The few waits (reuse of a slot) are bounded spins that end the launch with
// status 4.  The items of a list must be independent of each other: an item may
// not read what another item of the same list writes.
#pragma once
#include <cuda_bf16.h>

#include "spmm_small_m.cuh"

namespace tsp {

constexpr int kListMaxItems = 256;     // entries per launch (the table is staged in shared memory)
constexpr int kListSlots = 8;          // row tiles in flight per CTA
constexpr int kListMaxCtas = 1024;     // boundary areas in the scratch memory
constexpr int kListSpin = 1 << 22;     // iteration limit of the (rare) waits

struct ListItem {                      // 128 bytes, device memory
    const int8_t* x;
    const uint32_t* bitmap;
    const int* tile_off;
    const uint16_t* quarter_off;
    const uint32_t* signs;
    __nv_bfloat16* out;                // out[t * ld_out + n]
    const __nv_bfloat16* s;
    const __nv_bfloat16* ws;
    const __nv_bfloat16* residual;     // same indexing as out, or null
    int M, N, K, ld_out;               // N = output rows (a multiple of 64, at most 4095 * 64)
    int ws_num, epilogue, seg_gran;
    int seg_b[3];
    int pad[2];
    long long tile_base;               // tiles of all earlier entries
};
static_assert(sizeof(ListItem) == 128, "ListItem is staged as eight 16-byte words");

struct ListScratch {                   // head of the scratch area; one 16 x 64 int32 area per CTA follows
    unsigned int abort;
    unsigned int pad[3];
    unsigned int arrived[kListMaxCtas];    // CTAs that have pushed their piece of the row tile cut at a boundary
};
constexpr int kListAreaInts = 16 * 64;

#ifdef TSP_TUNING
// Tuning builds only: bit mask of stages to leave out, for cost accounting with the profiler's
// instruction counters (results are wrong by design): 1 decode, 2 sign loads, 4 slot atomics, 8 x + MMA.
__device__ int g_list_ablate = 0;
#define LIST_ABLATE(bit) (g_list_ablate & (bit))
#else
#define LIST_ABLATE(bit) 0
#endif

struct ListShare {                     // this CTA's share of the tile sequence, derived once per launch
    int item0, rt0, kt0;               // its first tile
    int n;                             // tiles
    int last_s;                        // index (within the share) of its last row tile
    int first_cnt, last_cnt;           // warps that hold tiles of the first / last row tile of the share
    int first_cut, last_cut;           // the first / last row tile is cut by a share boundary
};

template <int MT>
struct ListSmem {
    static constexpr int lut1 = 0;                                      // the 2 x 256 table entries, one copy
    static constexpr int share = 2048;
    static constexpr int items = share + 64;
    static constexpr int slot_ints = MT * 8 * kRedStride;
    static constexpr int slots = items + kListMaxItems * 128;           // int32 [kListSlots][MT*8][kRedStride]
    static constexpr int counts = slots + kListSlots * slot_ints * 4;   // uint [kListSlots] warps arrived
    static constexpr int gens = counts + kListSlots * 4;                // uint [kListSlots] times a slot was finished
    static constexpr int ready = gens + kListSlots * 4;                 // uint [kListSlots] 1: all partial sums are in, 2: claimed
    static constexpr int info = ready + kListSlots * 4;                 // uint [kListSlots] item << 13 | row tile << 1 | cut
    static constexpr int rest = (info + kListSlots * 4 + 127) / 128 * 128;
    static constexpr int total = kLut2Bytes + kLutBytes + rest;
};

// A tile of a warp's sequence: item << 24 | row tile << 12 | k-tile in one register (at most 256
// entries, 4095 row tiles and 4095 k-tiles each; all ones: the sequence is exhausted), and the index
// of its row tile within the CTA's share.
struct TileRef {
    uint32_t v;
    int s;
    __device__ __forceinline__ bool valid() const { return v != 0xFFFFFFFFu; }
    __device__ __forceinline__ int item() const { return (int)(v >> 24); }
    __device__ __forceinline__ int rt() const { return (int)((v >> 12) & 0xFFFu); }
    __device__ __forceinline__ int kt() const { return (int)(v & 0xFFFu); }
};

struct ListCursor {
    int item, rt, kt, s, left;         // position of the warp's next tile; tiles of the share not yet passed
    int KT, RT;                        // of the current item
};

// Tile `step` positions further along the CTA's share.
__device__ __forceinline__ TileRef list_advance(ListCursor& c, const ListItem* items, int step) {
    c.left -= step;
    if (c.left <= 0) return {0xFFFFFFFFu, 0};
    c.kt += step;
    while (c.kt >= c.KT) {
        c.kt -= c.KT;
        ++c.s;
        if (++c.rt >= c.RT) {
            ++c.item, c.rt = 0;
            c.KT = items[c.item].K >> 6, c.RT = items[c.item].N >> 6;
        }
    }
    return {((uint32_t)c.item << 24) | ((uint32_t)c.rt << 12) | (uint32_t)c.kt, c.s};
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

// Scale epilogue of one 64-column row tile by one warp.  `get(i)` returns accumulator i = t * 64 + c
// (and clears its source).  Every load - accumulators, token scales, weight scales, residuals - is
// issued before the first store: the output may alias any of them as far as the compiler knows, so a
// store in between would serialise the L2 round trips of the loads behind it (measured: 11 us per
// row tile instead of 1).
template <int MT, typename Get>
__device__ __forceinline__ void list_epilogue(const ListItem& it, int rt, int lane, Get get) {
    constexpr int NV = 2 * MT * 8;     // values per lane: i = lane + 32 k, token t = k / 2, column c = lane + 32 (k & 1)
    const int n_base = rt * 64;
    int v[NV];
    float s_el[MT * 8], ws_el[2];
    __nv_bfloat16 res[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) v[k] = (lane + 32 * k) < it.M * 64 ? get(lane + 32 * k) : 0;
#pragma unroll
    for (int t = 0; t < MT * 8; ++t) s_el[t] = t < it.M ? __bfloat162float(it.s[t]) : 1.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) ws_el[h] = __bfloat162float(it.ws[list_ws_group(n_base + lane + 32 * h, it)]);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const long long o = (long long)(k >> 1) * it.ld_out + n_base + lane + 32 * (k & 1);
        res[k] = (it.residual && (k >> 1) < it.M) ? it.residual[o] : __float2bfloat16_rn(0.f);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        if ((k >> 1) < it.M) {
            const long long o = (long long)(k >> 1) * it.ld_out + n_base + lane + 32 * (k & 1);
            __nv_bfloat16 r = scale_epilogue(v[k], s_el[k >> 1], ws_el[k & 1], it.epilogue);
            if (it.residual) r = __float2bfloat16_rn(__bfloat162float(res[k]) + __bfloat162float(r));
            it.out[o] = r;
        }
    }
}

// The last warp of a CTA to contribute to a row tile finishes it.  Kept out of line: it runs once per
// row tile and CTA, and its registers must not weigh on the decode loop.
// Whole row tile summed on this SM: epilogue straight from the shared-memory slot.
template <int MT>
__device__ __noinline__ void list_finish_local(const ListItem* it, int rt, int lane, int* sl) {
    list_epilogue<MT>(*it, rt, lane, [&](int i) {
        int* p = sl + (i >> 6) * kRedStride + (i & 63);
        const int v = *p;
        *p = 0;
        return v;
    });
}

// A piece of a row tile that other CTAs share: add it to the scratch area of the first of them; the
// last CTA to arrive reads the sums back, runs the epilogue and re-zeroes area and counter.
template <int MT>
__device__ __noinline__ void list_finish_cut(const ListItem* it, int rt, int lane, int* sl, ListScratch* sc, int* areas,
                                             int Gi, long long Ttot) {
    const int KT = it->K >> 6;
    const long long t0g = it->tile_base + (long long)rt * KT;              // the row tile's first tile
    const int cA = (int)(((t0g + 1) * Gi + Ttot - 1) / Ttot) - 1;          // CTAs whose shares reach into it
    const int cB = (int)(((t0g + KT) * Gi + Ttot - 1) / Ttot) - 1;
    int* area = areas + (size_t)cA * kListAreaInts;
#pragma unroll 4
    for (int i = lane; i < MT * 8 * 64; i += 32) {
        int* p = sl + (i >> 6) * kRedStride + (i & 63);
        const int v = *p;
        if (v != 0) {
            atomicAdd(area + i, v);
            *p = 0;
        }
    }
    __threadfence();
    __syncwarp();
    unsigned int prevg = 0;
    if (lane == 0) prevg = atomicAdd(&sc->arrived[cA], 1u);
    prevg = __shfl_sync(0xffffffffu, prevg, 0);
    if ((int)prevg == cB - cA) {
        __threadfence();
        list_epilogue<MT>(*it, rt, lane, [&](int i) {
            const int v = __ldcg(area + i);
            area[i] = 0;
            return v;
        });
        __threadfence();
        __syncwarp();
        if (lane == 0) sc->arrived[cA] = 0;
    }
}

// Bounded wait of a decoder warp until *p >= want (a shared-memory counter that the epilogue warp
// advances); gives up early when another warp has already given up.
__device__ __forceinline__ bool list_wait_ge(const volatile unsigned int* p, unsigned int want,
                                             const volatile unsigned int* abort_flag) {
    for (int i = 0; i < kListSpin; ++i) {
        if (*p >= want) return true;
        if ((i & 1023) == 1023 && *abort_flag) return false;
        __nanosleep(32);
    }
    return false;
}

// The epilogue warp: finishes complete row tiles until all `total` row tiles of the share are done.
template <int MT>
__device__ __forceinline__ bool list_epilogue_warp(unsigned int total, const ListItem* items, int* slots, unsigned int* counts,
                                                   volatile unsigned int* gens, volatile unsigned int* ready,
                                                   volatile unsigned int* info, ListScratch* sc, int* areas, int Gi,
                                                   long long Ttot, int lane) {
    using L = ListSmem<MT>;
    unsigned int finished = 0;
    int idle = 0;
    while (finished < total) {
        const unsigned int mask = __ballot_sync(0xffffffffu, lane < kListSlots && ready[lane & (kListSlots - 1)] == 1u);
        if (mask == 0) {
            if (++idle >= kListSpin) return false;
            if ((idle & 1023) == 1023) {
                unsigned int ab = 0;
                if (lane == 0) ab = *(volatile unsigned int*)&sc->abort;
                if (__shfl_sync(0xffffffffu, ab, 0)) return false;
            }
            __nanosleep(32);
            continue;
        }
        idle = 0;
        const int slot = __ffs(mask) - 1;
        __threadfence_block();
        const unsigned int inf = info[slot];
        const ListItem* it = items + (inf >> 13);
        const int rt = (int)((inf >> 1) & 0xFFFu);
        int* sl = slots + slot * L::slot_ints;
        if (inf & 1u) list_finish_cut<MT>(it, rt, lane, sl, sc, areas, Gi, Ttot);
        else list_finish_local<MT>(it, rt, lane, sl);
        __threadfence_block();
        __syncwarp();
        if (lane == 0) {
            counts[slot] = 0;
            ready[slot] = 0;
            __threadfence_block();
            atomicAdd((unsigned int*)&gens[slot], 1u);
        }
        __syncwarp();
        ++finished;
    }
    return true;
}

// WT warps per CTA: WT - 1 decoder warps and the epilogue warp (registers are allotted per four warps,
// so the warp count is kept a multiple of four).
template <int MT, int WT>
__global__ void __launch_bounds__(WT * 32, 1) spmm_list_kernel(const ListItem* __restrict__ items_g, int n_items,
                                                             uint8_t* __restrict__ scratch, int* status) {
    using L = ListSmem<MT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t dyn = (smem_u32(smem) + 127u) & ~127u;
    const uint32_t lut_base = (dyn + (uint32_t)kLutBytes - 1u) & ~((uint32_t)kLutBytes - 1u);
    const uint32_t sbase = (lut_base - dyn >= (uint32_t)L::rest) ? dyn : lut_base + kLut2Bytes;
    uint8_t* rest = smem + (sbase - smem_u32(smem));
    ListItem* items = reinterpret_cast<ListItem*>(rest + L::items);
    ListShare* share = reinterpret_cast<ListShare*>(rest + L::share);
    int* slots = reinterpret_cast<int*>(rest + L::slots);
    unsigned int* counts = reinterpret_cast<unsigned int*>(rest + L::counts);
    volatile unsigned int* gens = reinterpret_cast<volatile unsigned int*>(rest + L::gens);
    volatile unsigned int* ready = reinterpret_cast<volatile unsigned int*>(rest + L::ready);
    volatile unsigned int* info = reinterpret_cast<volatile unsigned int*>(rest + L::info);
    ListScratch* sc = reinterpret_cast<ListScratch*>(scratch);
    int* areas = reinterpret_cast<int*>(scratch + sizeof(ListScratch));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int cta = blockIdx.x, G = gridDim.x;

    griddep_launch_dependents();
    // ---- set-up, once per launch: item table, this CTA's share, decode tables, slots
    constexpr int W = WT - 1;          // decoder warps
    constexpr int NT = WT * 32;
    for (int i = tid; i < n_items * 8; i += NT)
        reinterpret_cast<uint4*>(items)[i] = __ldg(reinterpret_cast<const uint4*>(items_g) + i);
    for (int e = tid; e < 512; e += NT)
        reinterpret_cast<uint32_t*>(rest + L::lut1)[e] = e < 256 ? lut_entry(e) : lut_entry_upper(e - 256);
    for (int i = tid; i < kListSlots * L::slot_ints; i += NT) slots[i] = 0;
    if (tid < kListSlots) counts[tid] = 0, gens[tid] = 0, ready[tid] = 0, info[tid] = 0;
    __syncthreads();
    for (int i = tid; i < 512 * 8; i += NT) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(rest + L::lut1)[i >> 3];
        sts128(lut_base + i * 16, make_uint4(v, v, v, v));
    }
    const ListItem& last_item = items[n_items - 1];
    const long long Ttot = last_item.tile_base + (long long)(last_item.N >> 6) * (last_item.K >> 6);
    const int Gi = (int)(Ttot < G ? Ttot : G);      // CTAs that get a share (all of them unless the list is tiny)
    if (tid == 0) {
        ListShare sh = {0, 0, 0, 0, 0, 0, 0, 0, 0};
        if (cta < Gi) {
            const long long b0 = Ttot * cta / Gi, b1 = Ttot * (cta + 1) / Gi;
            int i = 0;
            while (i + 1 < n_items && items[i + 1].tile_base <= b0) ++i;
            const int KT = items[i].K >> 6;
            const long long off = b0 - items[i].tile_base;
            sh.item0 = i, sh.rt0 = (int)(off / KT), sh.kt0 = (int)(off - (long long)sh.rt0 * KT), sh.n = (int)(b1 - b0);
            // first row tile: tiles kt0 .. KT-1 of it (or fewer when the share ends inside it)
            const int first_len = min(KT - sh.kt0, sh.n);
            sh.first_cnt = min(W, first_len);
            sh.first_cut = (sh.kt0 > 0 || first_len < KT - sh.kt0) ? 1 : 0;
            // last row tile: walk to the share's last tile
            int it2 = i, rt2 = sh.rt0, s2 = 0;
            long long rem = (long long)sh.n - first_len;   // tiles after the first row tile
            int last_len = first_len, last_full = KT - sh.kt0;
            while (rem > 0) {
                if (++rt2 >= (items[it2].N >> 6)) ++it2, rt2 = 0;
                ++s2;
                const int kt_n = items[it2].K >> 6;
                last_len = (int)(rem < kt_n ? rem : kt_n), last_full = kt_n;
                rem -= last_len;
            }
            sh.last_s = s2, sh.last_cnt = min(W, last_len);
            sh.last_cut = s2 == 0 ? sh.first_cut : (last_len < last_full ? 1 : 0);
        }
        *share = sh;
    }
    __syncthreads();
    const ListShare sh = *share;

    if (warp == W) {
        // ---- the epilogue warp
        griddep_wait();   // scales, residuals and outputs may belong to the previous kernel
        if (sh.n > 0 && !list_epilogue_warp<MT>((unsigned int)sh.last_s + 1u, items, slots, counts, gens, ready, info, sc, areas, Gi,
                                                Ttot, lane) && lane == 0) {
            atomicExch(&sc->abort, 1u);
            atomicExch(status, ST_WAIT_TIMEOUT);
        }
        return;
    }

    const uint32_t lut_lo = lut_base | (uint32_t)(lane * 4), lut_hi = lut_lo + kLutBytes;
    ListCursor cur;
    cur.item = sh.item0, cur.rt = sh.rt0, cur.kt = sh.kt0, cur.s = 0, cur.left = sh.n;
    cur.KT = items[sh.item0].K >> 6, cur.RT = items[sh.item0].N >> 6;
    TileRef r0 = list_advance(cur, items, warp);   // the warp's first tile: number `warp` of the share (if it has that many)
    TileHead h0 = list_load_head(items, r0, lane);
    TileRef r1 = list_advance(cur, items, W);
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

    while (r0.valid()) {
        const TileRef r2 = list_advance(cur, items, W);
        const TileHead h2 = list_load_head(items, r2, lane);
        TileSigns s1 = s0;
        if (!LIST_ABLATE(2)) s1 = list_load_signs(items, r1, h1, lane);
        const int item = r0.item(), rt = r0.rt();
        const ListItem& it = items[item];
        uint4 bx[MT];
        if (!LIST_ABLATE(8)) load_x_frags<MT>(bx, it.x, it.K, 0, it.M, r0.kt(), g, q);
        uint32_t a[4][8];
        if (!LIST_ABLATE(1)) {
            decode_tile(h0, s0, lut_lo, lut_hi, a);
        } else {
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int j = 0; j < 8; ++j) a[r][j] = h0.bw.x ^ (uint32_t)(r * 8 + j) ^ s0.lo[r];
        }
        if (!LIST_ABLATE(8)) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_s8_16x8x32(acc[r][mt], a[r][0], a[r][1], a[r][2], a[r][3], bx[mt].x, bx[mt].y);
                    mma_s8_16x8x32(acc[r][mt], a[r][4], a[r][5], a[r][6], a[r][7], bx[mt].z, bx[mt].w);
                }
        } else {
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[r][0][0] += (int)(a[r][0] ^ a[r][1] ^ a[r][2] ^ a[r][3] ^ a[r][4] ^ a[r][5] ^ a[r][6] ^ a[r][7]);
        }

        if (!r1.valid() || r1.s != r0.s) {
            // ---- this warp leaves row tile number r0.s of the share: hand its partial sums on
            const int slot = r0.s & (kListSlots - 1);
            const unsigned int gen = (unsigned int)(r0.s / kListSlots);      // earlier row tiles that used this slot
            int* sl = slots + slot * L::slot_ints;
            if (gens[slot] < gen) ok = list_wait_ge(gens + slot, gen, &sc->abort);   // rare: eight row tiles ahead
            ok = __all_sync(0xffffffffu, ok);     // lanes may leave the wait on different sides of its limit
            if (!ok) break;
            __threadfence_block();
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int v = acc[r][mt][c];
                        if (v != 0 && !LIST_ABLATE(4))
                            atomicAdd(&sl[(mt * 8 + 2 * q + (c & 1)) * kRedStride + 16 * r + g + 8 * (c >> 1)], v);
                        acc[r][mt][c] = 0;
                    }
            __syncwarp();
            const int KT = it.K >> 6;
            const int expected = r0.s == 0 ? sh.first_cnt : (r0.s == sh.last_s ? sh.last_cnt : min(W, KT));
            const bool cut = (r0.s == 0 && sh.first_cut) || (r0.s == sh.last_s && sh.last_cut);
            unsigned int prev = 0;
            if (lane == 0) {
                __threadfence_block();
                prev = atomicAdd(&counts[slot], 1u);
            }
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if ((int)prev == expected - 1 && lane == 0) {
                // last decoder warp of the CTA for this row tile: all partial sums are in the slot
                info[slot] = ((unsigned int)item << 13) | ((unsigned int)rt << 1) | (cut ? 1u : 0u);
                __threadfence_block();
                ready[slot] = 1;
            }
        }
        r0 = r1, h0 = h1, s0 = s1;
        r1 = r2, h1 = h2;
    }
    if (!ok && lane == 0) {
        atomicExch(&sc->abort, 1u);
        atomicExch(status, ST_WAIT_TIMEOUT);
    }
}

}  // namespace tsp
