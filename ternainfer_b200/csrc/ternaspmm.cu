// libternaspmm.so for NVIDIA B200 (sm_100a): the extern "C" surface declared
// in include/ternaspmm.h and the host-side launch logic behind it.
//
// The entry points mirror kernels/TernaSpMM.cu of Gu-J/TernaInfer (same names,
// argument order and meaning); everything behind them is new.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <limits.h>
#include <stdlib.h>

#include <algorithm>
#include <vector>

#define TERNASPMM_TYPES_ONLY   // the item struct of the work lists; the prototypes use plain-C stand-in types
#include "ternaspmm.h"

#include "act_quant.cuh"
#include "dense_pair.cuh"
#include "dense_prefill.cuh"
#include "lm_head.cuh"
#include "mma_rate_probe.cuh"
#include "spmm_large_m.cuh"
#include "spmm_list.cuh"
#include "spmm_small_m.cuh"

namespace tsp {

__device__ int g_status_word = 0;

static int* status_device_ptr() {
    // One address per device; looked up once per device, outside any capture.
    static int* ptrs[64] = {nullptr};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
}

static thread_local int t_host_status = ST_OK;

static int device_sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!sms[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        sms[dev] = v;
    }
    return sms[dev];
}

// Launch-shape knobs.  The product reads ONE environment variable, TERNASPMM_PDL=0 (launch without
// programmatic dependent launch).  The others exist only in tuning builds (-DTSP_TUNING):
//   TERNASPMM_FAT=0              small-batch kernel: never use the one-CTA-per-SM shape
//   TERNASPMM_STAGE=0            small-batch kernel: no shared-memory slot for a warp's second tile
//   TERNASPMM_RPC2=0             small-batch kernel: never put two row tiles into one fat CTA
//   TERNASPMM_FORCE_S / _FORCE_W small-batch kernel: this K split and this many warps per CTA
//   TERNASPMM_CTAS_PER_SM_X10    small-batch kernel, thin shape: about that many CTAs per SM (x10)
//   TERNASPMM_MAX_WARPS          small-batch kernel, thin shape: cap on warps per CTA
//   TERNASPMM_CLUSTER_COST_X10   small-batch kernel, thin shape: price of a K split in tenths of a tile time
//   TERNASPMM_LARGE_MIN_M        smallest token count sent to the tcgen05 kernel (default 33)
//   TERNASPMM_LARGE_SPLIT=0      tcgen05 kernel without its cluster K split
//   TERNASPMM_LIST_WARPS         work-list kernel at 8 tokens: 20 (default), 24 or 28 warps per CTA
struct Tuning {
    int ctas_x10 = 0, max_warps = 0, pdl = 1, large_min_m = 33, large_split = 1, cluster_cost_x10 = 0, fat = 1,
        force_s = 0, force_w = 0, stage = 1, rpc2 = 1, list_warps = 20;
    Tuning() {
        if (const char* e = getenv("TERNASPMM_PDL")) pdl = atoi(e) != 0;
#ifdef TSP_TUNING
        if (const char* e = getenv("TERNASPMM_CTAS_PER_SM_X10")) ctas_x10 = atoi(e);
        if (const char* e = getenv("TERNASPMM_MAX_WARPS")) max_warps = atoi(e);
        if (const char* e = getenv("TERNASPMM_LARGE_MIN_M")) large_min_m = atoi(e) > 0 ? atoi(e) : large_min_m;
        if (const char* e = getenv("TERNASPMM_LARGE_SPLIT")) large_split = atoi(e) != 0;
        if (const char* e = getenv("TERNASPMM_CLUSTER_COST_X10")) cluster_cost_x10 = atoi(e);
        if (const char* e = getenv("TERNASPMM_FAT")) fat = atoi(e);
        if (const char* e = getenv("TERNASPMM_STAGE")) stage = atoi(e) != 0;
        if (const char* e = getenv("TERNASPMM_RPC2")) rpc2 = atoi(e) != 0;
        if (const char* e = getenv("TERNASPMM_FORCE_S")) force_s = atoi(e);
        if (const char* e = getenv("TERNASPMM_FORCE_W")) force_w = atoi(e);
        if (const char* e = getenv("TERNASPMM_LIST_WARPS")) list_warps = atoi(e);
#endif
    }
};
static const Tuning& tuning() {
    static Tuning t;
    return t;
}

// Shape of the most recent launch made on this thread (test hook, see ternaspmm_last_launch_shape).
struct LaunchEcho {
    int kernel = 0, tokens_per_pass = 0, splits = 0, warps = 0, row_tiles_per_cta = 0, ctas = 0;
};
static thread_local LaunchEcho t_echo;

// Limit of the device-side waits on a peer (fused tensor-parallel tail), in nanoseconds of the GPU's
// global timer; changed with ternaspmm_set_wait_limit_ms.
static unsigned long long g_wait_limit_ns = 1000ull * 1000 * 1000;

struct LaunchShape {
    int splits, warps;
    int rpc = 1;   // row tiles per CTA (fat shape only)
};

// K split (= cluster size, at most 8) and warps per CTA.  Take the smallest
// number of tiles per warp for which every CTA is resident at once (one wave:
// `warp_slots` warps and at most 2 CTAs per SM at this kernel's register and
// shared-memory budget), and for that the smallest cluster.
// TERNASPMM_CTAS_PER_SM_X10 > 0 overrides with "about that many CTAs per SM".
static LaunchShape choose_shape(int RT, int KT, int token_blocks, int max_warps, int warp_slots) {
    const int sms = device_sm_count();
    const long long rows = (long long)RT * token_blocks;
    const int max_w = tuning().max_warps > 0 && tuning().max_warps < max_warps ? tuning().max_warps : max_warps;
    const int max_s = KT > 1 ? (KT / 2 < 8 ? KT / 2 : 8) : 1;
    if (tuning().force_s > 0 && tuning().force_w > 0) return {tuning().force_s, tuning().force_w};
    if (tuning().ctas_x10 > 0) {
        const long long target = (long long)tuning().ctas_x10 * sms / 10;
        int s = (int)((target + rows - 1) / rows);
        s = s > max_s ? max_s : (s < 1 ? 1 : s);
        const int nt = (KT + s - 1) / s;
        return {s, nt < 2 ? 2 : (nt > max_w ? max_w : nt)};
    }
    // cost of a candidate in tenths of a tile time: tiles per warp, plus the cluster reduction when K is split
    LaunchShape best = {0, 0};
    long long best_cost = -1;
    for (int tpw = 1; tpw <= KT; ++tpw)
        for (int s = 1; s <= max_s; ++s) {
            const int nt = (KT + s - 1) / s;
            int w = (nt + tpw - 1) / tpw;
            if (w > max_w) continue;
            if (w < 2) w = 2;
            int per_sm = warp_slots / w;
            per_sm = per_sm > 2 ? 2 : per_sm;
            if (per_sm < 1 || rows * s > (long long)sms * per_sm) continue;
            const long long cost = 10ll * tpw + (s > 1 ? tuning().cluster_cost_x10 : 0);
            if (best_cost < 0 || cost < best_cost) best = {s, w}, best_cost = cost;
        }
    if (best_cost >= 0) return best;
    // more than one wave whatever we do: no K split, full CTAs
    return {1, KT < 2 ? 2 : (KT > max_w ? max_w : KT)};
}

// "Fat" shape: one CTA per SM with as many warps as the register file allows.  Measured on the
// BitNet-2B layers (QKV at 8 tokens: 5.3 -> 3.4 us), a launch whose row tiles fit the SMs once is
// fastest without any K split as long as a warp gets at most 2 (3 for 32-token blocks) tiles, and
// otherwise with the smallest split that gets there while the clusters still fit the chip in one
// wave; more CTAs than SMs (two thin CTAs per SM, each building its own tables) are slower.  A fat
// launch also leaves SMs free, on which the next launch of the stream starts its prologue at once
// (down projection inside the layer sweep: +4 % on the whole sweep against the thin shape).
// Returns splits = 0 when the thin shape should be used instead.
static LaunchShape choose_fat(int RT, int KT, int token_blocks, int max_warps, int mt) {
    const int sms = device_sm_count();
    const long long rows = (long long)RT * token_blocks;
    if (!tuning().fat) return {0, 0};
    // more row tiles than SMs, but at most twice as many: two row tiles per CTA, half of the warps each
    if (rows > sms && token_blocks == 1 && RT % 2 == 0 && RT / 2 <= sms && tuning().rpc2)
        return {1, max_warps & ~1, 2};
    if (rows > sms) return {0, 0};
    const int max_s = KT > 1 ? (KT / 2 < 8 ? KT / 2 : 8) : 1;
    const int limit = mt >= 4 ? 3 : 2;
    int pick = 0;
    for (int s = 1; s <= max_s && rows * s <= sms; ++s) {
        const int nt = (KT + s - 1) / s;
        pick = s;                                            // the largest feasible split if none reaches the limit
        if ((nt + max_warps - 1) / max_warps <= limit) break;
    }
    if (pick == 0) return {0, 0};
    const int nt = (KT + pick - 1) / pick;
    return {pick, nt < 2 ? 2 : (nt > max_warps ? max_warps : nt)};
}

template <int MT, int MAXW, int MINB>
static cudaError_t launch_small_m(SpmmParams& p, int token_blocks, int warp_slots, cudaStream_t stream,
                                  LaunchShape preset = {0, 0}) {
    using L = SmallMSmem<MT, MINB == 1 ? 2 : 1>;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    auto kern = spmm_small_m_kernel<MT, MAXW, MINB>;
    const LaunchShape shape = preset.splits > 0 ? preset : choose_shape(p.N / 64, p.K / 64, token_blocks, MAXW, warp_slots);
    p.splits = shape.splits;
    const int warps = shape.warps;
    // one CTA per SM (MINB == 1) leaves room for a 4 KB slot per warp: second tiles are decoded before the wait
    // (only the warps that have a second tile need one: the first nt - warps of them)
    const int nt = (p.K / 64 + shape.splits - 1) / shape.splits;
    p.rpc = shape.rpc;
    const int wpr = warps / shape.rpc;   // warps that share a row tile
    const int slots = (MINB == 1 && tuning().stage && nt > wpr) ? (shape.rpc == 2 ? warps : std::min(warps, nt - warps)) : 0;
    p.stage_second = slots > 0 ? 1 : 0;
    const int smem_bytes = L::total + slots * 4096;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             L::total + (MINB == 1 ? MAXW * 4096 : 0));
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const int RT = p.N / 64;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.splits, RT / shape.rpc, token_blocks);
    cfg.blockDim = dim3(warps * 32, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // Programmatic dependent launch: this kernel may start while the previous
    // kernel of the stream still runs; it prefetches its (immutable) weights
    // and waits (griddepcontrol.wait) before touching activations or outputs.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 2 : 1;
    t_echo = {MINB == 1 ? 1 : 2, MT * 8, p.splits, warps, shape.rpc, (int)(cfg.gridDim.x * cfg.gridDim.y * cfg.gridDim.z)};
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// 2-D tensor map over the activations x[M][K] (int8): tiles of NT tokens x
// 128 k, 128-byte swizzle, out-of-range rows and columns read as zero.
static thread_local int t_inject_encode_failure = 0;   // test hook: the next encode on this thread reports failure

// (also used for the dense weight matrix W[N][K]: rows = N, box = 128 rows)
static bool encode_x_map(CUtensorMap* map, const void* x, int M, int K, int NT) {
    if (t_inject_encode_failure) {
        t_inject_encode_failure = 0;
        return false;
    }
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || !ptr)
            return false;
        fn = reinterpret_cast<EncodeFn>(ptr);
    }
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K};
    const cuuint32_t box[2] = {(cuuint32_t)kLgKStep, (cuuint32_t)NT};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(x), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NT, bool DENSE = false>
static cudaError_t launch_large_m(const SpmmParams& p_in, cudaStream_t stream, const int8_t* dense_w = nullptr) {
    using L = LargeMSmem<NT, DENSE>;
    static bool attr_done[64] = {false};
    static int max_clusters[64][4] = {};   // co-resident clusters of 2 / 4 / 8 CTAs (index log2), 0 = not asked yet
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    auto kern = spmm_large_m_kernel<NT, DENSE>;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    SpmmParams p = p_in;
    CUtensorMap map, wmap;
    if (!encode_x_map(&map, p.x, p.M, p.K, NT)) return cudaErrorInvalidValue;   // reported as status 3, nothing is launched
    if (DENSE) {
        if (!encode_x_map(&wmap, dense_w, p.N, p.K, 128)) return cudaErrorInvalidValue;
    } else {
        wmap = map;   // unused by the kernel
    }
    const long long tiles = (long long)((p.N + 127) / 128) * ((p.M + NT - 1) / NT);
    const int sms = device_sm_count(), KS = (p.K + kLgKStep - 1) / kLgKStep;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(L::threads, 1, 1);
    cfg.dynamicSmemBytes = L::total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 2 : 1;
    // K split over a cluster when the tiles alone would leave more than half of the SMs idle:
    // the largest cluster of 2/4/8 CTAs that still fits the chip in one wave with >= 2 k-steps per CTA.
    p.splits = 1;
    if (!DENSE && tiles * 2 <= sms && tuning().large_split) {   // (the dense variant has no K split: its callers pick shapes that fill the chip)
        for (int lg = 3; lg >= 1; --lg) {
            const int S = 1 << lg;
            if (tiles * S > sms || KS < 2 * S || NT / S < 16) continue;
            if (max_clusters[dev][lg] == 0) {
                cfg.gridDim = dim3((unsigned)(tiles * S), 1, 1);
                attr[0].val.clusterDim.x = S;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
                    cudaGetLastError();
                    n = 0;
                }
                max_clusters[dev][lg] = n > 0 ? n : -1;
            }
            if (max_clusters[dev][lg] >= tiles) {
                p.splits = S;
                break;
            }
        }
    }
    attr[0].val.clusterDim.x = p.splits;
    // persistent: one CTA per SM walks over the tiles (with a K split: one tile per cluster)
    cfg.gridDim = dim3(p.splits > 1 ? (unsigned)(tiles * p.splits) : (unsigned)std::min<long long>(tiles, sms), 1, 1);
    t_echo = {DENSE ? 6 : 3, NT, p.splits, L::threads / 32, 2, (int)cfg.gridDim.x};
    return cudaLaunchKernelEx(&cfg, kern, p, map, wmap);
}

// Dense tcgen05 GEMM on CTA pairs (dense_pair.cuh): 256 weight rows x 256 tokens per cluster of two CTAs.
static cudaError_t launch_dense_pair(const SpmmParams& p_in, cudaStream_t stream, const int8_t* dense_w) {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    auto kern = spmm_dense_pair_kernel;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::total);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    SpmmParams p = p_in;
    p.splits = 1;
    CUtensorMap map, wmap;   // each CTA of a pair loads 128 tokens and 128 weight rows per stage
    if (!encode_x_map(&map, p.x, p.M, p.K, 128) || !encode_x_map(&wmap, dense_w, p.N, p.K, 128))
        return cudaErrorInvalidValue;   // reported as status 3, nothing is launched
    const long long tiles = (long long)((p.N + kPairRows - 1) / kPairRows) * ((p.M + kPairNT - 1) / kPairNT);
    const int pairs = (int)std::min<long long>(tiles, device_sm_count() / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(PairSmem::threads, 1, 1);
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.dynamicSmemBytes = PairSmem::total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 2 : 1;
    t_echo = {7, kPairNT, 2, PairSmem::threads / 32, 4, (int)cfg.gridDim.x};
    return cudaLaunchKernelEx(&cfg, kern, p, map, wmap);
}

static void run_spmm(int8_t* x, uint64_t* bitmap, int* tile_off, uint16_t* quarter_off, uint32_t* signs, void* out,
                     __nv_bfloat16* s, __nv_bfloat16* ws, int ws_num, int M, int N, int K, int epilogue,
                     cudaStream_t stream, const int* seg_bounds = nullptr, const __nv_bfloat16* residual = nullptr) {
    t_host_status = ST_OK;
    if (M < 1 || N < 64 || K < 64 || (N % 64) || (K % 64) ||
        (epilogue != EPI_RAW_I32 && epilogue != EPI_F32_DIV && (ws_num < 1 || ws_num > 4))) {
        fprintf(stderr, "ternaspmm: unsupported shape M=%d N=%d K=%d ws_num=%d (need M>=1, N%%64==0, K%%64==0, 1<=ws_num<=4)\n",
                M, N, K, ws_num);
        t_host_status = ST_BAD_SHAPE;
        return;
    }
    if (!x || !bitmap || !tile_off || !quarter_off || !signs || !out || ((epilogue == EPI_DECODE || epilogue == EPI_PREFILL) && (!s || !ws)) || (epilogue == EPI_F32_DIV && !s) ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(bitmap) & 15) ||
        (reinterpret_cast<uintptr_t>(signs) & 15)) {
        fprintf(stderr, "ternaspmm: null or misaligned pointer (x, bitmap and sign_words must be 16-byte aligned)\n");
        t_host_status = ST_BAD_POINTER;
        return;
    }
    SpmmParams p;
    p.x = x;
    p.bitmap = reinterpret_cast<const uint32_t*>(bitmap);
    p.tile_off = tile_off;
    p.quarter_off = quarter_off;
    p.signs = signs;
    p.out = out;
    p.s = s;
    p.ws = ws;
    p.residual = residual;
    p.ws_num = ws_num;
    p.M = M;
    p.N = N;
    p.K = K;
    p.epilogue = epilogue;
    if (seg_bounds) {   // explicit segment boundaries
        for (int i = 0; i < 3; ++i) p.seg_b[i] = (i + 1 < ws_num) ? seg_bounds[i] : INT_MAX;
        p.seg_gran = 1;
    } else {            // the reference's rules, see ws_group()
        const bool prefill = epilogue == EPI_PREFILL;
        p.seg_gran = prefill ? 128 : 8;
        if (N == 3840 && (prefill || ws_num == 3)) {
            p.seg_b[0] = 2560, p.seg_b[1] = 3200, p.seg_b[2] = INT_MAX;
        } else {
            const int gw = ws_num > 0 ? N / ws_num : N;
            p.seg_b[0] = gw, p.seg_b[1] = 2 * gw, p.seg_b[2] = 3 * gw;
        }
    }
    p.status = status_device_ptr();
    if (!p.status) {
        t_host_status = ST_LAUNCH;
        return;
    }
    cudaError_t e;
    // Kernel choice.  Up to 32 tokens: the small-batch kernel.  Above that the
    // tcgen05 kernel (with its cluster K split when the 128-row tiles alone
    // would occupy less than half of the SMs), except for small narrow weights
    // at up to 64 tokens, where the small-batch kernel run over two blocks of
    // 32 tokens is still a little faster (measured on the BitNet-2B shapes).
    const bool narrow = M <= 64 && (N + 127) / 128 < device_sm_count() / 2 && (long long)N * K <= (32ll << 20);
    if (M >= tuning().large_min_m && !(narrow && tuning().large_min_m == 33)) {
        p.splits = 1;
        e = M <= 64 ? launch_large_m<64>(p, stream) : (M <= 128 ? launch_large_m<128>(p, stream) : launch_large_m<256>(p, stream));
    } else {
        // thin: up to two CTAs per SM; fat: one CTA per SM with twice the warps (see choose_fat)
        const int RT = N / 64, KT = K / 64;
        if (M <= 8) {
            LaunchShape fat = choose_fat(RT, KT, 1, 28, 1);
            if (tuning().force_s > 0 && tuning().force_w > 14) fat = {tuning().force_s, tuning().force_w};   // tuning runs
            e = fat.splits ? launch_small_m<1, 28, 1>(p, 1, 28, stream, fat) : launch_small_m<1, 14, 2>(p, 1, 28, stream);
        } else if (M <= 16) {
            const LaunchShape fat = choose_fat(RT, KT, 1, 20, 2);
            e = fat.splits ? launch_small_m<2, 20, 1>(p, 1, 20, stream, fat) : launch_small_m<2, 10, 2>(p, 1, 20, stream);
        } else {
            const int tb = (M + 31) / 32;
            const LaunchShape fat = choose_fat(RT, KT, tb, 16, 4);
            e = fat.splits ? launch_small_m<4, 16, 1>(p, tb, 16, stream, fat) : launch_small_m<4, 8, 2>(p, tb, 16, stream);
        }
    }
    if (e != cudaSuccess) {
        fprintf(stderr, "ternaspmm: launch failed: %s\n", cudaGetErrorString(e));
        t_host_status = ST_LAUNCH;
    }
}

__global__ void sleep_kernel(double us) {
    if (threadIdx.x == 0) {
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        if (us > 1e6) us = 1e6;  // never wait longer than a second
        const unsigned long long want = (unsigned long long)(us * 1e3);
        for (unsigned it = 0; it < (1u << 28); ++it) {
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 >= want) break;
            __nanosleep(200);
        }
    }
    __syncwarp();
}

}  // namespace tsp

using namespace tsp;

extern "C" void checkLastCudaError(int line) {
    cudaError_t error = cudaGetLastError();
    if (error != cudaSuccess) {
        printf("Last Cuda Error Detected at line: %d, Error: %s.\n", line, cudaGetErrorString(error));
        exit(EXIT_FAILURE);
    }
}

extern "C" void bitlinear_TernaSpMM(int8_t* x, uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                                    uint32_t* sign_words, __nv_bfloat16* out, __nv_bfloat16* s, __nv_bfloat16* ws,
                                    int ws_num, int M, int N, int K, int /*split_k*/, int32_t* /*workspace*/,
                                    cudaStream_t stream) {
    run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, ws, ws_num, M, N, K,
             M <= 64 ? EPI_DECODE : EPI_PREFILL, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void bitlinear_TernaSpMM_decode(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                                           uint16_t* quarter_offsets, uint32_t* sign_words, __nv_bfloat16* out,
                                           __nv_bfloat16* s, __nv_bfloat16* ws, int ws_num, int M, int N, int K,
                                           int /*split_k*/, int32_t* /*workspace*/, cudaStream_t stream) {
    run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, ws, ws_num, M, N, K, EPI_DECODE, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void bitlinear_TernaSpMM_prefill(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                                            uint16_t* quarter_offsets, uint32_t* sign_words, __nv_bfloat16* out,
                                            __nv_bfloat16* s, __nv_bfloat16* ws, int ws_num, int M, int N, int K,
                                            int /*split_k*/, int32_t* /*workspace*/, cudaStream_t stream) {
    run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, ws, ws_num, M, N, K, EPI_PREFILL, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void bitlinear_TernaSpMM_residual(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                                            uint16_t* quarter_offsets, uint32_t* sign_words, __nv_bfloat16* out,
                                            __nv_bfloat16* s, __nv_bfloat16* ws, int ws_num, int M, int N, int K,
                                            __nv_bfloat16* residual, cudaStream_t stream) {
    run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, ws, ws_num, M, N, K,
             M <= 64 ? EPI_DECODE : EPI_PREFILL, stream, nullptr, residual);
    checkLastCudaError(__LINE__);
}

// Large-batch path through a dense workspace: decompress once, then the tensor-core kernel with both
// operands by TMA.  Returns false when the shape is one the on-chip path serves better.
static bool dense_prefill_pays(int M, int N, int K, long long workspace_bytes) {
    // Measured on the BitNet-2B layers (one call, microseconds, on chip / through the workspace):
    //   tokens           256          384          512          1024         2048         4096
    //   3840 x 2560   14.9 / 17.0  18.7 / 17.2  18.9 / 17.7  20.5 / 18.0  32.9 / 24.4  59.0 / 37.8
    //   13824 x 2560  20.3 / 21.6  31.5 / 27.1  32.0 / 28.0  46.7 / 36.1  87.3 / 58.5  168 / 107
    //   2560 x 6912   18.0 / 27.5  26.4 / 27.9  26.7 / 28.4  36.4 / 29.0  62.8 / 45.1  91.5 / 61.9
    // The on-chip kernel decodes every weight tile once per 256 tokens, so from the second token tile on
    // decoding once into the workspace wins; deep, narrow layers (few output tiles, a long K loop) need
    // more tokens, because on chip they split K over a cluster and the pair kernel does not.
    (void)N;
    if (workspace_bytes < (long long)N * K) return false;
    return M >= 384 && (K <= 4096 || M >= 1024);
}

static cudaError_t launch_decompress(const SpmmParams& p, int8_t* dense, cudaStream_t stream) {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    const int smem_bytes = kLut2Bytes + kLutBytes + 2048 + 256;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(decompress_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const long long tiles = (long long)(p.N / 64) * (p.K / 64);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)std::min<long long>(device_sm_count(), (tiles + kDecompressWarps - 1) / kDecompressWarps), 1, 1);
    cfg.blockDim = dim3(kDecompressWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, decompress_kernel, p, dense);
}

extern "C" void bitlinear_TernaSpMM_ws(int8_t* x, uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                                       uint32_t* sign_words, __nv_bfloat16* out, __nv_bfloat16* s, __nv_bfloat16* ws,
                                       int ws_num, int M, int N, int K, __nv_bfloat16* residual, void* workspace,
                                       long long workspace_bytes, int path, cudaStream_t stream) {
    const int epilogue = M <= 64 ? EPI_DECODE : EPI_PREFILL;
    const bool dense = path == 2 || (path == 0 && workspace && !(reinterpret_cast<uintptr_t>(workspace) & 127) &&
                                    dense_prefill_pays(M, N, K, workspace_bytes));   // (a workspace that cannot be used is not an error)
    if (!dense) {
        run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, ws, ws_num, M, N, K, epilogue, stream, nullptr,
                 residual);
        checkLastCudaError(__LINE__);
        return;
    }
    t_host_status = ST_OK;
    if (M < 1 || N < 64 || K < 64 || (N % 64) || (K % 64) || ws_num < 1 || ws_num > 4) {
        fprintf(stderr, "ternaspmm: unsupported shape M=%d N=%d K=%d ws_num=%d\n", M, N, K, ws_num);
        t_host_status = ST_BAD_SHAPE;
        return;
    }
    if (!x || !bitmap || !tile_offsets || !quarter_offsets || !sign_words || !out || !s || !ws || !workspace ||
        workspace_bytes < (long long)N * K || (reinterpret_cast<uintptr_t>(x) & 15) ||
        (reinterpret_cast<uintptr_t>(bitmap) & 15) || (reinterpret_cast<uintptr_t>(sign_words) & 15) ||
        (reinterpret_cast<uintptr_t>(workspace) & 127)) {
        fprintf(stderr, "ternaspmm: bitlinear_TernaSpMM_ws: null or misaligned pointer, or a workspace below N*K bytes "
                        "(workspace: 128-byte aligned)\n");
        t_host_status = ST_BAD_POINTER;
        return;
    }
    SpmmParams p = {};
    p.x = x, p.bitmap = reinterpret_cast<const uint32_t*>(bitmap), p.tile_off = tile_offsets, p.quarter_off = quarter_offsets;
    p.signs = sign_words, p.out = out, p.s = s, p.ws = ws, p.residual = residual;
    p.ws_num = ws_num, p.M = M, p.N = N, p.K = K, p.epilogue = epilogue, p.splits = 1;
    {   // the reference's scale-segment rules (see ws_group in spmm_small_m.cuh)
        const bool prefill = epilogue == EPI_PREFILL;
        p.seg_gran = prefill ? 128 : 8;
        if (N == 3840 && (prefill || ws_num == 3)) {
            p.seg_b[0] = 2560, p.seg_b[1] = 3200, p.seg_b[2] = INT_MAX;
        } else {
            const int gw = N / ws_num;
            p.seg_b[0] = gw, p.seg_b[1] = 2 * gw, p.seg_b[2] = 3 * gw;
        }
    }
    p.status = status_device_ptr();
    if (!p.status) {
        t_host_status = ST_LAUNCH;
        return;
    }
    int8_t* dense_w = static_cast<int8_t*>(workspace);
    cudaError_t e = cudaSuccess;
#ifdef TSP_TUNING
    static const int tune_nt = getenv("TERNASPMM_DENSE_NT") ? atoi(getenv("TERNASPMM_DENSE_NT")) : 0;
    static const int tune_skip = getenv("TERNASPMM_DENSE_SKIP_DECOMPRESS") ? atoi(getenv("TERNASPMM_DENSE_SKIP_DECOMPRESS")) : 0;
    if (!tune_skip) e = launch_decompress(p, dense_w, stream);
    static const int tune_pair = getenv("TERNASPMM_DENSE_PAIR") ? atoi(getenv("TERNASPMM_DENSE_PAIR")) : 1;
    if (e == cudaSuccess)
        e = (M <= 128 || tune_nt == 128) ? launch_large_m<128, true>(p, stream, dense_w)
            : (tune_pair ? launch_dense_pair(p, stream, dense_w) : launch_large_m<256, true>(p, stream, dense_w));
#else
    e = launch_decompress(p, dense_w, stream);
    if (e == cudaSuccess)
        e = M <= 128 ? launch_large_m<128, true>(p, stream, dense_w) : launch_dense_pair(p, stream, dense_w);
#endif
    if (e != cudaSuccess) {
        fprintf(stderr, "ternaspmm: launch failed: %s\n", cudaGetErrorString(e));
        t_host_status = ST_LAUNCH;
    }
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_accumulate_i32(int8_t* x, uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                                         uint32_t* sign_words, int32_t* out, int M, int N, int K,
                                         cudaStream_t stream) {
    run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, nullptr, nullptr, 1, M, N, K, EPI_RAW_I32,
             stream);
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_linear_segments(int8_t* x, uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                                         uint32_t* sign_words, __nv_bfloat16* out, __nv_bfloat16* s,
                                         __nv_bfloat16* ws, int ws_num, int M, int N, int K, int seg1, int seg2,
                                         int seg3, int prefill_form, cudaStream_t stream) {
    const int b[3] = {seg1, seg2, seg3};
    const int epi = prefill_form < 0 ? (M <= 64 ? EPI_DECODE : EPI_PREFILL) : (prefill_form ? EPI_PREFILL : EPI_DECODE);
    run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, ws, ws_num, M, N, K, epi, stream, b);
    checkLastCudaError(__LINE__);
}

static void run_norm_quant(bool gated, int mode, __nv_bfloat16* x, __nv_bfloat16* w, float eps, int M, int K,
                           int8_t* q, __nv_bfloat16* s_out, float* ss_out, cudaStream_t stream) {
    t_host_status = ST_OK;
    if (M < 1 || K < 16 || (K % 16) || K > 56 * 1024) {
        fprintf(stderr, "ternaspmm: norm_quant needs M>=1 and K a multiple of 16 up to 57344 (got M=%d K=%d)\n", M, K);
        t_host_status = ST_BAD_SHAPE;
        return;
    }
    if (!x || (mode != ACT_PLAIN && !w) || !q || (!s_out && mode != ACT_NORM_ONLY) || (mode == ACT_SCALE_SUMSQ && !ss_out) ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
        (reinterpret_cast<uintptr_t>(q) & 15)) {
        fprintf(stderr, "ternaspmm: norm_quant: null or misaligned pointer\n");
        t_host_status = ST_BAD_POINTER;
        return;
    }
    typedef void (*Kern)(const __nv_bfloat16*, const __nv_bfloat16*, float, int, int8_t*, __nv_bfloat16*, float*);
    Kern kern = gated ? (mode == ACT_RMSNORM ? norm_quant_kernel<true, ACT_RMSNORM> : norm_quant_kernel<true, ACT_SCALE_SUMSQ>)
                      : mode == ACT_NORM_ONLY ? norm_quant_kernel<false, ACT_NORM_ONLY>
                      : (mode == ACT_RMSNORM ? norm_quant_kernel<false, ACT_RMSNORM>
                                             : (mode == ACT_SCALE_SUMSQ ? norm_quant_kernel<false, ACT_SCALE_SUMSQ>
                                                                        : norm_quant_kernel<false, ACT_PLAIN>));
    static bool attr_done[64][8] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    const int slot = (gated ? 4 : 0) + mode;
    if (!attr_done[dev][slot]) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 56 * 1024);
        attr_done[dev][slot] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M, 1, 1);
    cfg.blockDim = dim3(std::min(kActMaxThreads, std::max(64, (K / 8 + 31) / 32 * 32)), 1, 1);   // one vector per thread
    cfg.dynamicSmemBytes = (size_t)K * 2;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, eps, K, q, s_out, ss_out) !=
        cudaSuccess)
        t_host_status = ST_LAUNCH;
}

extern "C" void ternaspmm_rmsnorm_quant(__nv_bfloat16* x, __nv_bfloat16* norm_weight, float eps, int M, int K,
                                       int8_t* q, __nv_bfloat16* s_out, cudaStream_t stream) {
    run_norm_quant(false, ACT_RMSNORM, x, norm_weight, eps, M, K, q, s_out, nullptr, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_relu2_gate_rmsnorm_quant(__nv_bfloat16* x13, __nv_bfloat16* norm_weight, float eps, int M,
                                                  int K, int8_t* q, __nv_bfloat16* s_out, cudaStream_t stream) {
    run_norm_quant(true, ACT_RMSNORM, x13, norm_weight, eps, M, K, q, s_out, nullptr, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_rmsnorm(__nv_bfloat16* x, __nv_bfloat16* norm_weight, float eps, int M, int K, __nv_bfloat16* y,
                                  cudaStream_t stream) {
    run_norm_quant(false, ACT_NORM_ONLY, x, norm_weight, eps, M, K, reinterpret_cast<int8_t*>(y), nullptr, nullptr, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_quant(__nv_bfloat16* x, int M, int K, int8_t* q, __nv_bfloat16* s_out, cudaStream_t stream) {
    run_norm_quant(false, ACT_PLAIN, x, nullptr, 0.f, M, K, q, s_out, nullptr, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_scale_quant_sumsq(__nv_bfloat16* x, __nv_bfloat16* weight, int gated, int M, int K,
                                           int8_t* q, __nv_bfloat16* s_out, float* ss_out, cudaStream_t stream) {
    run_norm_quant(gated != 0, ACT_SCALE_SUMSQ, x, weight, 0.f, M, K, q, s_out, ss_out, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_partial_f32(int8_t* x, uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                                     uint32_t* sign_words, float* out, __nv_bfloat16* s, int M, int N, int K,
                                     cudaStream_t stream) {
    run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, nullptr, 1, M, N, K, EPI_F32_DIV, stream);
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_tp_finish(float* buf, __nv_bfloat16* ws, float eps, int full_width, int M, int N,
                                   __nv_bfloat16* residual, __nv_bfloat16* out, cudaStream_t stream) {
    t_host_status = ST_OK;
    if (!buf || !ws || !out || M < 1 || N < 1) {
        t_host_status = ST_BAD_POINTER;
        return;
    }
    const long long total = (long long)M * N;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 4 * device_sm_count()) blocks = 4 * device_sm_count();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, tp_finish_kernel, (const float*)buf, (const __nv_bfloat16*)ws, eps, full_width, M, N,
                           (const __nv_bfloat16*)residual, out) != cudaSuccess)
        t_host_status = ST_LAUNCH;
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_tp_allreduce_finish(float** bufs, unsigned int** flags, __nv_bfloat16** outs, int rank,
                                             int world, unsigned int* counters, __nv_bfloat16* ws, float eps,
                                             int full_width, int M, int N, __nv_bfloat16* residual,
                                             cudaStream_t stream) {
    t_host_status = ST_OK;
    if (!bufs || !flags || !outs || !counters || !ws || world < 1 || world > 8 || rank < 0 || rank >= world || M < 1 ||
        N < 4 || (N % 4)) {
        fprintf(stderr, "ternaspmm: tp_allreduce_finish: bad arguments (world 1..8, N a multiple of 4)\n");
        t_host_status = ST_BAD_POINTER;
        return;
    }
    TpPeers peers = {};
    for (int r = 0; r < world; ++r) {
        if (!bufs[r] || !flags[r] || !outs[r]) {
            t_host_status = ST_BAD_POINTER;
            return;
        }
        peers.buf[r] = bufs[r];
        peers.flag[r] = flags[r];
        peers.out[r] = outs[r];
    }
    int* status = status_device_ptr();
    if (!status) {
        t_host_status = ST_LAUNCH;
        return;
    }
    // this rank finishes 1/world of the outputs: one 4-element vector per thread, at most two blocks per SM
    const long long vecs = ((long long)M * N / 4 + world - 1) / world;
    int blocks = (int)std::max<long long>(1, std::min<long long>((vecs + 255) / 256, 2ll * device_sm_count()));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, tp_allreduce_finish_kernel, peers, rank, world, counters, counters + 1,
                           (const __nv_bfloat16*)ws, eps, full_width, M, N, (const __nv_bfloat16*)residual,
                           status, g_wait_limit_ns) != cudaSuccess)
        t_host_status = ST_LAUNCH;
    checkLastCudaError(__LINE__);
}

// ---- work lists ----------------------------------------------------------------------------------
struct ternaspmm_list {
    void* device_table;
    void* scratch;
    int entries, mt;
};

static size_t list_scratch_bytes() { return sizeof(ListScratch) + (size_t)device_sm_count() * kListAreaInts * 4; }

// Validates the items and turns them into device entries.  Returns false on a bad item.
static bool list_entries(const ternaspmm_list_item* items, int n, std::vector<ListItem>& out, int& max_m) {
    max_m = 0;
    long long tiles = 0;
    if (n > kListMaxItems) {
        fprintf(stderr, "ternaspmm: a list holds at most %d items (got %d)\n", kListMaxItems, n);
        t_host_status = ST_BAD_SHAPE;
        return false;
    }
    for (int i = 0; i < n; ++i) {
        const ternaspmm_list_item& u = items[i];
        if (u.M < 1 || u.M > 16 || u.N < 64 || u.K < 64 || (u.N % 64) || (u.K % 64) || u.K / 64 > 4095 || u.N / 64 > 4095 ||
            u.ws_num < 1 || u.ws_num > 4) {
            fprintf(stderr, "ternaspmm: list item %d: unsupported shape M=%d N=%d K=%d ws_num=%d (need 1<=M<=16, N%%64==0, "
                            "K%%64==0, N and K below 262144)\n", i, u.M, u.N, u.K, u.ws_num);
            t_host_status = ST_BAD_SHAPE;
            return false;
        }
        if (!u.x || !u.bitmap || !u.tile_offsets || !u.quarter_offsets || !u.sign_words || !u.out || !u.s || !u.ws ||
            (reinterpret_cast<uintptr_t>(u.x) & 15) || (reinterpret_cast<uintptr_t>(u.bitmap) & 15) ||
            (reinterpret_cast<uintptr_t>(u.sign_words) & 15)) {
            fprintf(stderr, "ternaspmm: list item %d: null or misaligned pointer\n", i);
            t_host_status = ST_BAD_POINTER;
            return false;
        }
        const int epi = u.prefill_form < 0 ? (u.M <= 64 ? EPI_DECODE : EPI_PREFILL) : (u.prefill_form ? EPI_PREFILL : EPI_DECODE);
        ListItem e = {};
        e.x = u.x, e.bitmap = reinterpret_cast<const uint32_t*>(u.bitmap), e.tile_off = u.tile_offsets;
        e.quarter_off = u.quarter_offsets, e.signs = u.sign_words;
        e.out = reinterpret_cast<__nv_bfloat16*>(u.out), e.residual = reinterpret_cast<const __nv_bfloat16*>(u.residual);
        e.s = reinterpret_cast<const __nv_bfloat16*>(u.s), e.ws = reinterpret_cast<const __nv_bfloat16*>(u.ws);
        e.M = u.M, e.N = u.N, e.K = u.K, e.ld_out = u.N, e.ws_num = u.ws_num, e.epilogue = epi;
        if (u.seg1 || u.seg2 || u.seg3) {   // explicit boundaries
            const int b[3] = {u.seg1, u.seg2, u.seg3};
            for (int k = 0; k < 3; ++k) e.seg_b[k] = (k + 1 < u.ws_num) ? b[k] : INT_MAX;
            e.seg_gran = 1;
        } else {                            // the reference's rules (see ws_group in spmm_small_m.cuh)
            const bool prefill = epi == EPI_PREFILL;
            e.seg_gran = prefill ? 128 : 8;
            if (u.N == 3840 && (prefill || u.ws_num == 3)) {
                e.seg_b[0] = 2560, e.seg_b[1] = 3200, e.seg_b[2] = INT_MAX;
            } else {
                const int gw = u.N / u.ws_num;
                e.seg_b[0] = gw, e.seg_b[1] = 2 * gw, e.seg_b[2] = 3 * gw;
            }
        }
        e.tile_base = tiles;
        tiles += (long long)(u.N / 64) * (u.K / 64);
        out.push_back(e);
        max_m = std::max(max_m, u.M);
    }
    if (tiles / std::max(1, device_sm_count()) > (1ll << 30)) {
        t_host_status = ST_BAD_SHAPE;
        return false;
    }
    return true;
}

extern "C" int ternaspmm_list_plan(const ternaspmm_list_item* items, int n_items, long long* table_bytes,
                                   long long* scratch_bytes) {
    t_host_status = ST_OK;
    std::vector<ListItem> e;
    int max_m;
    if (!items || n_items < 1 || !list_entries(items, n_items, e, max_m)) {
        if (t_host_status == ST_OK) t_host_status = ST_BAD_POINTER;
        return -1;
    }
    if (table_bytes) *table_bytes = (long long)e.size() * sizeof(ListItem);
    if (scratch_bytes) *scratch_bytes = (long long)list_scratch_bytes();
    return (int)e.size();
}

extern "C" ternaspmm_list* ternaspmm_list_create(const ternaspmm_list_item* items, int n_items, void* device_table,
                                                 void* scratch, cudaStream_t stream) {
    t_host_status = ST_OK;
    std::vector<ListItem> e;
    int max_m;
    if (!items || n_items < 1 || !device_table || !scratch || (reinterpret_cast<uintptr_t>(device_table) & 15) ||
        (reinterpret_cast<uintptr_t>(scratch) & 15)) {
        t_host_status = ST_BAD_POINTER;
        return nullptr;
    }
    if (!list_entries(items, n_items, e, max_m)) return nullptr;
    if (cudaMemcpyAsync(device_table, e.data(), e.size() * sizeof(ListItem), cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaMemsetAsync(scratch, 0, list_scratch_bytes(), stream) != cudaSuccess || cudaStreamSynchronize(stream) != cudaSuccess) {
        t_host_status = ST_LAUNCH;
        return nullptr;
    }
    ternaspmm_list* l = static_cast<ternaspmm_list*>(malloc(sizeof(ternaspmm_list)));
    if (!l) return nullptr;
    l->device_table = device_table, l->scratch = scratch, l->entries = (int)e.size();
    l->mt = max_m <= 8 ? 1 : 2;
    return l;
}

extern "C" void ternaspmm_list_destroy(ternaspmm_list* l) { free(l); }

template <int MT, int W>
static cudaError_t launch_list(const ternaspmm_list* l, int* status, cudaStream_t stream) {
    using L = ListSmem<MT>;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    auto kern = spmm_list_kernel<MT, W>;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(std::min(device_sm_count(), kListMaxCtas), 1, 1);       // one persistent CTA per SM
    cfg.blockDim = dim3(W * 32, 1, 1);                  // W - 1 decoder warps and one epilogue warp
    cfg.dynamicSmemBytes = L::total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    t_echo = {5, MT * 8, 1, W, 0, (int)cfg.gridDim.x};
    return cudaLaunchKernelEx(&cfg, kern, static_cast<const ListItem*>(l->device_table), l->entries,
                              static_cast<uint8_t*>(l->scratch), status);
}

extern "C" void ternaspmm_list_run(ternaspmm_list* l, cudaStream_t stream) {
    t_host_status = ST_OK;
    if (!l) {
        t_host_status = ST_BAD_POINTER;
        return;
    }
    int* status = status_device_ptr();
    if (!status) {
        t_host_status = ST_LAUNCH;
        return;
    }
#ifdef TSP_TUNING
    if (const char* ab = getenv("TERNASPMM_LIST_ABLATE")) {
        const int v = atoi(ab);
        cudaMemcpyToSymbol(g_list_ablate, &v, sizeof(int));
    }
#endif
    cudaError_t e;
    if (l->mt == 2) e = launch_list<2, 16>(l, status, stream);
    else if (tuning().list_warps == 24) e = launch_list<1, 24>(l, status, stream);
    else if (tuning().list_warps == 28) e = launch_list<1, 28>(l, status, stream);
    else e = launch_list<1, 20>(l, status, stream);   // 96 registers per thread, no spills: measured faster than 24 or 28 warps with spills
    if (e != cudaSuccess) {
        fprintf(stderr, "ternaspmm: list launch failed: %s\n", cudaGetErrorString(e));
        t_host_status = ST_LAUNCH;
    }
    checkLastCudaError(__LINE__);
}

extern "C" long long ternaspmm_lm_head_scratch_bytes(void) { return (long long)kHeadScratchBytes; }

extern "C" void ternaspmm_lm_head_argmax(__nv_bfloat16* h, __nv_bfloat16* embedding, int M, int V, int K, float* logits,
                                        long long* argmax, int round_bf16, void* scratch, cudaStream_t stream) {
    t_host_status = ST_OK;
    if (M < 1 || M > 8 || V < 1 || K < 32 || (K % 32) || K > 12288) {
        fprintf(stderr, "ternaspmm: lm_head_argmax needs 1 <= M <= 8, V >= 1, K a multiple of 32 up to 12288 (got M=%d V=%d K=%d)\n",
                M, V, K);
        t_host_status = ST_BAD_SHAPE;
        return;
    }
    if (!h || !embedding || (!logits && !argmax) || (argmax && !scratch) || (reinterpret_cast<uintptr_t>(h) & 15) ||
        (reinterpret_cast<uintptr_t>(embedding) & 15) || (reinterpret_cast<uintptr_t>(scratch) & 15)) {
        fprintf(stderr, "ternaspmm: lm_head_argmax: null or misaligned pointer (h, embedding, scratch: 16 bytes)\n");
        t_host_status = ST_BAD_POINTER;
        return;
    }
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * (12288 * 2 + 64)) != cudaSuccess) {
            t_host_status = ST_LAUNCH;
            return;
        }
        attr_done[dev] = true;
    }
    HeadParams p;
    p.h = h, p.emb = embedding, p.logits = logits, p.argmax = argmax;
    p.counter = reinterpret_cast<unsigned int*>(scratch);
    p.cand = reinterpret_cast<HeadCandidate*>(reinterpret_cast<uint8_t*>(scratch) + 16);
    p.M = M, p.V = V, p.K = K, p.round_bf16 = round_bf16;
    const int groups = (V + 15) / 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(std::min(std::min(device_sm_count(), groups), kHeadMaxCtas), 1, 1);
    cfg.blockDim = dim3(kHeadWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = 8 * (K * 2 + 64);
    cfg.stream = stream;
    // No programmatic dependent launch for this kernel: it wants every SM for itself from the first cycle.
    // Launched early behind a kernel that releases its dependents at once (the library's norm kernel), its
    // CTAs compete for SMs with the still unplaced CTAs of the linears before it: measured on the 30-layer
    // model, the decoded token took 5 % longer.  In stream order it starts a few microseconds later and
    // runs on an empty chip.
    t_echo = {4, 8, 1, kHeadWarps, 0, (int)cfg.gridDim.x};
    if (cudaLaunchKernelEx(&cfg, lm_head_kernel, p) != cudaSuccess) t_host_status = ST_LAUNCH;
    checkLastCudaError(__LINE__);
}

// ---- output head without any caller-provided scratch memory -------------------------------------
// Some callers of this library cannot hand it scratch memory at all: an operator plugged into a
// serving runtime that owns every byte of device memory through its own arena and forbids its
// operators to call cudaMalloc; a control loop for which the device-wide synchronisation hidden in
// cudaMalloc / cudaFree is unacceptable; code that runs while a stream is being captured, where an
// allocation is an error.  For them the arg-max candidates and the arrival counter of the head
// kernel live in the array below, which is part of the library's image: every GPU that loads the
// library holds these 16 KB until the process exits.
constexpr int kHeadStaticCtas = 256;   // candidate slots: the launch uses min(SMs, row groups, this many) CTAs
static __device__ __align__(256) unsigned char g_head_static_scratch[16 + sizeof(HeadCandidate) * 8 * kHeadStaticCtas];

// Device address of the array above on the current device.  The array's NAME is only a host-side
// handle here - passing it to a kernel would hand the GPU a host address - so the real address is
// asked for once per device, with that device current, and the answer is kept.
static void* head_static_scratch_ptr() {
    static void* ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_head_static_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return nullptr;
        }
        ptrs[dev] = p;
    }
    return ptrs[dev];
}

extern "C" void ternaspmm_lm_head_argmax_noalloc(__nv_bfloat16* h, __nv_bfloat16* embedding, int M, int V, int K,
                                                float* logits, long long* argmax, int round_bf16, cudaStream_t stream) {
    t_host_status = ST_OK;
    if (M < 1 || M > 8 || V < 1 || K < 32 || (K % 32) || K > 12288) {
        fprintf(stderr, "ternaspmm: lm_head_argmax_noalloc: the built-in scratch area holds candidates for at most 8 rows; "
                        "needs 1 <= M <= 8, V >= 1, K a multiple of 32 up to 12288 (got M=%d V=%d K=%d)\n", M, V, K);
        t_host_status = ST_BAD_SHAPE;
        return;
    }
    if (!h || !embedding || (!logits && !argmax) || (reinterpret_cast<uintptr_t>(h) & 15) ||
        (reinterpret_cast<uintptr_t>(embedding) & 15)) {
        fprintf(stderr, "ternaspmm: lm_head_argmax_noalloc: null or misaligned pointer (h, embedding: 16 bytes)\n");
        t_host_status = ST_BAD_POINTER;
        return;
    }
    void* scratch = head_static_scratch_ptr();   // the first call on a device looks the address up
    if (!scratch) {
        fprintf(stderr, "ternaspmm: lm_head_argmax_noalloc: cannot resolve the built-in scratch area on this device\n");
        t_host_status = ST_LAUNCH;
        return;
    }
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * (12288 * 2 + 64)) != cudaSuccess) {
            t_host_status = ST_LAUNCH;
            return;
        }
        attr_done[dev] = true;
    }
    // every call shares the area and finds the previous call's candidates in it; only the arrival
    // counter has to start at zero, and it is cleared here rather than trusted
    if (cudaMemsetAsync(scratch, 0, 16, stream) != cudaSuccess) {
        t_host_status = ST_LAUNCH;
        return;
    }
    HeadParams p;
    p.h = h, p.emb = embedding, p.logits = logits, p.argmax = argmax;
    p.counter = reinterpret_cast<unsigned int*>(scratch);
    p.cand = reinterpret_cast<HeadCandidate*>(reinterpret_cast<uint8_t*>(scratch) + 16);
    p.M = M, p.V = V, p.K = K, p.round_bf16 = round_bf16;
    const int groups = (V + 15) / 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(std::min(std::min(device_sm_count(), groups), kHeadStaticCtas), 1, 1);
    cfg.blockDim = dim3(kHeadWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = 8 * (K * 2 + 64);
    cfg.stream = stream;
    if (cudaLaunchKernelEx(&cfg, lm_head_kernel, p) != cudaSuccess) t_host_status = ST_LAUNCH;
    checkLastCudaError(__LINE__);
}

extern "C" void ternaspmm_debug_inject_host_failure(int kind) {
    if (kind == 1) t_inject_encode_failure = 1;
}

extern "C" int ternaspmm_last_status(void);

// Measurement hook (see mma_rate_probe.cuh): int8 tensor-core operations per second that this GPU issues
// from shared-memory operands, over all SMs; 0 on failure.  Synchronises the stream.
extern "C" double ternaspmm_debug_int8_mma_rate(int iters, cudaStream_t stream) {
    t_host_status = ST_OK;
    if (iters < 64) iters = 64;
    iters = (iters + 63) / 64 * 64;
    int* status = status_device_ptr();
    const int smem_bytes = 1024 + 1024 + kLgAStage + 256 * kLgKStep;
    if (!status || cudaFuncSetAttribute(int8_mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
        t_host_status = ST_LAUNCH;
        return 0.0;
    }
    const int sms = device_sm_count();
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return 0.0;
    int8_mma_rate_kernel<<<sms, 128, smem_bytes, stream>>>(64, status);   // warm-up
    cudaEventRecord(e0, stream);
    int8_mma_rate_kernel<<<sms, 128, smem_bytes, stream>>>(iters, status);
    cudaEventRecord(e1, stream);
    float ms = 0.f;
    const bool ok = cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess && ms > 0.f;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (!ok || ternaspmm_last_status() != 0) return 0.0;
    return 2.0 * 128 * 256 * 32 * 4.0 * iters * sms / (ms * 1e-3);
}

extern "C" void ternaspmm_set_wait_limit_ms(int ms) {
    if (ms < 1) ms = 1;
    if (ms > 10000) ms = 10000;
    g_wait_limit_ns = (unsigned long long)ms * 1000ull * 1000ull;
}

extern "C" void ternaspmm_last_launch_shape(int* out6) {
    if (!out6) return;
    out6[0] = t_echo.kernel, out6[1] = t_echo.tokens_per_pass, out6[2] = t_echo.splits, out6[3] = t_echo.warps;
    out6[4] = t_echo.row_tiles_per_cta, out6[5] = t_echo.ctas;
}

extern "C" int ternaspmm_last_status(void) {
    if (t_host_status != ST_OK) return t_host_status;
    int v = 0;
    int* d = status_device_ptr();
    if (!d) return ST_LAUNCH;
    if (cudaMemcpy(&v, d, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ST_LAUNCH;
    if (v != 0) {
        int zero = 0;
        cudaMemcpy(d, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    return v;
}

extern "C" void bitlinear_TernaSpMM_benchmark(int mode, int warmup_iters, int bench_iters, int8_t* x,
                                              uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                                              uint32_t* sign_words, __nv_bfloat16* out, __nv_bfloat16* s,
                                              __nv_bfloat16* ws, int ws_num, int M, int N, int K, int split_k,
                                              int32_t* workspace, cudaStream_t stream) {
    if (mode < 0 || mode > 2) mode = 0;
    const int epilogue = mode == 1 ? EPI_PREFILL : (mode == 2 ? EPI_DECODE : (M <= 64 ? EPI_DECODE : EPI_PREFILL));
    (void)split_k;
    (void)workspace;
    for (int i = 0; i < warmup_iters; ++i)
        run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, ws, ws_num, M, N, K, epilogue, stream);
    cudaStreamSynchronize(stream);
    checkLastCudaError(__LINE__);
    cudaEvent_t start, stop;
    cudaEventCreate(&start);
    cudaEventCreate(&stop);
    cudaEventRecord(start, stream);
    for (int i = 0; i < bench_iters; ++i)
        run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, s, ws, ws_num, M, N, K, epilogue, stream);
    cudaEventRecord(stop, stream);
    cudaEventSynchronize(stop);
    checkLastCudaError(__LINE__);
    float total_ms = 0.f;
    cudaEventElapsedTime(&total_ms, start, stop);
    const float avg_us = bench_iters > 0 ? total_ms / bench_iters * 1000.0f : 0.f;
    printf("Shape(M=%d, N=%d, K=%d): %.2f us (avg over %d iters, warmup=%d)\n", M, N, K, avg_us, bench_iters,
           warmup_iters);
    cudaEventDestroy(start);
    cudaEventDestroy(stop);
}

#ifdef TSP_PHASE_TIMERS
// Tuning builds only: copy the per-CTA phase timestamps of the last launch.
extern "C" int ternaspmm_debug_read_phases(unsigned long long* dst, int ctas) {
    if (ctas > 4096) ctas = 4096;
    return (int)cudaMemcpyFromSymbol(dst, g_phase_log, sizeof(unsigned long long) * ctas * kPhaseSlots);
}
#endif

extern "C" void gpu_sleep(double sleep_us, cudaStream_t stream) { sleep_kernel<<<1, 32, 0, stream>>>(sleep_us); }
