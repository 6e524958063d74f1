// libternaspmm.so for NVIDIA B200 (sm_100a): the extern "C" surface declared
// in include/ternaspmm.h and the host-side launch logic behind it.
//
// The entry points mirror kernels/TernaSpMM.cu of Gu-J/TernaInfer (same names,
// argument order and meaning); everything behind them is new.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

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

template <int MT, int MAXW>
static cudaError_t launch_small_m(const SpmmParams& p, int token_blocks, cudaStream_t stream) {
    using L = SmallMSmem<MT>;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    auto kern = spmm_small_m_kernel<MT, MAXW>;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const int RT = p.N / 64, KT = p.K / 64;
    const int nt = (KT + p.splits - 1) / p.splits;
    int warps = nt < 2 ? 2 : (nt > MAXW ? MAXW : nt);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.splits, RT, token_blocks);
    cfg.blockDim = dim3(warps * 32, 1, 1);
    cfg.dynamicSmemBytes = L::total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// K split (= cluster size, at most 8): enough CTAs to fill the device about
// twice, but never fewer than two k-tiles per CTA.
static int choose_splits(int RT, int KT, int token_blocks) {
    const int target = 2 * device_sm_count();
    const long long ctas = (long long)RT * token_blocks;
    int s = (int)((target + ctas - 1) / ctas);
    if (s > 8) s = 8;
    if (s > KT / 2) s = KT / 2;
    if (s < 1) s = 1;
    return s;
}

static void run_spmm(int8_t* x, uint64_t* bitmap, int* tile_off, uint16_t* quarter_off, uint32_t* signs, void* out,
                     __nv_bfloat16* s, __nv_bfloat16* ws, int ws_num, int M, int N, int K, int epilogue,
                     cudaStream_t stream) {
    t_host_status = ST_OK;
    if (M < 1 || N < 64 || K < 64 || (N % 64) || (K % 64) ||
        (epilogue != EPI_RAW_I32 && (ws_num < 1 || ws_num > 4))) {
        fprintf(stderr, "ternaspmm: unsupported shape M=%d N=%d K=%d ws_num=%d (need M>=1, N%%64==0, K%%64==0, 1<=ws_num<=4)\n",
                M, N, K, ws_num);
        t_host_status = ST_BAD_SHAPE;
        return;
    }
    if (!x || !bitmap || !tile_off || !quarter_off || !signs || !out || (epilogue != EPI_RAW_I32 && (!s || !ws)) ||
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
    p.ws_num = ws_num;
    p.M = M;
    p.N = N;
    p.K = K;
    p.epilogue = epilogue;
    p.status = status_device_ptr();
    if (!p.status) {
        t_host_status = ST_LAUNCH;
        return;
    }
    cudaError_t e;
    if (M <= 8) {
        p.splits = choose_splits(N / 64, K / 64, 1);
        e = launch_small_m<1, 16>(p, 1, stream);
    } else if (M <= 16) {
        p.splits = choose_splits(N / 64, K / 64, 1);
        e = launch_small_m<2, 16>(p, 1, stream);
    } else {
        const int tb = (M + 31) / 32;
        p.splits = choose_splits(N / 64, K / 64, tb);
        e = launch_small_m<4, 8>(p, tb, stream);
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

extern "C" void ternaspmm_accumulate_i32(int8_t* x, uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                                         uint32_t* sign_words, int32_t* out, int M, int N, int K,
                                         cudaStream_t stream) {
    run_spmm(x, bitmap, tile_offsets, quarter_offsets, sign_words, out, nullptr, nullptr, 1, M, N, K, EPI_RAW_I32,
             stream);
    checkLastCudaError(__LINE__);
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

extern "C" void gpu_sleep(double sleep_us, cudaStream_t stream) { sleep_kernel<<<1, 32, 0, stream>>>(sleep_us); }
