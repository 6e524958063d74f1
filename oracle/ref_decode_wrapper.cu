// Test infrastructure: builds the REFERENCE's own small-batch CUDA kernels
// (Gu-J/TernaInfer kernels/src/SpMM/SpMM_Kernel.cuh:16-163 and
// Reduction_Kernel.cuh:23-63) for sm_100a from the sources where they lie in
// the reference checkout, so that the GPU tests can compare the new library
// with the reference's own implementation on identical inputs.  Nothing of
// the reference is copied into this repository: the two headers are included
// from the checkout at build time (oracle/Makefile passes -I) and the output
// goes to oracle/_ref/, which is not committed.
//
// The reference's host launcher (kernels/src/TernaSpMM_API.cuh:40-136) cannot
// be included because that header pulls in an un-vendored CUTLASS; the few
// lines below restate what it does for the decode path: pick the tiling from
// the token count, size the dynamic shared memory, launch the SpMM kernel on
// grid (max(tokens/TILE_N,1), N_out*split_k/64) and then the split-K
// reduction on tokens*N_out/256 blocks of one warp.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "SpMM_Kernel.cuh"
#include "Reduction_Kernel.cuh"

namespace {

template <typename Cfg>
cudaError_t launch_ref_spmm(cudaStream_t st, const uint32_t* vals, const int* tile_off, const uint16_t* med_off,
                            const uint64_t* bitmap, const int8_t* x, int32_t* ws, int n_out, int tokens, int k,
                            int split_k) {
    const int pipeline = Cfg::TILE_N * TILE_K * 2 + Cfg::MY_MAX_INT8_NNZS_INTILE + Cfg::TILE_BITMAP_M_V3 * Cfg::TILE_BITMAP_K_V3 * 8;
    const int staging = (Cfg::TILE_M + PADDING_SHARED_MEM_FOR_C) * Cfg::TILE_N * 4;
    const int smem = pipeline > staging ? pipeline : staging;
    cudaError_t e = cudaFuncSetAttribute(mySpMM_Kernel_bitmap_v3<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int gx = tokens / Cfg::TILE_N > 0 ? tokens / Cfg::TILE_N : 1;
    dim3 grid(gx, n_out * split_k / Cfg::TILE_M, 1), block(WARP_SIZE * Cfg::BLOCK_WARPS, 1, 1);
    mySpMM_Kernel_bitmap_v3<Cfg><<<grid, block, smem, st>>>(vals, tile_off, med_off, bitmap, x, ws, n_out, tokens, k, split_k);
    return cudaGetLastError();
}

}  // namespace

// Same argument order as bitlinear_TernaSpMM_decode (kernels/TernaSpMM.cu:79).
// Returns a CUDA error code (0 = ok); tokens must be 8, 16, 32 or 64.
extern "C" int ref_bitlinear_TernaSpMM_decode(int8_t* x, uint64_t* bitmap, int* tile_off, uint16_t* med_off,
                                              uint32_t* vals, __nv_bfloat16* out, __nv_bfloat16* s,
                                              __nv_bfloat16* ws, int ws_num, int tokens, int n_out, int k,
                                              int split_k, int32_t* workspace, cudaStream_t st) {
    cudaError_t e;
    switch (tokens) {
        case 8: e = launch_ref_spmm<TilingConfigBitmapV3<4, 1, 1, 1>>(st, vals, tile_off, med_off, bitmap, x, workspace, n_out, tokens, k, split_k); break;
        case 16: e = launch_ref_spmm<TilingConfigBitmapV3<4, 1, 1>>(st, vals, tile_off, med_off, bitmap, x, workspace, n_out, tokens, k, split_k); break;
        case 32: e = launch_ref_spmm<TilingConfigBitmapV3<4, 1, 2>>(st, vals, tile_off, med_off, bitmap, x, workspace, n_out, tokens, k, split_k); break;
        case 64: e = launch_ref_spmm<TilingConfigBitmapV3<4, 1, 4>>(st, vals, tile_off, med_off, bitmap, x, workspace, n_out, tokens, k, split_k); break;
        default: return (int)cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return (int)e;
    SplitK_Reduction<<<dim3(n_out * tokens / 256, 1, 1), dim3(WARP_SIZE, 1, 1), 0, st>>>(out, workspace, n_out, tokens, split_k, s, ws, ws_num);
    return (int)cudaGetLastError();
}

// The reference's prefill stage 1 (kernels/src/SpMM/SpMM_Kernel.cuh:165-295, launched as in
// kernels/src/TernaSpMM_API.cuh:139-162): decompress the packed weight into a dense row-major
// int8 matrix dense[n_out][k] (the operand its CUTLASS GEMM then reads).  Needs no CUTLASS, so it
// pins the packed FORMAT of the prefill path with the reference's own code; the GEMM and its
// epilogue visitor cannot be built here.  Returns a CUDA error code.
extern "C" int ref_decompress_prefill(uint64_t* bitmap, int* tile_off, uint16_t* med_off, uint32_t* vals,
                                      int8_t* dense, int n_out, int k, int split_k, cudaStream_t st) {
    using Cfg = TilingConfigBitmapV3<4, 1, 1>;
    const int smem = Cfg::MY_MAX_INT8_NNZS_INTILE * 2 + Cfg::TILE_BITMAP_M_V3 * Cfg::TILE_BITMAP_K_V3 * 8;
    cudaError_t e = cudaFuncSetAttribute(mySpMM_Kernel_bitmap_prefill<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(1, n_out * split_k / Cfg::TILE_M, 1), block(WARP_SIZE * Cfg::BLOCK_WARPS, 1, 1);
    mySpMM_Kernel_bitmap_prefill<Cfg><<<grid, block, smem, st>>>(vals, tile_off, med_off, bitmap,
                                                                 reinterpret_cast<int32_t*>(dense), n_out, 1, k, split_k);
    return (int)cudaGetLastError();
}
