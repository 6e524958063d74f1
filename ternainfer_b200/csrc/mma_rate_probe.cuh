// Measurement hook: the rate at which one SM issues tcgen05.mma kind::i8 (M = 128, N = 256, K = 32) when
// both operands sit in shared memory and nothing else runs - the ceiling for the tensor-core kernels of
// this library (spmm_large_m.cuh, dense_pair.cuh), which the roofline figures of the prefill path are
// quoted against.  One CTA per SM: allocate tensor memory, fill 48 KB of operands with arbitrary bytes,
// issue `iters` groups of four MMAs (alternating between two accumulators), commit every 64 groups and
// wait for the commit with a bounded wait.  No counterpart in the reference.
#pragma once
#include "spmm_large_m.cuh"

namespace tsp {

__global__ void __launch_bounds__(128, 1) int8_mma_rate_kernel(int iters, int* status) {
    extern __shared__ __align__(128) uint8_t probe_smem[];
    const uint32_t dyn = smem_u32(probe_smem);
    const uint32_t base = (dyn + 1023u) & ~1023u;
    uint8_t* p = probe_smem + (base - dyn);
    const uint32_t bar = base, slot = base + 16, A = base + 1024, B = A + kLgAStage;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(p + 32);
    for (int i = threadIdx.x; i < (kLgAStage + 256 * kLgKStep) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(p + 1024)[i] = ((uint32_t)i * 2654435761u) ^ ((uint32_t)i >> 3);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    if (threadIdx.x < 32) tmem_alloc(slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(p + 16);
    if (threadIdx.x == 0) {
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | (8u << 24);
        uint32_t parity = 0;
        bool ok = true;
        for (int it = 0; it < iters && ok; it += 64) {
            for (int k = 0; k < 64; ++k)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    umma_i8(tmem + (uint32_t)((k & 1) * 256), umma_desc_sw128(A + 32 * j), umma_desc_sw128(B + 32 * j), idesc, 1u);
            umma_commit(bar);
            ok = wait_or_abort(bar, parity, abort_flag);
            parity ^= 1;
        }
        if (!ok) atomicExch(status, ST_WAIT_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

}  // namespace tsp
