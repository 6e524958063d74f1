// Decompress kernel of the large-batch path with a workspace, for sm_100a.
//
// At hundreds or thousands of tokens the tcgen05 kernel that decodes the packed weights on chip
// (spmm_large_m.cuh) decodes every weight tile once per 256-token tile - eight times at 2048 tokens -
// and its decoder warps, not its tensor cores, set the pace.  When the caller provides the workspace
// the reference's own prefill path requires (N*K bytes: its decompress kernel writes the dense int8
// matrix there, kernels/src/SpMM/SpMM_Kernel.cuh:165-295 of Gu-J/TernaInfer, before the CUTLASS GEMM
// reads it back), the weights are decoded ONCE per call by this kernel into that workspace - dense
// int8 W[N][K], row-major, which at BitNet-2B sizes (35 MB at most) stays in the 126 MB L2 - and the
// tensor-core kernel then takes both operands by TMA.
//
// Persistent CTAs, one per SM; every warp takes tiles warp, warp + W, ... of the weight with the
// same register pipeline and table decode as the small-batch kernels and writes each lane's
// sixteen consecutive k of a row as one 16-byte store.
#pragma once
#include "spmm_small_m.cuh"

namespace tsp {

constexpr int kDecompressWarps = 20;

__global__ void __launch_bounds__(kDecompressWarps * 32, 1) decompress_kernel(const SpmmParams p, int8_t* __restrict__ dense) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t dyn = (smem_u32(smem) + 127u) & ~127u;
    const uint32_t lut_base = (dyn + (uint32_t)kLutBytes - 1u) & ~((uint32_t)kLutBytes - 1u);
    const uint32_t sbase = (lut_base - dyn >= 2048u) ? dyn : lut_base + kLut2Bytes;
    uint32_t* lut1 = reinterpret_cast<uint32_t*>(smem + (sbase - smem_u32(smem)));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int KT = p.K >> 6;
    const long long tiles = (long long)(p.N >> 6) * KT;
    const long long stride = (long long)gridDim.x * kDecompressWarps;

    griddep_launch_dependents();
    for (int e = tid; e < 512; e += blockDim.x) lut1[e] = e < 256 ? lut_entry(e) : lut_entry_upper(e - 256);
    __syncthreads();
    for (int i = tid; i < 512 * 8; i += blockDim.x) sts128(lut_base + i * 16, make_uint4(lut1[i >> 3], lut1[i >> 3], lut1[i >> 3], lut1[i >> 3]));
    __syncthreads();
    const uint32_t lut_lo = lut_base | (uint32_t)(lane * 4), lut_hi = lut_lo + kLutBytes;

    long long t = (long long)blockIdx.x + (long long)gridDim.x * warp;   // consecutive tiles go to different SMs
    TileHead h0 = load_head(p, t, t < tiles, lane);
    TileHead h1 = load_head(p, t + stride, t + stride < tiles, lane);
    TileSigns s0 = load_signs(p, h0, t < tiles, lane);
    griddep_wait();   // the workspace may still be read by the previous kernel of the stream
    for (; t < tiles; t += stride) {
        const TileHead h2 = load_head(p, t + 2 * stride, t + 2 * stride < tiles, lane);
        const TileSigns s1 = load_signs(p, h1, t + stride < tiles, lane);
        const int rt = (int)(t / KT), kt = (int)(t - (long long)rt * KT);
        // lane (g, q), word r, half h: row 64 rt + 16 r + 8 h + g, k 64 kt + 16 q .. + 15
        int8_t* dst = dense + ((size_t)rt * 64 + g) * p.K + (size_t)kt * 64 + q * 16;
        const uint32_t w[4] = {h0.bw.x, h0.bw.y, h0.bw.z, h0.bw.w};
        int pos = s0.pos;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            uint32_t a[8];
            const int c = __popc(w[r]);
            decode_word2(w[r], __funnelshift_r(s0.lo[r], s0.hi[r], (uint32_t)pos), c, lut_lo, lut_hi, a);
            pos += c;
#pragma unroll
            for (int h = 0; h < 2; ++h)
                *reinterpret_cast<uint4*>(dst + (size_t)(16 * r + 8 * h) * p.K) = make_uint4(a[h], a[2 + h], a[4 + h], a[6 + h]);
        }
        h0 = h1, h1 = h2, s0 = s1;
    }
}

}  // namespace tsp
