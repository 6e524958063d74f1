/*
 * CPU oracle for the TernaSpMM path, plain C.  TEST INFRASTRUCTURE ONLY: the
 * product library never links or calls this file; it is the checker in the
 * tests and the timed CPU baseline of the benchmark.
 *
 * Restates the arithmetic of Gu-J/TernaInfer (paths inside that repository):
 *   contraction  acc[t][n] = sum_k x[t][k] * W[n][k], int32 exact
 *                (kernels/src/SpMM/MatMulUtilities.cuh:180-224, the int8 MMA;
 *                 kernels/src/TernaSpMM_API.cuh:166-207, the CUTLASS int8 GEMM)
 *   decode epilogue   bf16_rn(float(acc) / s[t] * ws[g])
 *                (kernels/src/SpMM/Reduction_Kernel.cuh:42-62)
 *   prefill epilogue  bf16_rn(float(acc) * (ws[g] / s[t])), 0 when s == 0
 *                (kernels/src/GEMM/epilogue_visitor_scale_ws.h:135-148,183-210)
 * The reference has no CPU GEMM of its own (its test compares against cuBLAS
 * on the GPU, tests/test_kernel.cu:148-230), so this is a restatement of the
 * formulas, pinned by the numpy oracle and the reference packer's golden
 * vectors rather than by a reference CPU routine: parity of the arithmetic is
 * otherwise unpinned.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC -o oracle/libternaspmm_oracle.so oracle/ternaspmm_oracle.c
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16_rn(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FC0; /* NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; a timing run sets the thread count itself. */
void oracle_set_num_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* One weight row against all token rows; cloned per ISA so the library built
 * on one machine runs at full speed (and never faults) on another. */
__attribute__((target_clones("arch=skylake-avx512", "arch=haswell", "default")))
static void dot_row(const int8_t* w, const int8_t* x, int M, int N, int K, int32_t* acc_col) {
    for (int t = 0; t < M; ++t) {
        const int8_t* xr = x + (size_t)t * K;
        int32_t sum = 0;
        for (int k = 0; k < K; ++k) sum += (int32_t)xr[k] * (int32_t)w[k];
        acc_col[(size_t)t * N] = sum;
    }
}

/* acc[M][N] int32 from dense ternary W[N][K] and int8 x[M][K]. */
void oracle_gemm_i32(const int8_t* x, const int8_t* W, int M, int N, int K, int32_t* acc) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) dot_row(W + (size_t)n * K, x, M, N, K, acc + n);
}

static int group_decode(int n, int N, int ws_num) {
    int col = n & ~7;
    if (ws_num == 3 && N == 3840) return col < 2560 ? 0 : (col < 3200 ? 1 : 2);
    return col / (N / ws_num);
}

static int group_prefill(int n, int N, int ws_num) {
    int col = n & ~127, g;
    if (N == 3840) g = col < 2560 ? 0 : (col < 3200 ? 1 : 2);
    else g = col / (N / ws_num);
    return g < ws_num ? g : ws_num - 1;
}

/* mode 0 = decode epilogue, 1 = prefill epilogue.  s, ws, out are bf16 bits. */
void oracle_epilogue(const int32_t* acc, const uint16_t* s, const uint16_t* ws, int ws_num, int M, int N, int mode,
                     uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < M; ++t) {
        const float s_el = bf16_to_f32(s[t]);
        for (int n = 0; n < N; ++n) {
            const float a = (float)acc[(size_t)t * N + n];
            float v;
            if (mode == 0) {
                const float w = bf16_to_f32(ws[group_decode(n, N, ws_num)]);
                volatile float q = a / s_el; /* keep the two roundings separate */
                v = q * w;
            } else {
                const float w = bf16_to_f32(ws[group_prefill(n, N, ws_num)]);
                volatile float c = (s_el != 0.f) ? w / s_el : 0.f;
                v = a * c;
            }
            out[(size_t)t * N + n] = f32_to_bf16_rn(v);
        }
    }
}

/* Whole operator on dense ternary weights; mode -1 = dispatcher rule
 * (tokens <= 64 -> decode, kernels/TernaSpMM.cu:34). */
void oracle_ternaspmm(const int8_t* x, const int8_t* W, const uint16_t* s, const uint16_t* ws, int ws_num, int M,
                      int N, int K, int mode, int32_t* acc_scratch, uint16_t* out) {
    oracle_gemm_i32(x, W, M, N, K, acc_scratch);
    if (mode < 0) mode = M <= 64 ? 0 : 1;
    oracle_epilogue(acc_scratch, s, ws, ws_num, M, N, mode, out);
}
