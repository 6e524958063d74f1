/*
 * libternaspmm.so - C ABI of the TernaSpMM operator for NVIDIA B200 (sm_100a).
 *
 * TernaSpMM is a linear layer  out[M,N] = x_q[M,K] * W[N,K]^T  with ternary
 * weights W in {-1,0,+1} stored compressed (1-bit non-zero bitmaps + packed
 * sign bits of the non-zeros + per-tile offsets), int8 activations x_q with a
 * per-token bf16 scale s, a 4-slot bf16 per-segment weight scale ws, and bf16
 * output.  The entry points, their argument order and their meaning are those
 * of the reference library (citations: file:line inside Gu-J/TernaInfer), so a
 * caller that binds the reference's libternaspmm.so binds this one unchanged.
 *
 * Plain C: pointers and sizes only.  bf16 values are passed as uint16_t bit
 * patterns; a CUDA stream is passed as an opaque pointer (cudaStream_t).
 *
 * Ownership: the caller owns every device buffer; the compute entry points
 * allocate nothing, never synchronise and never copy through the host, so
 * they may be called while the stream is being captured into a CUDA graph.
 *
 * Weight layout: the four arrays keep the reference's element types and
 * sizes (bitmap N*K/64 u64, tile_offsets N*K/4096+1 i32, quarter_offsets
 * 3*N*K/4096 u16, sign_words tile_offsets[last]/32 u32) but the order of the
 * 4096 weights inside a 64x64 tile is the B200 order produced by
 * convert_reorderd() / the Python packer, not the reference's mma.m16n8k16
 * order.  ternaspmm_transcode_reference_layout() converts arrays packed by the
 * reference's packer.  Requirements: N % 64 == 0, K % 64 == 0, M >= 1,
 * x / bitmap / sign_words 16-byte aligned, and sign_words readable for two
 * words (8 bytes) past its last word tile_offsets[last]/32 - 1: the kernels
 * fetch a lane's sign window as a pair of words without looking at its length.
 * (The reference's own caller allocates 32 spare bytes, tests/test_kernel.cu:
 * 257-288; the packers of this library pad 4 words.)
 */
#ifndef TERNASPMM_H_
#define TERNASPMM_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* ternaspmm_stream_t; /* cudaStream_t */
typedef uint16_t ternaspmm_bf16;  /* bf16 bit pattern */

/* One item of a work list (see ternaspmm_list_plan below). */
typedef struct {
    int8_t* x;                   /* int8 [M][K] */
    uint64_t* bitmap;
    int* tile_offsets;
    uint16_t* quarter_offsets;
    uint32_t* sign_words;
    ternaspmm_bf16* out;         /* bf16 [M][N] */
    ternaspmm_bf16* s;           /* bf16 [M] */
    ternaspmm_bf16* ws;          /* bf16 [4] */
    ternaspmm_bf16* residual;    /* bf16 [M][N] or null */
    int ws_num, M, N, K;
    int seg1, seg2, seg3;        /* explicit scale-segment boundaries; all zero = the reference's rule */
    int prefill_form;            /* 0 = decode epilogue, 1 = prefill epilogue, -1 = by token count */
} ternaspmm_list_item;

typedef struct ternaspmm_list ternaspmm_list;

#ifndef TERNASPMM_TYPES_ONLY   /* the library's own translation unit takes the types only */

/* ---- entry points that replace the reference's, same signatures -------- */

/* Replaces bitlinear_TernaSpMM (kernels/TernaSpMM.cu:25-71).  M <= 64 uses
 * the decode epilogue  bf16(float(acc)/s[t]*ws[g]), M > 64 the prefill
 * epilogue  bf16(float(acc)*(ws[g]/s[t])).  split_k and workspace are
 * accepted for compatibility; the K-split is chosen internally and reduced
 * through cluster shared memory, the workspace is never touched. */
void bitlinear_TernaSpMM(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                         uint16_t* quarter_offsets, uint32_t* sign_words,
                         ternaspmm_bf16* out, ternaspmm_bf16* s, ternaspmm_bf16* ws,
                         int ws_num, int M, int N, int K, int split_k,
                         int32_t* workspace, ternaspmm_stream_t stream);

/* Replaces bitlinear_TernaSpMM_decode (kernels/TernaSpMM.cu:79-107): decode
 * epilogue for any M. */
void bitlinear_TernaSpMM_decode(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                                uint16_t* quarter_offsets, uint32_t* sign_words,
                                ternaspmm_bf16* out, ternaspmm_bf16* s, ternaspmm_bf16* ws,
                                int ws_num, int M, int N, int K, int split_k,
                                int32_t* workspace, ternaspmm_stream_t stream);

/* Replaces bitlinear_TernaSpMM_prefill (kernels/TernaSpMM.cu:110-138):
 * prefill epilogue for any M. */
void bitlinear_TernaSpMM_prefill(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                                 uint16_t* quarter_offsets, uint32_t* sign_words,
                                 ternaspmm_bf16* out, ternaspmm_bf16* s, ternaspmm_bf16* ws,
                                 int ws_num, int M, int N, int K, int split_k,
                                 int32_t* workspace, ternaspmm_stream_t stream);

/* Replaces bitlinear_TernaSpMM_benchmark (kernels/TernaSpMM.cu:141-236):
 * mode 0/1/2 = auto/prefill/decode (out of range -> 0); warm-up, CUDA-event
 * timing loop, prints "Shape(M=.., N=.., K=..): %.2f us ...".  Synchronises. */
void bitlinear_TernaSpMM_benchmark(int mode, int warmup_iters, int bench_iters,
                                   int8_t* x, uint64_t* bitmap, int* tile_offsets,
                                   uint16_t* quarter_offsets, uint32_t* sign_words,
                                   ternaspmm_bf16* out, ternaspmm_bf16* s, ternaspmm_bf16* ws,
                                   int ws_num, int M, int N, int K, int split_k,
                                   int32_t* workspace, ternaspmm_stream_t stream);

/* Replaces checkLastCudaError (kernels/TernaSpMM.cu:15-22): prints and
 * exit(EXIT_FAILURE) when cudaGetLastError() reports an error. */
void checkLastCudaError(int line);

/* Replaces reorder_WT_h (kernels/TernaSpMM.cu:241-280).  Host buffers, bf16
 * [N][K].  The B200 layout needs no pre-permutation, so this is a copy; it is
 * kept so that callers written against the reference (tests/test_kernel.cu:
 * 253) keep working. */
void reorder_WT_h(ternaspmm_bf16* W, ternaspmm_bf16* W_reordered, int N, int K);

/* Replaces convert_reorderd (kernels/TernaSpMM.cu:282-439): host packer.
 * Input bf16 [N][K] holding {-1,0,+1}.  The six tile arguments must be
 * 64,16,8,64,64,8 as in the reference's only call (tests/test_kernel.cu:255).
 * Allocates the outputs like the reference: tile_offsets, quarter_offsets and
 * sign_words with malloc (caller frees), bitmap with cudaMallocHost (caller
 * cudaFreeHost).  *max_nnz receives the largest padded per-tile count (the
 * reference declares this parameter as int&, the same ABI).  Returns the
 * number of 64x64 tiles or -1. */
int convert_reorderd(ternaspmm_bf16* W, int N, int K, int tile_N, int warp_subtile_N,
                     int subtile_N, int tile_K, int warp_subtile_K, int subtile_K,
                     uint64_t** bitmap, int** tile_offsets, uint16_t** quarter_offsets,
                     uint32_t** sign_words, int* max_nnz);

/* Replaces gpu_sleep (kernels/TernaSpMM.cu:442-457): a one-warp spacer kernel
 * that waits sleep_us microseconds (bounded at one second). */
void gpu_sleep(double sleep_us, ternaspmm_stream_t stream);

/* ---- additions (no counterpart in the reference) ------------------------ */

/* Status of the most recent compute call on this thread's device: 0 = ok,
 * 1 = bad shape, 2 = bad pointer/alignment, 3 = launch failure (also a failed
 * tensor-map encode: nothing was launched), 4 = a bounded device-side wait ran
 * out (an mbarrier hand-off inside the tensor-core kernel, or a peer's signal
 * in the fused tensor-parallel tail) and the kernel returned early.  Reading
 * the device word synchronises the device; do not call while capturing. */
int ternaspmm_last_status(void);

/* Limit of the device-side wait for a peer's signal in
 * ternaspmm_tp_allreduce_finish, in milliseconds of the GPU's global timer
 * (default 1000, clamped to 1..10000).  Process-wide. */
void ternaspmm_set_wait_limit_ms(int ms);

/* Measurement hook: int8 tensor-core operations per second that the GPU issues with tcgen05.mma
 * (128 x 256 x 32 per instruction, operands resident in shared memory, one CTA per SM, `iters` groups of
 * four instructions per SM) - the ceiling that the tensor-core kernels of this library are quoted
 * against in bench.py.  Synchronises the stream; returns 0 on failure. */
double ternaspmm_debug_int8_mma_rate(int iters, ternaspmm_stream_t stream);

/* Test hook: shape of the most recent kernel launch made by this thread.
 * out6 = {kernel (1 = small-batch kernel, one fat CTA per SM; 2 = small-batch
 * kernel, thin CTAs; 3 = tcgen05 kernel; 4 = output head; 5 = work list; 6 = tcgen05 kernel
 * on dense weights from the workspace, single CTAs; 7 = the same on CTA pairs), tokens per pass, K split (cluster
 * size), warps per CTA, 64-row tiles per CTA, CTAs}. */
void ternaspmm_last_launch_shape(int* out6);

/* Test hook (host-side fault injection): kind 1 makes the next tensor-map
 * encode of this thread report failure, so the call ends with status 3
 * without launching anything. */
void ternaspmm_debug_inject_host_failure(int kind);

/* Test hook: same contraction, raw int32 accumulators out[M][N]. */
void ternaspmm_accumulate_i32(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                              uint16_t* quarter_offsets, uint32_t* sign_words,
                              int32_t* out, int M, int N, int K,
                              ternaspmm_stream_t stream);

/* Same operator with explicit scale-segment boundaries instead of the
 * reference's hard-coded rules (equal widths, or 2560/640/640 when N == 3840):
 * output column n uses ws[(n >= seg1) + (n >= seg2) + (n >= seg3)], limited to
 * ws_num-1; unused boundaries are ignored.  Needed for head-sharded QKV and
 * for models whose q/k/v widths are not BitNet-2B's.  prefill_form: 0 = decode
 * epilogue, 1 = prefill epilogue, -1 = by token count like bitlinear_TernaSpMM. */
void ternaspmm_linear_segments(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                               uint16_t* quarter_offsets, uint32_t* sign_words,
                               ternaspmm_bf16* out, ternaspmm_bf16* s, ternaspmm_bf16* ws,
                               int ws_num, int M, int N, int K, int seg1, int seg2, int seg3,
                               int prefill_form, ternaspmm_stream_t stream);

/* bitlinear_TernaSpMM with the residual add of the decoder block fused into
 * the epilogue: out = bf16(residual + bf16(linear(x))), residual bf16 [M][N]
 * (may alias out; null = plain linear). */
void bitlinear_TernaSpMM_residual(int8_t* x, uint64_t* bitmap, int* tile_offsets,
                                  uint16_t* quarter_offsets, uint32_t* sign_words,
                                  ternaspmm_bf16* out, ternaspmm_bf16* s, ternaspmm_bf16* ws,
                                  int ws_num, int M, int N, int K, ternaspmm_bf16* residual,
                                  ternaspmm_stream_t stream);

/* bitlinear_TernaSpMM_residual with the workspace of the reference's prefill path and its size.  The
 * reference's prefill path decompresses the weight into a dense int8 matrix W[N][K] in the workspace
 * before its GEMM (kernels/src/TernaSpMM_API.cuh:139-162, 262-285), so its callers already hold N*K
 * bytes there (model.py:34-42 allocates the largest layer's).  When workspace_bytes >= N*K and the call
 * has at least 384 tokens (1024 for layers with K > 4096), this entry decodes the weight once per call
 * into the workspace (which stays in L2 at these sizes) and runs a tcgen05 kernel on CTA pairs
 * (256 x 256 tiles, both operands by TMA), instead of decoding every weight tile once per 256-token
 * tile on chip; otherwise it behaves like bitlinear_TernaSpMM_residual.  path: 0 = choose, 1 = never
 * use the workspace, 2 = always (needs the N*K bytes).  workspace 128-byte aligned; results are
 * bit-identical either way. */
void bitlinear_TernaSpMM_ws(int8_t* x, uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                            uint32_t* sign_words, ternaspmm_bf16* out, ternaspmm_bf16* s, ternaspmm_bf16* ws,
                            int ws_num, int M, int N, int K, ternaspmm_bf16* residual, void* workspace,
                            long long workspace_bytes, int path, ternaspmm_stream_t stream);

/* Fused front-end of a ternary linear: y = RMSNorm(x) * norm_weight (fp32 sum
 * of squares, bf16 result), then the per-token absmax int8 quantiser of
 * model.py:120-123: s = 127 / clamp(max|y|, 1e-5), q = clamp(round(y*s)).
 * One kernel instead of the reference's RMSNorm + Triton quantiser chain.
 * x bf16 [M][K], norm_weight bf16 [K], q int8 [M][K], s_out bf16 [M];
 * K a multiple of 16, at most 57344; x, norm_weight, q 16-byte aligned. */
void ternaspmm_rmsnorm_quant(ternaspmm_bf16* x, ternaspmm_bf16* norm_weight, float eps, int M, int K,
                             int8_t* q, ternaspmm_bf16* s_out, ternaspmm_stream_t stream);

/* The same for the input of the down projection (model.py:277-282): x13 bf16
 * [M][2K] holds [x1 | x3]; y = RMSNorm(relu(x1)^2 * x3) * norm_weight. */
void ternaspmm_relu2_gate_rmsnorm_quant(ternaspmm_bf16* x13, ternaspmm_bf16* norm_weight, float eps, int M,
                                        int K, int8_t* q, ternaspmm_bf16* s_out, ternaspmm_stream_t stream);

/* RMSNorm alone, in the summation order of ternaspmm_rmsnorm_quant: y = bf16((x * rstd) * norm_weight),
 * rstd = 1 / sqrt(sum(x^2) / K + eps).  One launch instead of the chain of elementwise kernels of an
 * eager RMSNorm (the model's final norm in front of the output head, model.py:385 of the reference).
 * x, y bf16 [M][K] (y may alias x), norm_weight bf16 [K]; K a multiple of 16, at most 57344; 16-byte
 * aligned pointers. */
void ternaspmm_rmsnorm(ternaspmm_bf16* x, ternaspmm_bf16* norm_weight, float eps, int M, int K, ternaspmm_bf16* y,
                       ternaspmm_stream_t stream);

/* Plain per-token absmax quantiser (model.py:120-123) as one kernel. */
void ternaspmm_quant(ternaspmm_bf16* x, int M, int K, int8_t* q, ternaspmm_bf16* s_out,
                     ternaspmm_stream_t stream);

/* Front-end of a row-parallel (K-sharded) linear: y = x * weight WITHOUT the RMS factor
 * (gated != 0: x holds [x1 | x3] and the value is relu(x1)^2 * x3), quantised per token with
 * the shard's own absmax; ss_out[t] = this shard's sum of squares, to be all-reduced. */
void ternaspmm_scale_quant_sumsq(ternaspmm_bf16* x, ternaspmm_bf16* weight, int gated, int M, int K,
                                 int8_t* q, ternaspmm_bf16* s_out, float* ss_out,
                                 ternaspmm_stream_t stream);

/* Contraction with fp32 output out[t][n] = float(acc) / s[t] (no weight scale): the partial
 * result of one K shard, ready for a sum all-reduce. */
void ternaspmm_partial_f32(int8_t* x, uint64_t* bitmap, int* tile_offsets, uint16_t* quarter_offsets,
                           uint32_t* sign_words, float* out, ternaspmm_bf16* s, int M, int N, int K,
                           ternaspmm_stream_t stream);

/* Tail of a row-parallel linear after the all-reduce: buf = fp32 [M*N] summed partials followed
 * by fp32 [M] summed squares; out = bf16(buf * rsqrt(ss/full_width + eps) * ws[0]) (+ residual). */
void ternaspmm_tp_finish(float* buf, ternaspmm_bf16* ws, float eps, int full_width, int M, int N,
                         ternaspmm_bf16* residual, ternaspmm_bf16* out, ternaspmm_stream_t stream);

/* The same tail with the all-reduce fused in, for one process per GPU with peer-mapped (symmetric)
 * buffers.  bufs[r] / flags[r] / outs[r] = rank r's partial buffer (fp32 [M*N] partials + [M] sums
 * of squares, written by ternaspmm_partial_f32 / ternaspmm_scale_quant_sumsq), flag array (uint32
 * [16], zero-initialised once) and bf16 output buffer [M*N], as mapped in THIS process; counters =
 * two local uint32 (zero-initialised) of this call site.  Every rank launches it once per call.  It
 * signals the peers, waits until all of them have signalled, reduces ITS slice of the outputs over
 * all ranks' partials (plain peer loads over NVLink, rank order), applies the RMS factor, ws[0] and
 * the optional residual, pushes the finished bf16 slice into every rank's output buffer (plain peer
 * stores), and returns only after every peer's slice has arrived: the result is outs[rank].  All
 * waits are bounded (ternaspmm_set_wait_limit_ms); when one runs out, status 4 is recorded and
 * outs[rank] is filled with bf16 NaN.  Each call site needs its own buffers, flags and counters; a
 * call site's buffers may be reused by its next call without any further synchronisation. */
void ternaspmm_tp_allreduce_finish(float** bufs, unsigned int** flags, ternaspmm_bf16** outs, int rank,
                                   int world, unsigned int* counters, ternaspmm_bf16* ws, float eps,
                                   int full_width, int M, int N, ternaspmm_bf16* residual,
                                   ternaspmm_stream_t stream);

/* ---- work lists: many independent small-batch linears in one persistent launch ------------------
 * One item is what one call of bitlinear_TernaSpMM / ternaspmm_linear_segments /
 * bitlinear_TernaSpMM_residual computes, for 1 <= M <= 16 tokens.  A list runs all its items in ONE
 * kernel launch: a CTA per SM stays resident, builds the decode tables once and streams the items'
 * weights back to back, so the per-call costs (launch, table build, dependency wait, grid drain)
 * are paid once per list instead of once per linear.  The items must be independent: no item may
 * read what another item of the same list writes.  Results are bit-identical to the per-call
 * entry points.  Usage: ternaspmm_list_plan() -> sizes; the caller allocates the device table and
 * the scratch area; ternaspmm_list_create() uploads the table and zeroes the scratch area
 * (synchronises the stream; not while capturing); ternaspmm_list_run() launches (no allocation,
 * no synchronisation: may be captured into a CUDA graph, any number of times);
 * ternaspmm_list_destroy() frees the host-side handle.  Runs of lists that share a scratch area
 * must not overlap on the GPU.  If a run ends with status 4, zero the scratch area before reuse. */
/* Number of device table entries (= items), or -1 for a bad item or more than 256 items;
 * *table_bytes / *scratch_bytes receive the sizes of the two device buffers. */
int ternaspmm_list_plan(const ternaspmm_list_item* items, int n_items, long long* table_bytes,
                        long long* scratch_bytes);
ternaspmm_list* ternaspmm_list_create(const ternaspmm_list_item* items, int n_items, void* device_table,
                                      void* scratch, ternaspmm_stream_t stream);
void ternaspmm_list_run(ternaspmm_list* list, ternaspmm_stream_t stream);
void ternaspmm_list_destroy(ternaspmm_list* list);

/* Output head for decode-sized batches: logits[t][v] = sum_k h[t][k] * embedding[v][k] for
 * 1 <= M <= 8 rows of hidden states, bf16 inputs, fp32 accumulation, and the greedy token per
 * row, in one launch that reads the embedding once.  Replaces the dense bf16 GEMM over the tied
 * embedding (model.py:367, :385 of the reference) plus the torch.argmax of its generation loop
 * (generate.py:283, :305) for decode steps.  logits: fp32 [M][V] or null; with round_bf16 != 0
 * every value is rounded to bf16 first, as the reference's bf16 linear returns it.  argmax:
 * int64 [M] or null: index of the largest (rounded) logit, smallest index on ties.  scratch:
 * ternaspmm_lm_head_scratch_bytes() bytes of device memory, zero-initialised once by the caller
 * (the kernel leaves its counter at zero); calls that share a scratch area must not overlap on
 * the GPU.  K a multiple of 32, at most 12288; h, embedding and scratch 16-byte aligned. */
void ternaspmm_lm_head_argmax(ternaspmm_bf16* h, ternaspmm_bf16* embedding, int M, int V, int K, float* logits,
                              long long* argmax, int round_bf16, void* scratch, ternaspmm_stream_t stream);
long long ternaspmm_lm_head_scratch_bytes(void);

/* No counterpart in the reference.  ternaspmm_lm_head_argmax for callers that cannot provide
 * scratch memory - an operator inside a runtime that owns all device memory and forbids
 * cudaMalloc, a latency-critical loop that must not hit the device-wide synchronisation of an
 * allocation, code running under stream capture.  Same arguments minus `scratch`: the arg-max
 * candidates and the arrival counter live in a 16 KB array inside the library image (held by every
 * GPU that loads the library until the process exits).  Limits: 1 <= M <= 8 rows (what the built-in
 * area has room for; more is rejected with status 1 and a message), K a multiple of 32 up to 12288,
 * at most 256 CTAs.  Nothing is allocated or freed, here or in a library routine.  The first call on
 * a device looks up the array's device address (cudaGetSymbolAddress); make that first call outside
 * any stream capture.  All calls on a device share the one area: it is cleared where it must start
 * from zero at the head of every call, and calls that overlap on the GPU (different streams) race. */
void ternaspmm_lm_head_argmax_noalloc(ternaspmm_bf16* h, ternaspmm_bf16* embedding, int M, int V, int K,
                                      float* logits, long long* argmax, int round_bf16,
                                      ternaspmm_stream_t stream);

/* Host packer from int8 ternary [N][K] into caller-provided arrays
 * (bitmap N*K/64, tile_offsets tiles+1, quarter_offsets 3*tiles, sign_words
 * at least N*K/32 + 4 words, zero-filled by the call).  Returns the number of
 * sign words used, or -1. */
long long ternaspmm_pack_i8(const int8_t* W, int N, int K, uint64_t* bitmap,
                            int* tile_offsets, uint16_t* quarter_offsets,
                            uint32_t* sign_words);

/* Inverse of the packer (host): writes int8 ternary [N][K]. Returns 0/-1. */
int ternaspmm_unpack_i8(const uint64_t* bitmap, const int* tile_offsets,
                        const uint32_t* sign_words, int N, int K, int8_t* W);

/* Host transcoder: arrays packed by the reference's compress_weight
 * (convert/convert_utils.py:52-228) -> B200 layout.  tile_offsets are the
 * same in both layouts; bitmap, sign_words and the three per-tile u16 are
 * rewritten into the out_* arrays (same sizes as the inputs). */
int ternaspmm_transcode_reference_layout(const uint64_t* ref_bitmap, const int* tile_offsets,
                                         const uint32_t* ref_sign_words, int N, int K,
                                         uint64_t* out_bitmap, uint16_t* out_quarter_offsets,
                                         uint32_t* out_sign_words);

#endif /* TERNASPMM_TYPES_ONLY */

#ifdef __cplusplus
}
#endif
#endif /* TERNASPMM_H_ */
