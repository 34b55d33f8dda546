/*
 * C ABI of libmach_b200.so: the sm_100a implementation of the quantized-linear hot path
 * (dynamic activation quantisation, block-scaled GEMM, SwiGLU + requant epilogue,
 * residual + RMSNorm + requant) behind the vllm-mach plugin API.
 *
 * Conventions
 *  - Every pointer is a device pointer owned by the caller unless stated otherwise.
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and nothing
 *    synchronises. No compute entry point allocates device memory (only the explicit
 *    mach_ar_buffer_* / mach_ar_ipc_* set-up calls do).
 *  - Return value: 0 on success, otherwise one of MACH_ERR_*; mach_last_error() gives text.
 *  - Row-major, contiguous unless a leading dimension is given.
 *
 * Scale layouts
 *  - "swizzled" E8M0 scales: the 128-row x 4-group atom of
 *    src/vllm_mach/mxfp6/mxfp8_mlp.py:107-110; byte offset of (row, group) is
 *    ((((row/128)*ceil(K/128) + group/4)*32 + row%32)*4 + (row%128)/32)*4 + group%4 and the
 *    buffer holds ceil(rows/128)*128*ceil(K/128)*4 bytes (mach_mx_sf_bytes).
 *  - "logical" E8M0 scales: uint8 [rows, K/32] row-major (checkpoint format,
 *    tests/native_mxfp6/test_mxfp8_sm120.py:33-39).
 */
#ifndef MACH_B200_H_
#define MACH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MACH_ABI_VERSION 3

#if defined(__GNUC__)
#define MACH_API __attribute__((visibility("default")))
#else
#define MACH_API
#endif

#define MACH_OK 0
#define MACH_ERR_INVALID 1      /* null pointer, negative size, misaligned pointer */
#define MACH_ERR_UNSUPPORTED 2  /* shape outside what the kernels implement */
#define MACH_ERR_CUDA 3         /* a CUDA runtime / driver call failed */
#define MACH_ERR_DEVICE 4       /* a bounded device wait gave up (see mach_device_status) */

/* Weight element formats of the block-scaled GEMM. */
#define MACH_FMT_E4M3 0 /* 1 byte per element, row = K bytes */
#define MACH_FMT_E2M3 3 /* 6-bit, 4 codes per 3 bytes, row = 3K/4 bytes */
#define MACH_FMT_E3M2 4 /* 6-bit, 4 codes per 3 bytes, row = 3K/4 bytes */

/* Row order of a weight matrix. */
#define MACH_LAYOUT_ROWS 0       /* rows as in the checkpoint ([gate rows | up rows] for gate_up) */
#define MACH_LAYOUT_GATE_UP_32 1 /* gate_up rows interleaved in groups of 32: physical rows
                                    [64j, 64j+32) = gate features [32j, 32j+32), the next 32 rows
                                    the matching up features (mach_mx_interleave_gate_up) */

MACH_API int mach_abi_version(void);
/* Text of the last error on the calling thread ("" if none). Host memory, never freed. */
MACH_API const char* mach_last_error(void);
/* Reads (synchronously) the device status word: 0 healthy, else the code of the first
 * device-side wait that gave up. Clears it when `clear` is non-zero. The hundreds digit names
 * the kernel (1 feature-major MX GEMM, 2 block-FP8 tile GEMM, 3 single-CTA persistent MX GEMM,
 * 4 fused all-reduce: 401 partial-sum flag, 402 result flag, 403 failed workspace, 5 grouped
 * MoE GEMM, 6 CTA-pair MX GEMM, 7 persistent block-FP8 GEMM, 8 one-token-tile MX GEMM); the
 * units digit the barrier (1 free stage, 2 filled stage, 3 finished accumulator, 4 drained
 * accumulator). */
MACH_API int mach_device_status(int* status_out, int clear);

/* Bytes of a swizzled E8M0 scale buffer for `rows` x K. */
MACH_API size_t mach_mx_sf_bytes(int64_t rows, int64_t k);

/* BF16 [M,K] (leading dimension ldx elements) -> E4M3 codes [M,K] + swizzled E8M0 scales.
 * Replaces torch.ops.mxfp6.quantize_mxfp8 (src/vllm_mach/mxfp6/dense_mxfp8.py:40) with the
 * rule of src/vllm_mach/mxfp6/mxfp8_norm_quant.py:29-39. K % 32 == 0. */
MACH_API int mach_mxfp8_quantize(const void* x_bf16, int64_t ldx, void* codes, void* scales, int64_t m,
                        int64_t k, void* stream);

/* BF16 [M, 2I] = [gate | up] -> MXFP8 of bf16(bf16(silu(gate)) * up): codes [M,I] + swizzled
 * scales. Replaces _silu_quant (src/vllm_mach/mxfp6/mxfp8_mlp.py:87-110). I % 32 == 0. */
MACH_API int mach_swiglu_mxfp8_quantize(const void* gate_up_bf16, void* codes, void* scales, int64_t m,
                               int64_t i, void* stream);

/* The same producer with the reference's OTHER SwiGLU contract ("champion", for its MXFP8
 * 4B/2B profile, src/vllm_mach/mxfp8/swiglu_quant.py:46-70; the two must not be mixed up):
 * v = bf16(silu(gate) * up) with ONE BF16 rounding; E8M0 = smallest power of two >=
 * amax * rcp.approx(448) (cvt.rp.satfinite.ue8m0x2); codes = e4m3(clamp(v * rcp.approx(2^e)));
 * an all-zero block stores scale byte 0 and zero codes. */
MACH_API int mach_swiglu_mxfp8_quantize_champion(const void* gate_up_bf16, void* codes,
                                                 void* scales, int64_t m, int64_t i,
                                                 void* stream);

/* s = x + residual (FP32); residual_out = bf16(s);
 * y = bf16(s * rsqrt(mean(s^2) + eps) * (weight + weight_bias)); then MXFP8 of y.
 * Replaces _norm / _norm_quant (src/vllm_mach/mxfp6/gemma_norm.py:13-29,
 * src/vllm_mach/mxfp6/mxfp8_norm_quant.py:15-39). residual may be NULL (no add, residual_out
 * ignored); norm_out may be NULL; codes+scales may both be NULL (no quantisation).
 * residual_out may alias x or residual. H % 32 == 0, H <= 16384. */
MACH_API int mach_add_rmsnorm_mxfp8(const void* x_bf16, const void* residual_bf16, const void* weight_bf16,
                           float eps, float weight_bias, void* norm_out_bf16,
                           void* residual_out_bf16, void* codes, void* scales, int64_t m,
                           int64_t h, void* stream);

/* Tail of the fused all-reduce for an already reduced BF16 sum `a`:
 * res = bf16(a + residual); norm = bf16(res * rsqrt(mean(res^2) + eps) * (weight_bias + gamma)),
 * the norm being taken of the BF16-ROUNDED sum; then MXFP8 of norm. Same arguments as
 * mach_add_rmsnorm_mxfp8. Follows FusedOp / rms_norm of
 * native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh:1092-1108,1303-1342. */
MACH_API int mach_residual_rmsnorm_rounded_mxfp8(const void* a_bf16, const void* residual_bf16,
                                                 const void* gamma_bf16, float eps,
                                                 float weight_bias, void* norm_out_bf16,
                                                 void* residual_out_bf16, void* codes,
                                                 void* scales, int64_t m, int64_t h, void* stream);

/* Gated RMSNorm over 128-wide heads + MXFP8: the producer in front of the linear-attention
 * output projection. Replaces the producer half of mxfp6.gemm_from_gdn
 * (src/vllm_mach/mxfp6/gdn_output.py:11-13,56-64; the unfused form is RMSNormGated with
 * norm_before_gate + SiLU followed by out_proj): per (token, head), rstd = 1/sqrt(mean(x^2)+eps),
 * v = bf16(((x * rstd) * w) * silu(z)), then the activation quantiser along K = heads * 128.
 * core BF16 [M, heads, 128] contiguous; gate BF16 with `ld_gate` elements per token;
 * norm_weight [128] BF16 or FP32. Follow with mach_mx_gemm on the out_proj weight. */
MACH_API int mach_gated_rmsnorm_mxfp8_quantize(const void* core_bf16, const void* gate_bf16,
                                               int64_t ld_gate, const void* norm_weight,
                                               int weight_is_f32, float eps, void* codes,
                                               void* scales, int64_t m, int64_t heads,
                                               void* stream);

/* Checkpoint weight quantiser: BF16 [N, K] -> E4M3 codes [N, K] + LOGICAL E8M0 scales uint8
 * [N, K/32], by the rule of quantize_block (src/vllm_mach/mxfp8/reconstruct_model.py:34-50;
 * golden vector tests/test_mxfp8_reconstruct_model.py:142-156): maximum m of the block in BF16,
 * mantissa rounded up from 0.75 ((bits + 32) & 0xFF80), E8M0 = 127 + floor(log2) - 8, codes =
 * RTNE(x / 2^(E8M0 - 127)). A load-time / conversion-time step. K % 32 == 0. */
MACH_API int mach_mxfp8_quantize_weight(const void* w_bf16, void* codes, void* logical_scales,
                                        int64_t n, int64_t k, void* stream);

/* uint8 [rows, K/32] logical <-> swizzled. Pad bytes of the swizzled buffer are written as
 * 127 (scale 1.0) by pack. Replaces mxfp6.pack_scales / unpack_scales
 * (src/vllm_mach/mxfp6/dense.py:186, tests/native_mxfp6/test_mxfp8_producers.py:38-41). */
MACH_API int mach_mx_pack_scales(const void* logical, void* swizzled, int64_t rows, int64_t k,
                        void* stream);
MACH_API int mach_mx_unpack_scales(const void* swizzled, void* logical, int64_t rows, int64_t k,
                          void* stream);

/* out[M,N] (BF16) = dq(A) * dq(W)^T, FP32 accumulate. A: E4M3 codes [M,K] + swizzled scales;
 * W: codes [N, K] (E4M3) or packed 6-bit [N, 3K/4] + swizzled scales.
 * Replaces torch.ops.mxfp8_sm120.gemm / torch.ops.mxfp6.gemm_w6a8_pdl
 * (src/vllm_mach/mxfp6/dense_mxfp8.py:85-96, src/vllm_mach/mxfp6/ar_norm.py:144-147).
 * K % 32 == 0, N % 16 == 0. With w_layout = MACH_LAYOUT_GATE_UP_32 the rows of W are
 * interleaved but the output columns are still [gate | up] (N % 64 == 0, M > 64). */
MACH_API int mach_mx_gemm(const void* a_codes, const void* a_scales, const void* w, const void* w_scales,
                 void* out_bf16, int64_t m, int64_t n, int64_t k, int w_format, int w_layout,
                 void* stream);

/* Fused gate_up GEMM + SwiGLU + MXFP8 requant: W is [2I, K] = [gate rows | up rows];
 * writes codes [M, I] and swizzled scales for the down projection. Equals
 * mach_mx_gemm followed by mach_swiglu_mxfp8_quantize bit for bit (for M <= 64 when both run
 * with the same cluster split, i.e. the same FP32 summation order over K), without the BF16
 * [M, 2I] round trip. Replaces gate_up_proj + torch.ops.vllm.mach_swiglu_mxfp8_down's
 * producer half (src/vllm_mach/mxfp6/mxfp8_mlp.py:15-22,62-84).
 * MACH_LAYOUT_ROWS: I % 128 == 0. MACH_LAYOUT_GATE_UP_32: I % 32 == 0. */
MACH_API int mach_mx_gemm_swiglu(const void* a_codes, const void* a_scales, const void* w,
                        const void* w_scales, void* out_codes, void* out_scales, int64_t m,
                        int64_t i, int64_t k, int w_format, int w_layout, void* stream);

/* Row permutation [gate rows | up rows] -> MACH_LAYOUT_GATE_UP_32 of a [2I, row_bytes] byte
 * matrix (weight codes, or logical uint8 scales before packing). Out of place; a load-time
 * transform like the repacking of src/vllm_mach/mxfp6/dense.py:185-188. I % 32 == 0. */
MACH_API int mach_mx_interleave_gate_up(const void* src, void* dst, int64_t two_i,
                                        int64_t row_bytes, void* stream);

/* Block-FP8 activation quantiser: BF16 [M,K] -> E4M3 [M,K] + FP32 scales, one per 1x128,
 * stored column-major (element (row, g) at g*M + row). scale = max(amax,1e-10)/448,
 * q = clamp(x/scale, +-448). Replaces _quant (src/vllm_mach/fp8/_quantize_kernel.py:7-18). */
MACH_API int mach_fp8_group_quantize(const void* x_bf16, void* q, void* scales_f32, int64_t m, int64_t k,
                            void* stream);

/* SiLU(gate)*up in FP32 + 1x128 FP8 quantisation, scale = max(amax/448, 1/(448*512)).
 * input BF16 [M, 2I]; out E4M3 [M, I]; scales FP32 [M, I/128] row-major or column-major
 * (transposed != 0). Replaces torch.ops.mach_fp8_activation.run
 * (native/fp8_activation/activation.cu:18-60). */
MACH_API int mach_silu_mul_fp8_group_quantize(const void* input_bf16, void* out, void* scales_f32,
                                     int64_t m, int64_t i, int transposed, void* stream);

/* y[m,n] = bf16( sum_g fma(dot_f32(A[m,g*128:], B[n,g*128:]), sa[m,g]*sb[n/128,g], acc) ),
 * g ascending. A E4M3 [M,K]; B E4M3 [N,K]; sa FP32 column-major (g*M + m); sb FP32
 * [ceil(N/128), K/128] row-major. Replaces torch.ops.vllm_mach_block_fp8.mm and
 * ordered.gemm (native/block_fp8/block_fp8.cu:233-255, src/vllm_mach/fp8/ordered.py:38-64).
 * K % 128 == 0, N % 16 == 0. */
MACH_API int mach_block_fp8_gemm(const void* a, const void* b, const void* sa, const void* sb,
                        void* out_bf16, int64_t m, int64_t n, int64_t k, void* stream);

/* The same product evaluated exactly as the reference's small-batch route does
 * (ordered.gemm, src/vllm_mach/fp8/ordered.py:38-64): every 128-K group's FP32 dot is written
 * unscaled to `raw_scratch` (FP32 [K/128, M, N], caller-owned, contents undefined afterwards),
 * then ONE fma chain per output runs over the groups in ascending order. M <= 64. */
MACH_API int mach_block_fp8_gemm_ordered(const void* a, const void* b, const void* sa,
                                         const void* sb, void* out_bf16, void* raw_scratch,
                                         int64_t m, int64_t n, int64_t k, void* stream);

/* mach_block_fp8_gemm_ordered without a caller-supplied scratch: the per-group dots go to an
 * 8 MiB array that is part of the library image, so this call never allocates (no cudaMalloc,
 * no cudaFree, no framework allocator). It has no counterpart in the reference. It is meant
 * for callers that have no way to obtain device memory at call time: a serving worker whose
 * free HBM was handed to the KV cache at start-up, so a late cudaMalloc can fail, or a host
 * binding that cannot reach the framework's caching allocator to get a [K/128, M, N] buffer.
 *  - Limit: (K/128) * M * N * 4 bytes <= 8 MiB (and M <= 64); larger problems are refused with
 *    MACH_ERR_UNSUPPORTED and must use mach_block_fp8_gemm_ordered.
 *  - The 8 MiB are resident on every GPU that loads the library until the process exits.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current); make that first call before any
 *    stream capture begins.
 *  - All calls on a device share the one array and it keeps the previous call's contents;
 *    every element a call reads is written by that same call first, so nothing needs
 *    clearing, but two calls that overlap on the GPU (different streams) race on it. */
MACH_API int mach_block_fp8_gemm_ordered_static(const void* a, const void* b, const void* sa,
                                                const void* sb, void* out_bf16, int64_t m,
                                                int64_t n, int64_t k, void* stream);

/* ---- Row-parallel all-reduce fused with residual add + RMSNorm (+ MXFP8) over NVLink.
 * Replaces torch.ops.mach_norm_quant.run and the FlashInfer workspace it uses
 * (native/ar_norm/binding.cu:11-70, src/vllm_mach/mxfp6/ar_norm.py:113-141,
 * src/vllm_mach/mxfp6/compiled_ar_norm.py:7-84). One process per GPU. Every rank allocates one
 * communication buffer, exports it, opens every peer's, and creates a workspace from the
 * `world` base pointers (buffers[rank] = its own). These calls allocate / map memory and
 * synchronise; the reduce call itself does neither.
 *   a = bf16(sum over ranks in rank order, FP32); res = bf16(a + residual);
 *   norm = bf16(res * rsqrt(mean(res^2) + eps) * (weight_bias + gamma)); codes/scales = MXFP8(norm).
 * All ranks must call with the same (m, h, algo) in the same order. algo: 0 = choose,
 * 1 = one-shot, 2 = two-shot with one flag per (rank, CTA), 3 = two-shot with one flag per
 * (rank, phase) published by the grid's last CTA (what 0 chooses above 256 KiB with more than
 * two ranks; launched cooperatively, so a grid that cannot be co-resident is held back or
 * refused by the driver instead of spinning).
 * partial_bf16 may be NULL after mach_mx_gemm_reduce_scatter of the same [m, h] on this
 * workspace (anything else is refused with MACH_ERR_INVALID). norm_out, residual_out,
 * codes+scales may be NULL.
 * residual_out may alias residual. hidden % 32 == 0, hidden <= 8192, world <= 8.
 *
 * Failure behaviour: every device-side wait for a peer is bounded (mach_ar_set_wait_limit_us,
 * about one second by default). A wait that gives up records 401 (scatter flag) or 402 (gather
 * flag) in the device status word (mach_device_status), marks the workspace as failed and
 * writes NaN (BF16) / 0x7F (E4M3) / 0xFF (E8M0) into the outputs of the affected rows; every
 * later call on a failed workspace returns poisoned outputs at once (status 403) until all
 * ranks have called mach_ar_reset. Poll mach_device_status at a host synchronisation point
 * (end of a step) to learn of it. */
MACH_API size_t mach_ar_buffer_bytes(int world, int64_t tokens_cap, int64_t hidden);
MACH_API int mach_ar_buffer_alloc(size_t bytes, void** dev_ptr); /* zero-filled */
MACH_API int mach_ar_buffer_free(void* dev_ptr);
MACH_API int mach_ar_ipc_export(void* dev_ptr, void* handle_64_bytes);
MACH_API int mach_ar_ipc_open(const void* handle_64_bytes, void** peer_ptr);
MACH_API int mach_ar_ipc_close(void* peer_ptr);
MACH_API int mach_ar_create(int world, int rank, int64_t tokens_cap, int64_t hidden,
                            void* const* buffers, void** workspace);
MACH_API int mach_ar_destroy(void* workspace);
/* Upper bound of every device-side wait of calls on this workspace (host state, takes effect
 * with the next call). */
MACH_API int mach_ar_set_wait_limit_us(void* workspace, int64_t microseconds);
/* Clears this rank's epoch, flags and failed mark (synchronises `stream`). Collective by
 * contract: every rank calls it with no reduce in flight, with a host barrier before and after
 * (the reference re-creates its FlashInfer workspace instead, src/vllm_mach/mxfp6/ar_norm.py:113-128). */
MACH_API int mach_ar_reset(void* workspace, void* stream);
MACH_API int mach_allreduce_residual_rmsnorm_mxfp8(void* workspace, const void* partial_bf16,
                                                   const void* residual_bf16,
                                                   const void* gamma_bf16, float eps,
                                                   float weight_bias, void* norm_out_bf16,
                                                   void* residual_out_bf16, void* codes,
                                                   void* scales, int64_t m, int64_t h, int algo,
                                                   void* stream);

/* Owner form of the same reduce (row ownership between norms; replaces reduce_owner +
 * gather_mx8 of native/owner_prefill/owner.cu:64-160 for any world <= 8 and any M): rank r owns
 * rows [first, first + count) given by mach_ar_owner_rows (contiguous blocks of ceil(M / world)).
 * Every owner pulls its rows of all ranks' partial sums over NVLink, reduces them in rank
 * order, adds ITS rows of the residual, normalises and quantises them, and stores each row's
 * codes and scales into every rank's communication buffer as it produces them (the stores run
 * beside the pulls; one flag exchange closes the step). Outputs: codes E4M3 [M, H] + swizzled E8M0 scales for ALL
 * rows on every rank (what the next block-scaled GEMM consumes); residual_out_rows and
 * norm_out_rows (may be NULL) BF16 [count, H] for the OWNED rows only; residual_rows is BF16
 * [count, H], the owned rows of the residual stream. Same arithmetic and rounding points as
 * mach_allreduce_residual_rmsnorm_mxfp8, hence the same bytes.
 * partial_bf16 == NULL: the producing GEMM wrote its BF16 [M, H] output (leading dimension H)
 * to the address mach_ar_partial_ptr returns (inside this rank's communication buffer, fixed
 * for the life of the workspace), which saves one local copy.
 * codes / scales == the addresses mach_ar_codes_ptr returns (the all-rows code matrix and the
 * swizzled scale buffer inside this rank's communication buffer, fixed for the life of the
 * workspace): nothing is copied out, the next GEMM reads them where they are. They stay valid
 * until the next reduce on the same workspace is launched; any other pair of pointers receives
 * a copy. Launched cooperatively. */
MACH_API int mach_ar_owner_rows(int world, int rank, int64_t m, int64_t* first, int64_t* count);
MACH_API int mach_ar_partial_ptr(void* workspace, void** partial_bf16);
MACH_API int mach_ar_codes_ptr(void* workspace, void** codes, void** scales);
MACH_API int mach_allreduce_owner_rmsnorm_mxfp8(void* workspace, const void* partial_bf16,
                                                const void* residual_rows_bf16,
                                                const void* gamma_bf16, float eps,
                                                float weight_bias, void* norm_out_rows_bf16,
                                                void* residual_out_rows_bf16, void* codes,
                                                void* scales, int64_t m, int64_t h, void* stream);

/* All `world` ranks of a group whose communication buffers live on ONE device, run as a
 * single cooperative grid (kernels that wait on one another must not be separate launches on
 * one GPU). workspaces[r] must be rank r of `world`; the per-rank arrays hold what rank r
 * would pass to mach_allreduce_residual_rmsnorm_mxfp8 (owner_form == 0, `algo` as there) or to
 * mach_allreduce_owner_rmsnorm_mxfp8 (owner_form != 0). For validating the multi-rank
 * protocols on a machine with fewer GPUs than ranks; no counterpart in the reference. */
MACH_API int mach_allreduce_local_ranks(int world, void* const* workspaces,
                                        const void* const* partials,
                                        const void* const* residuals, const void* gamma_bf16,
                                        float eps, float weight_bias, void* const* norm_outs,
                                        void* const* residual_outs, void* const* codes,
                                        void* const* scales, int64_t m, int64_t h, int algo,
                                        int owner_form, void* stream);

/* Row-parallel GEMM whose epilogue is the reduce-scatter: the BF16 partial sums [M, N] never go
 * to a local matrix, every row is stored (NVLink peer store) into the all-reduce buffer of the
 * rank that owns it. Follow it on the same stream with
 * mach_allreduce_residual_rmsnorm_mxfp8(workspace, partial = NULL, ...), which then only
 * reduces, normalises and gathers. Fuses the down projection with the first half of the
 * deferred reduce of the reference (runtime.patch:398-433; the reference runs the GEMM and the
 * collective as separate launches). N must equal the workspace's hidden size; shapes that do
 * not take the CTA-pair kernel (M <= 192 for narrow N) return MACH_ERR_UNSUPPORTED and the
 * caller uses mach_mx_gemm + the all-reduce with a partial tensor. Every rank must make the
 * same choice. */
MACH_API int mach_mx_gemm_reduce_scatter(void* ar_workspace, const void* a_codes,
                                         const void* a_scales, const void* w,
                                         const void* w_scales, int64_t m, int64_t n, int64_t k,
                                         int w_format, void* stream);

/* ---- Mixture-of-experts layer (replaces the stages of Mxfp6Sm120Experts.apply and the shims
 * of src/vllm_mach/mxfp6/moe_utils.py:47-488: quantize_mxfp8 + route, grouped_gemm,
 * silu_grouped_gemm, reduce). All device-side, stream-ordered, no host read-back.
 *
 * mach_moe_router_topk: logits BF16 [M, E] -> softmax (FP32) -> top-k (ties: lowest index) ->
 *   renormalised weights FP32 [M, topk] + ids int32 [M, topk]. E <= 1024, topk <= 32.
 * mach_moe_route: expert-major permutation. expert_map (int32 [global experts] -> local id or
 *   -1, may be NULL) selects this rank's experts. Every non-empty expert gets a segment padded
 *   to 128 rows. Outputs: counts int32 [E], offsets int32 [E+1], pos_of int32 [M*topk]
 *   (permuted row of each pair, -1 if not local), src_of int32 [rows_cap] (token of each
 *   permuted row, -1 for padding), work int32 [3*work_cap] = (expert, first row, rows <=
 *   chunk_rows) and num_work int32 [1]. Capacities from mach_moe_rows_cap / mach_moe_work_cap.
 *   chunk_rows in {16 (only when M <= 16), 64, 128, 256}.
 * mach_moe_gather_quantize: BF16 hidden [M, K] -> MXFP8 codes [rows_cap, K] + swizzled scales
 *   in permuted order.
 * mach_moe_grouped_gemm: per work item and 128-row weight tile, out rows [first, first+rows) =
 *   A . W_expert^T. W is the experts stacked, [E * w_rows, K] (w_rows % 128 == 0) with scales
 *   packed over the stacked matrix. swiglu != 0: W rows are gate/up interleaved by 32 per
 *   expert; writes E4M3 codes [rows_cap, w_rows/2] + swizzled scales; else BF16 [rows_cap, w_rows].
 * mach_moe_combine: out[m] = bf16(sum_k w[m,k] * y[pos_of[m,k]]), k ascending, FP32. */
MACH_API int mach_moe_router_topk(const void* logits_bf16, void* topk_weights_f32,
                                  void* topk_ids_i32, int64_t m, int64_t experts, int64_t topk,
                                  void* stream);
MACH_API int64_t mach_moe_rows_cap(int64_t tokens, int64_t topk, int64_t experts);
MACH_API int64_t mach_moe_work_cap(int64_t tokens, int64_t topk, int64_t experts,
                                   int64_t chunk_rows);
MACH_API int mach_moe_route(const void* topk_ids_i32, const void* expert_map_i32, int64_t m,
                            int64_t topk, int64_t experts, int64_t chunk_rows, int64_t rows_cap,
                            int64_t work_cap, void* counts, void* offsets, void* pos_of,
                            void* src_of, void* work, void* num_work, void* stream);
MACH_API int mach_moe_gather_quantize(const void* hidden_bf16, const void* src_of,
                                      const void* offsets, int64_t experts, int64_t rows_cap,
                                      int64_t k, void* codes, void* scales, void* stream);
/* Token-major form of the same step (same bytes out): each token is quantised once and stored
 * to its top-k permuted rows pos_of[token, j] (< 0: skipped). */
MACH_API int mach_moe_scatter_quantize(const void* hidden_bf16, const void* pos_of, int64_t m,
                                       int64_t topk, int64_t k, void* codes, void* scales,
                                       void* stream);
MACH_API int mach_moe_grouped_gemm(const void* a_codes, const void* a_scales, const void* w,
                                   const void* w_scales, void* out, void* out_scales,
                                   const void* work, const void* num_work, int64_t work_cap,
                                   int64_t rows_cap, int64_t experts, int64_t w_rows, int64_t k,
                                   int64_t chunk_rows, int w_format, int swiglu, void* stream);
MACH_API int mach_moe_combine(const void* y_bf16, const void* topk_weights_f32,
                              const void* pos_of, void* out_bf16, int64_t m, int64_t h,
                              int64_t topk, void* stream);

/* Small-batch schedule of the whole layer (M <= 8 tokens, topk <= 16): three launches (quantise
 * + expert map, W1 + SwiGLU + requant, W2 + weighted reduce) on the CUDA cores instead of the
 * permutation and the grouped tensor-core GEMMs; same rounding points, the dot products summed
 * in a different order. Replaces the reference's decode schedules (src/vllm_mach/mxfp6/moe.py:
 * 74-88,126-188). Weights in the kernel layout of mach_moe_grouped_gemm (W1 stacked with
 * gate/up rows interleaved by 32, swizzled scales packed over the stack). `scratch`:
 * mach_moe_small_scratch_bytes bytes, caller-owned, contents undefined afterwards. */
MACH_API size_t mach_moe_small_scratch_bytes(int64_t tokens, int64_t topk, int64_t hidden,
                                             int64_t inter);
MACH_API int mach_moe_small_batch(const void* hidden_bf16, const void* topk_weights_f32,
                                  const void* topk_ids_i32, const void* expert_map_i32,
                                  const void* w13, const void* s13, const void* w2, const void* s2,
                                  void* scratch, void* out_bf16, int64_t m, int64_t topk,
                                  int64_t experts, int64_t hidden, int64_t inter, int w_format,
                                  void* stream);

/* Staged form of the layer, for callers that drive the stages themselves the way the
 * reference's shims do (mxfp6_sm120_route / _grouped_gemm / _silu_grouped_gemm / _reduce,
 * src/vllm_mach/mxfp6/moe_utils.py:205-488). The activation arrives already quantised:
 * mach_moe_scatter_codes copies codes [M, K] + logical scales [M, K/32] of every token into
 * its top-k permuted rows pos_of[token, j] (swizzled scales out). mach_moe_stage_offsets turns
 * the route outputs into the shims' int64 pair: expert_offsets[E + 1] = routed rows before
 * each expert (true counts), scale_offsets[E + 1] = first row of each expert's 128-row padded
 * segment; unlike the reference, whose permuted ACTIVATION rows are unpadded, here activation
 * and scale rows share the padded index space, so the permuted buffers need
 * mach_moe_rows_cap rows. mach_moe_work_from_offsets rebuilds the grouped GEMM's work list
 * from that pair on the device. */
MACH_API int mach_moe_scatter_codes(const void* codes_in, const void* logical_scales,
                                    const void* pos_of, int64_t m, int64_t topk, int64_t k,
                                    void* codes, void* scales, void* stream);
MACH_API int mach_moe_stage_offsets(const void* counts, const void* offsets, int64_t experts,
                                    void* expert_offsets_i64, void* scale_offsets_i64,
                                    void* stream);
MACH_API int mach_moe_work_from_offsets(const void* expert_offsets_i64,
                                        const void* scale_offsets_i64, int64_t experts,
                                        int64_t chunk_rows, int64_t work_cap, void* work,
                                        void* num_work, void* stream);

/* Tuning / experiment knobs (process-global, not thread-safe; 0 restores the heuristic):
 * "split" (cluster size along K of the feature-major GEMM: 1..8), "split_fill_pct" (grow the
 * cluster until CTAs reach this percentage of the SM count), "stages" (pipeline
 * depth), "bn" (token-major N tile: 128, 256), "swap_max_m" (largest batch handled
 * feature-major at all), "wide_max_m" / "narrow_max_m" (largest batch a wide / a narrow weight
 * matrix runs feature-major; heuristic 32-64 / 256), "mid" (0: batches up to 128 tokens skip
 * the one-token-tile kernel), "smem_cap_kb" (cap on dynamic shared memory per CTA), "tm_min_m"
 * (smallest batch for the persistent 256-token kernels), "tm_bn" (their tile width), "pair"
 * (0: single-CTA persistent kernel instead of the cta_group::2 kernel), "panel_m"
 * (raster panel height). A library built with -DMACH_EXPERIMENTS (kernel sweeps only) also
 * takes experiment bits that switch parts of the MMA loops off; the default build has none.
 * No counterpart in the reference (its tile table is torch.ops.mxfp6.set_w6a8_config,
 * src/vllm_mach/mxfp6/moe_projection.py:35-105, an SM120 table). */
MACH_API int mach_tune_set(const char* name, int value);
/* Diagnostics: "last_pairs" = CTA pairs launched by the most recent cta_group::2 GEMM
 * (bounded by cudaOccupancyMaxActiveClusters); -1 for unknown names. */
MACH_API int mach_tune_get(const char* name);

#ifdef __cplusplus
}
#endif
#endif /* MACH_B200_H_ */
