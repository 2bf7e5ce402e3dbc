/*
 * libi8linear — C ABI of the B200 (sm_100a) INT8 quantized-linear kernels.
 *
 * Every entry point
 *   - takes plain device pointers, sizes and a CUDA stream handle (cudaStream_t passed as void*),
 *   - allocates nothing, never synchronises the device, launches on the given stream,
 *   - returns 0 on success or a negative I8L_ERR_* code; i8l_last_error() gives the text for the
 *     calling thread's most recent failure.
 * The library contains no CPU fallback: on a device that is not compute capability 10.x every
 * launch entry point returns I8L_ERR_ARCH.
 *
 * "Reference" below is the jiaoch/Triton-INT8 project; file:line cites name the Python/Triton code a
 * function replaces.  Tensors are row-major and contiguous; a leading batch dimension is folded into
 * the rows.  All of rows/cols/M/N/K must be multiples of 128 (the reference has no masking either).
 */
#ifndef I8LINEAR_H_
#define I8LINEAR_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported-symbol marker (the library is built with hidden default visibility). */
#define I8L_API __attribute__((visibility("default")))

#define I8L_OK 0
#define I8L_ERR_SHAPE (-1)   /* a dimension is zero, negative, too large or not a multiple of 128 */
#define I8L_ERR_ALIGN (-2)   /* a pointer is not 16-byte aligned */
#define I8L_ERR_ARCH (-3)    /* current device is not sm_100 */
#define I8L_ERR_CUDA (-4)    /* a CUDA runtime/driver call failed */
#define I8L_ERR_TIMEOUT (-5) /* a bounded device-side wait gave up (see i8l_gemm status word) */
#define I8L_ERR_ARG (-6)     /* unsupported combination of options / null pointer */

/* Quantisation group of one scale. */
#define I8L_GRAN_TILE128 0  /* one scale per 128x128 tile            (reference block_channel A/dY) */
#define I8L_GRAN_GROUP128 1 /* one scale per (row, 128 contraction elements)                        */
#define I8L_GRAN_ROW 2      /* one scale per row over the whole contraction axis (per token/channel)*/
#define I8L_GRAN_TILE128X256 5 /* one scale per 128 rows x 256 contraction elements (the activation
                                  grouping of the reference's TileLang forward, tilelang/block_channel_fwd.py:185-188) */

/* Arithmetic of scale and rounding.  x is bf16 widened to fp32, amax the group's max |x|. */
#define I8L_QMODE_TRITON 0 /* amax=max(amax,1e-4); s=127/amax (IEEE); q=clamp(floor(x*s+.5),-128,127); stores 1/s.
                              triton/block_channel_fwd32.py:101-129,160-192 */
#define I8L_QMODE_RNE 1    /* s=rcp(max(amax,1e-4))*127; q=clamp(rint(x*s),-127,127); stores rcp(s).
                              tilelang/block_channel_bwd.py:96-104, tilelang/block_channel_fwd.py:206-230 */
#define I8L_QMODE_FUSED 2  /* s=127/(amax+1e-5); q=floor(x*s+.5); stores s (the GEMM divides).
                              triton/fused_triton_fwd32.py:49-59, triton/fused_triton_bwd33.py:50-56 */
#define I8L_QMODE_ROWRCP 3 /* s=rcp(max(amax,1e-4))*127; q=clamp(floor(x*s+.5),-128,127); stores amax/127.
                              triton/double-channle_fwd32.py:157-160,132-135 */

#define I8L_QMODE_TRITON_BF16S 4 /* as TRITON, the stored 1/s rounded to bf16 (kept in an fp32 array): the
                                    TileLang forward's quantizers write their scales to bf16 tensors and
                                    widen them afterwards.  tilelang/block_channel_fwd.py:133,149,191,204 */

/* Walsh-Hadamard rotation applied (in fp32, result rounded to bf16) before quantisation,
 * always along the contraction axis of the operand. */
#define I8L_HAD_NONE 0
#define I8L_HAD_128 128   /* independent 128-point transforms */
#define I8L_HAD_FULL (-1) /* one transform over the whole (power-of-two) contraction axis; ROW only */

/*
 * Quantise x (bf16 [batch, rows, cols]) in 128x128 tiles read once from HBM.
 *
 * Two operands can be produced from the same read:
 *   q  / scale   : the operand x itself, contraction axis = cols.  q is int8 [batch, rows, cols].
 *                  scale: TILE128 -> fp32 [batch, rows/128, cols/128]; GROUP128 -> [batch, rows, cols/128].
 *   qt / scale_t : the operand x^T (per batch), contraction axis = rows.  qt is int8 [batch, cols, rows].
 *                  scale_t: TILE128 -> [batch, cols/128, rows/128]; GROUP128 -> [batch, cols, rows/128].
 * I8L_GRAN_TILE128X256 (scale fp32 [batch, rows/128, cols/256], cols a multiple of 256) produces q only,
 * without rotation.
 * Either pair may be NULL (not produced).  hadamard is I8L_HAD_NONE or I8L_HAD_128; the rotation
 * always runs along the contraction axis of the operand it belongs to (cols for q, rows for qt), so
 * with a rotation the two operands come from two passes over x instead of one.
 * Replaces triton_per_block_quant (triton/block_channel_fwd32.py:194-212,
 * triton/block_channel_bwd33.py:122-138) and, through qt, the transposed copies a linear layer's
 * dW = dY^T X needs.
 */
I8L_API int i8l_quant_tile(const void* x, int64_t batch, int64_t rows, int64_t cols, int gran, int qmode,
                   int hadamard, int8_t* q, float* scale, int8_t* qt, float* scale_t, void* stream);

/*
 * Quantise each row of x (bf16 [rows, cols]) with one scale over the whole row.
 * q int8 [rows, cols], scale fp32 [rows].  hadamard: NONE, 128 or FULL (cols a power of two,
 * cols <= 32768).  Replaces triton_per_token_quant (triton/block_channel_fwd32.py:132-157) and
 * triton_per_row_quant_2d/3d incl. the torch glue between their two passes
 * (triton/double-channle_fwd32.py:140-175,229-266, triton/double_channel_bwd33.py:142-176).
 */
I8L_API int i8l_quant_row(const void* x, int64_t rows, int64_t cols, int qmode, int hadamard, int8_t* q,
                  float* scale, void* stream);

/*
 * Quantise the transpose of x (bf16 [rows, cols]) with one scale per column of x: the operand is
 * x^T [cols, rows], contraction axis = rows.  qt int8 [cols, rows], scale_t fp32 [cols].
 * colmax_scratch: fp32 [cols] device scratch, overwritten.  hadamard: NONE only.
 * No counterpart function in the reference: it is triton_per_token_quant applied to W^T, which a
 * linear layer's dX = dY W needs (the reference would transpose on the host first).
 */
I8L_API int i8l_quant_col_t(const void* x, int64_t rows, int64_t cols, int qmode, int8_t* qt, float* scale_t,
                    float* colmax_scratch, void* stream);

/*
 * As i8l_quant_col_t, with a 128-point Walsh-Hadamard rotation along the rows of x (the contraction
 * axis of the transposed operand) in front: W^T of a rotated linear layer's dX GEMM.  Two passes over
 * x (column absmax of the rotated values, then quantise); qmode TRITON, RNE or ROWRCP (the last one
 * gives the transposed double_channel operands of a backward pass).
 * No counterpart in the reference.
 */
I8L_API int i8l_quant_col_t_rot(const void* x, int64_t rows, int64_t cols, int qmode, int8_t* qt,
                                float* scale_t, float* colmax_scratch, void* stream);

/*
 * Same result as i8l_quant_col_t, for callers that cannot hand over scratch memory: code running
 * where device allocation is off limits (inside a framework's memory-pool callback or a stream
 * capture section, in a plugin sandbox that forbids cudaMalloc, or late in a job when the pool is
 * exhausted) still has to quantise W^T for the dX GEMM.  The column-absmax scratch is a fixed
 * array of I8L_STATIC_SCRATCH_MAX_COLS floats (256 KiB) built into the library image; every GPU
 * that loads the library holds it until the process exits.  No counterpart in the reference.
 *   - cols > I8L_STATIC_SCRATCH_MAX_COLS is rejected with I8L_ERR_SHAPE.
 *   - The first call on each device resolves the array's device address (a synchronous runtime
 *     query made with that device current); make that first call before any stream capture.
 *   - Nothing is allocated or freed, by this function or by anything it calls.
 *   - All calls on a device share the one array; it is re-zeroed on the given stream at the start
 *     of every call, so back-to-back calls on one stream are safe, but two calls whose kernels
 *     may overlap on the GPU (different streams) race on it and give wrong scales.
 */
#define I8L_STATIC_SCRATCH_MAX_COLS 65536
I8L_API int i8l_quant_col_t_static(const void* x, int64_t rows, int64_t cols, int qmode, int8_t* qt,
                                   float* scale_t, void* stream);

/* Scale layouts understood by the GEMM. */
#define I8L_ASCALE_TILE 0  /* a_scale fp32 [batch, M/128, K/128] */
#define I8L_ASCALE_GROUP 1 /* a_scale fp32 [batch, M, K/128]     */
#define I8L_ASCALE_TILE256 2 /* a_scale fp32 [batch, M/128, K/256]: one scale serves two consecutive K blocks
                                (tilelang/block_channel_fwd.py:33,76); K a multiple of 256 */
#define I8L_BSCALE_CHANNEL 0 /* b_scale fp32 [N]  (shared B) or [batch, N]      : K-invariant        */
#define I8L_BSCALE_TILE 1    /* b_scale fp32 [N/128, K/128] or [batch, N/128, K/128]                  */
#define I8L_BSCALE_GROUP 2   /* b_scale fp32 [N, K/128]     or [batch, N, K/128]                      */

#define I8L_GEMM_EXACT_ORDER 1 /* per K step evaluate (float(P)*a_s)*b_s then add, unfused: bit-equal to the
                                  reference's fp32 result.  Without it the K-invariant factor is applied once
                                  at the end, multiply-adds are fused and, for per-tile A scales with per-tile or
                                  per-channel B scales, the int32 partials enter the fp32 sum through a bounded
                                  bias that is removed at the end of the tile (same int32 partials; fp32 result
                                  within 1e-4 relative of the exact sum at K = 32768, typically 1e-6; scale
                                  products times 1.3e7 must stay finite in fp32). */
#define I8L_GEMM_DIVIDE 2      /* scales are multipliers s: acc += float(P) / (a_s*b_s)  (fused variants); together with
                                  EXACT_ORDER a true division per element, otherwise a multiplication by the rounded
                                  reciprocal of a_s*b_s (differs from the division by at most 1 ulp per K block) */
#define I8L_GEMM_OUT_F32 4     /* C is fp32 instead of bf16 */
#define I8L_GEMM_PRODUCT_FIRST 8 /* with EXACT_ORDER: evaluate float(P) * (a_s*b_s) instead of (float(P)*a_s)*b_s per K
                                    step, the order of the reference's TileLang kernels
                                    (tilelang/block_channel_fwd.py:75-81, tilelang/block_channel_bwd.py:76-81) */

/*
 * Block-scaled INT8 GEMM: for every 128-wide K block kb, P = A_q[:,kb] . B_q[:,kb]^T exactly in int32
 * (tcgen05.mma kind::i8, TMEM accumulator), then acc_f32 += float(P) * a_scale * b_scale;
 * C = bf16(acc * post_scale + bias).
 *   a_q int8 [batch, M, K]; b_q int8 [N, K] (b_batched=0) or [batch, N, K] (b_batched=1);
 *   bias bf16 [N] or NULL; C bf16 (or fp32) [batch, M, N];
 *   status: device int32 word (zeroed by the caller) that receives a non-zero code if a bounded
 *   wait inside the kernel gave up; may be NULL.
 * Replaces triton_gemm / int8_gemm_kernel of triton/block_channel_fwd32.py:12-96 (TILE, CHANNEL),
 * triton/block_channel_bwd33.py:8-84 (TILE, TILE, b_batched) and, with I8L_GEMM_DIVIDE and
 * I8L_BSCALE_GROUP / TILE, the arithmetic of triton/fused_triton_fwd32.py:42-65 and
 * triton/fused_triton_bwd33.py:43-58.
 */
I8L_API int i8l_gemm_block(const int8_t* a_q, const int8_t* b_q, const float* a_scale, const float* b_scale,
                   int a_scale_kind, int b_scale_kind, int b_batched, const void* bias,
                   float post_scale, void* c, int64_t batch, int64_t M, int64_t N, int64_t K,
                   int flags, int32_t* status, void* stream);

/*
 * The fused variant as ONE kernel, bf16 in and bf16 (or fp32) out: per 128 x 128 output tile and 128-wide K
 * step the A tile and the B tile are read as bf16, scaled by 127 / (amax + 1e-5) (A: per 128 x 128 tile;
 * B: per row and K step when b_batched == 0, per 128 x 128 tile when b_batched == 1), rounded with
 * floor(x*s + 0.5) into the tensor core's shared-memory stage, multiplied exactly in int32
 * (tcgen05.mma kind::i8) and accumulated as acc += float(P) / (s_a * s_b); no int8 tensor or scale is written
 * to global memory.  Same integers, scales and results as i8l_quant_tile(I8L_QMODE_FUSED) on each operand
 * followed by i8l_gemm_block(I8L_GEMM_DIVIDE); the quantization work is repeated for every output tile that
 * consumes an operand tile, as in the reference.
 *   a bf16 [batch, M, K]; b bf16 [N, K] (b_batched = 0) or [batch, N, K] (b_batched = 1); c [batch, M, N].
 *   flags: I8L_GEMM_EXACT_ORDER (a true division per element and unfused adds: the reference's fp32 result
 *   bit for bit; otherwise a multiplication by the rounded reciprocal of s_a*s_b), I8L_GEMM_OUT_F32.
 * Replaces fused_int8_gemm_kernel and its launcher: triton/fused_triton_fwd32.py:23-96,
 * triton/fused_triton_bwd33.py:24-86.
 */
I8L_API int i8l_fused_gemm(const void* a_bf, const void* b_bf, void* c, int64_t batch, int64_t M, int64_t N,
                           int64_t K, int b_batched, int flags, int32_t* status, void* stream);

/*
 * Row x column scaled INT8 GEMM: int32 accumulation over the whole K in TMEM, then
 * C = bf16( bf16((float(acc) * a_scale[m]) * b_scale[n]) * post_scale + bias ).
 * The intermediate bf16 rounding reproduces the reference, which stores the GEMM result as bf16
 * and multiplies by 1/K afterwards (triton/double-channle_fwd32.py:58-59,284); with
 * post_scale == 1 and no bias it is the identity.
 *   a_scale fp32 [batch, M]; b_scale fp32 [N] or [batch, N].
 * Replaces triton/double-channle_fwd32.py:11-90 and triton/double_channel_bwd33.py:11-87.
 */
I8L_API int i8l_gemm_rowcol(const int8_t* a_q, const int8_t* b_q, const float* a_scale, const float* b_scale,
                    int b_batched, const void* bias, float post_scale, void* c, int64_t batch,
                    int64_t M, int64_t N, int64_t K, int flags, int32_t* status, void* stream);

/*
 * Raw int32 accumulators, for parity checks.  per_block=0: out int32 [batch, M, N] = sum over all K.
 * per_block=1: out int32 [batch, K/128, M, N], one partial product per 128-wide K block.
 * No counterpart in the reference (its kernels never expose the integer partials).
 */
I8L_API int i8l_gemm_dump_i32(const int8_t* a_q, const int8_t* b_q, int b_batched, int32_t* out,
                      int64_t batch, int64_t M, int64_t N, int64_t K, int per_block,
                      int32_t* status, void* stream);

/*
 * Column-parallel dX (one process per GPU, W split along N): the block-scaled GEMM of
 * i8l_gemm_block (per-tile a scales, per-channel or per-tile b scales, bf16 output, batch 1) whose
 * epilogue scatters the partial product for a reduce-scatter along M.  Row block o (rows
 * [o*M/world, (o+1)*M/world)) is written to c_slots[o] + rank*(M/world)*N, i.e. into slot `rank` of a
 * bf16 [world, M/world, N] buffer that lives in rank o's memory.  c_slots is a HOST array of `world`
 * device pointers: c_slots[rank] is local, the others are peer mappings of the other ranks' buffers
 * (CUDA IPC or symmetric memory; plain stores over NVLink, no multicast).  The caller orders the
 * ranks around the call (all ranks' previous readers done before, all writers done after) and then
 * sums its own buffer with i8l_sum_slots.  M must be a multiple of 128*world, world <= I8L_MAX_RANKS.
 * No counterpart in the reference (it has no multi-GPU code).
 */
#define I8L_MAX_RANKS 8
I8L_API int i8l_gemm_block_scatter(const int8_t* a_q, const int8_t* b_q, const float* a_scale, const float* b_scale,
                           int b_scale_kind, float post_scale, void* const* c_slots, int world, int rank,
                           int64_t M, int64_t N, int64_t K, int32_t* status, void* stream);

/*
 * out bf16 [rows, cols] = sum over w of slots bf16 [world, rows, cols], added in slot order in fp32 and
 * rounded once (deterministic).  cols a multiple of 8.  No counterpart in the reference.
 */
I8L_API int i8l_sum_slots(const void* slots, void* out, int world, int64_t rows, int64_t cols, void* stream);

/*
 * The GEMMs are persistent kernels with one CTA per SM (about 210 KB of shared memory each), so a kernel
 * launched beside one on another stream finds no free SM until the GEMM ends.  This sets, for the calling
 * host thread, the number of CTAs the following GEMM launches may use (0 = all SMs, the default): a
 * column-parallel backward pass gives the dW GEMM a few SMs fewer while the reduce-scatter of dX is in
 * flight, so that the collective overlaps the GEMM instead of queueing behind it.  No counterpart in the
 * reference (it has no multi-GPU code).
 */
I8L_API int i8l_set_cta_limit(int max_ctas);

/*
 * Test hook for the bounded waits of the GEMM kernels (not for production use; process-wide until reset).
 * Every wait on an mbarrier inside the GEMMs gives up after a number of polls (about two seconds' worth)
 * and the kernel then returns with I8L_ERR_TIMEOUT in the caller's status word instead of hanging.
 * max_polls > 0 lowers that limit for all following launches (0 restores the default);
 * withhold_one_load != 0 makes the operand producer of every CTA leave out the last load of its first
 * tile, so that the waits depending on it run into the limit.  Together they let a test see the timeout
 * path end to end without a fault, a trap or an unbounded spin.  No counterpart in the reference.
 */
I8L_API int i8l_test_set_wait_limit(uint32_t max_polls, int withhold_one_load);

/* Text of the calling thread's most recent error ("" if none). */
I8L_API const char* i8l_last_error(void);

/* Library version, e.g. 100 = 0.1.0 */
I8L_API int i8l_version(void);

#ifdef __cplusplus
}
#endif
#endif /* I8LINEAR_H_ */
