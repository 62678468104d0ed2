/*
 * quik_b200 -- C ABI of the B200 (sm_100a) implementation of QUIK's mixed-precision
 * quantized linear layer.
 *
 * Every entry point takes plain device pointers and sizes, launches on the CUDA
 * stream it is given (a cudaStream_t passed as void*; NULL = legacy default
 * stream) on the calling thread's current device, never allocates or frees
 * device memory, never synchronises, and returns QUIK_OK (0) or a negative
 * error code (see quik_strerror).  Inputs are borrowed and never modified.
 * Outputs are caller-allocated.  All matrices are dense row-major.
 *
 * Each declaration cites the interface of the reference project
 * (IST-DASLab/QUIK, paths relative to its root) that it replaces.
 */
#ifndef QUIK_B200_H_
#define QUIK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------ */
#define QUIK_OK                 0
#define QUIK_ERR_NULL          -1   /* a required pointer is NULL                               */
#define QUIK_ERR_BITS          -2   /* "bits argument must be either 4 or 8" (asymmetric.cpp:20) */
#define QUIK_ERR_SHAPE         -3   /* size / divisibility requirement violated                 */
#define QUIK_ERR_ALIGN         -4   /* a pointer or row pitch is not 16-byte aligned            */
#define QUIK_ERR_DTYPE         -5   /* dtype code is not QUIK_F16 / QUIK_BF16 (or unsupported)  */
#define QUIK_ERR_CUDA          -6   /* a CUDA runtime / driver call failed (quik_last_cuda_error)*/
#define QUIK_ERR_SCRATCH       -7   /* scratch buffer missing or too small                      */
#define QUIK_ERR_UNSUPPORTED   -8   /* valid for the reference, outside this build's limits     */
#define QUIK_ERR_DEVICE_WAIT   -9   /* a bounded on-device wait ran out (reported via status)   */
#define QUIK_ERR_TOO_LARGE    -10   /* sizes exceed the fixed scratch area of the no-allocation call */

/* ---- element types of floating tensors --------------------------------------------------- */
#define QUIK_F16   0
#define QUIK_BF16  1

/* ---- integer-GEMM engines (quik_config_set(QUIK_CFG_GEMM_ENGINE, ...)) -------------------- */
#define QUIK_CFG_GEMM_ENGINE   1
#define QUIK_ENGINE_AUTO       0    /* the fastest engine measured: tcgen05 with both operands in shared memory         */
#define QUIK_ENGINE_TCGEN05    1    /* tcgen05, both operands read from shared memory                              */
#define QUIK_ENGINE_MMA_SYNC   2    /* legacy mma.sync tensor path (comparison engine)                            */
#define QUIK_ENGINE_TCGEN05_TS 3    /* tcgen05, token operand moved (4-bit codes: widened) into tensor memory; measured
                                       slower (the small operand ring in tensor memory cannot hide the hand-over
                                       latency), kept as the comparison engine for packed 4-bit operand loads     */
/* Output-tile width of the tcgen05 engine: 0 = chosen per problem (so that the tiles fill whole waves of CTAs),
 * else a multiple of 16 from 32 to 256. */
#define QUIK_CFG_TILE_N        2
/* Layers with few tokens (8-bit layers with 17 to QUIK_STREAM_M_MAX tokens always use the tcgen05 streaming engine
 * unless this is 0).  M <= QUIK_SMALL_M_MAX tokens: 1 (default) weight streaming, engine chosen by the size of the
 * weights; 2 mma.sync fed by direct loads; 3 tcgen05 fed by a TMA ring (8-bit layers, and 4-bit layers whose token
 * codes come one per byte); 4 mma.sync fed by a TMA ring; 0 the tensor-core GEMM for 8-bit layers.
 * (4-bit layers also choose by the operand layout, see quik_mixed_linear.) */
#define QUIK_CFG_SMALL_M       3
/* CTA pairs (cta_group::2, 256-row tiles) in the tcgen05 engine: 0 = when M > 128, 1 = never, 2 = always. */
#define QUIK_CFG_CTA_PAIR      4
/* Programmatic dependent launch of the layer's kernels (quantizer, GEMM, weight streaming): 1 (default) a
 * kernel may start, set up and ask L2 to prefetch its weights while its predecessor in the stream still runs;
 * it waits for the predecessor's completion before its first global load or store, so results are those of
 * plain stream order; 0 launches in plain stream order. */
#define QUIK_CFG_PDL           5
/* Threads that issue the integer products of a tile in the tcgen05 engine with both operands in shared memory: 1
 * (default) a single thread issues everything; 2 two threads share the k-slices of every block of a long sum
 * (K_int >= 2048) and accumulate into the same tensor-memory accumulator (integer sums do not depend on the order of
 * their terms; the outlier product stays on one thread).  One thread cannot issue these instructions as fast as the
 * tensor pipe could execute them, but under the board's power limit the second thread was measured to gain 1-2 %. */
#define QUIK_CFG_MMA_ISSUERS   6
/* 1: the tiled tcgen05 engine loads its token operand (re-read by every column tile, small enough for L2) with an L2
 * evict-last hint, so that data streaming through L2 meanwhile does not push it out; 0 (default): plain loads. */
#define QUIK_CFG_L2_HINT       7
/* Weight-streaming engine behind the TMA ring (few tokens).  The weights are constants of the layer, so their loads need
 * not wait for the kernel that produces the token codes.  1 (default): the weight tiles of the first ring fill are
 * loaded before that wait, the token tiles of the same stages after it (measured 56.8 against 58.1 us for the four
 * Llama-2-7B layers at 16 tokens); 0: only an L2 prefetch of the first tiles precedes the wait; 2: like 1 plus an L2
 * prefetch of the later tiles (measured slower: 60.7 us). */
#define QUIK_CFG_STREAM_PRELOAD 8
/* Ring depth of the same engine: a CTA streams at (bytes in flight) / (loaded DRAM latency), and a grid of at most one
 * CTA per SM would leave half of every SM's shared memory unused with the 5-stage ring that two CTAs per SM share.
 * 2 (default): 11 stages when the grid has at most one CTA per SM, and a K split is halved when that brings the grid
 * down to one CTA per SM; 0: 11 stages for such grids, splits unchanged; 1: always 5 stages.  Measured on the four
 * Llama-2-7B layers at 16 tokens: 54.7 / 55.2 / 58.1 us per step for 2 / 0 / 1; no difference on the 70B layers. */
#define QUIK_CFG_STREAM_RING   9

const char *quik_version(void);
const char *quik_strerror(int status);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char *quik_last_cuda_error(void);
/* The settings are process-wide single words meant to be set before the layers run.  Setting one while other threads
 * launch is safe but each of those launches sees either the old or the new value. */
int quik_config_set(int key, int value);
int quik_config_get(int key);
/* Diagnostics: the tile shape the selected tcgen05 engine would use on the current device for M tokens, N output channels,
 * K_int integer and F outlier columns: CTAs per tile (1, or 2 = a CTA pair working on 256 rows) and tile width.
 * No reference counterpart (CUTLASS fixes one threadblock shape per kernel, src/matmul/matmul.cu:24-34). */
int quik_gemm_plan(int M, int N, int K_int, int F, int *ctas, int *block_n);
/* Every on-device wait (mbarrier, flag) is bounded; a kernel whose wait ran out records it in a
 * per-device status word and returns early.  This call synchronises the current device, returns
 * QUIK_OK or QUIK_ERR_DEVICE_WAIT, and clears the word when `clear` is non-zero. */
int quik_device_status(int clear);
/* Self-test of that mechanism (no reference counterpart): launches a one-CTA kernel that waits on a barrier nothing
 * arrives on, for at most limit_us microseconds (1 .. 1,000,000).  The wait gives up like the waits of the product
 * kernels do: the kernel returns normally, *device_result (an int in device memory, may be NULL) is set to 2, and the
 * next quik_device_status call reports QUIK_ERR_DEVICE_WAIT.  Nothing faults or hangs. */
int quik_selftest_bounded_wait(unsigned int limit_us, int *device_result, void *stream);
/* Diagnostics: when `device_buffer` (16 x uint64 per launched CTA, caller-owned device memory) is
 * non-NULL, every tcgen05 GEMM launch writes per-CTA cycle counters there: [0] MMA issue loop,
 * [1] of which waiting for a free accumulator region, [2] waiting for operands, [3] tiles of the CTA,
 * [4] epilogue waiting for an outlier product, [5] waiting for an integer product, [6] parking outlier
 * products, [7] final epilogues.  The ring streaming engine for few tokens (stream_w_mma) writes clock64 at [0] kernel
 * entry, [1] after the wait for its predecessor, [2] first block consumed, [3] last block consumed, [4] after the
 * reduction, [5] end, then [6] its number of k-blocks, [7] its rank in the cluster, [8] the global timer at its end.
 * NULL switches it off (default).  No reference counterpart. */
int quik_debug_counters(void *device_buffer);

/* ==== asymmetric activation quantizer ======================================================
 * Replaces quik.asymmetric.quantize (src/asymmetric/asymmetric.cpp:16-25, kernel
 * src/asymmetric/asymmetric.cu:340-584).
 *   src          [rows, cols]  fp16 / bf16 (dtype)
 *   int_indices  [num_int]     int64 column ids that are quantized, in output order
 *   fp_indices   [num_fp]      int64 column ids copied verbatim, in output order
 *   dst          bits=4: uint8 [rows, num_int/2], element 2j of the gathered row in the low
 *                nibble of byte j;  bits=8: int8 [rows, num_int]
 *   meta         [2*rows] dtype, interleaved (scale, zero) per row
 *   fp_x         [rows, num_fp] dtype
 * Requires num_int + num_fp == cols, num_int even, bits in {4, 8}, cols <= 65536.
 */
int quik_asym_quantize(const void *src, int dtype, int rows, int cols,
                       const int64_t *int_indices, int num_int,
                       const int64_t *fp_indices, int num_fp, int bits,
                       void *dst, void *meta, void *fp_x, void *stream);

/* Same operator with 16-bit column ids (a layer converts its index buffers once) and a
 * choice of code layout: wide != 0 stores one int8 per code for bits=4 as well
 * (dst int8 [rows, num_int]), the operand layout of the tensor-core GEMM.
 * No counterpart in the reference; used by the fused layer path (experiments/qlinear.py:114-117).
 */
int quik_asym_quantize_u16(const void *src, int dtype, int rows, int cols,
                           const uint16_t *int_indices, int num_int,
                           const uint16_t *fp_indices, int num_fp, int bits, int wide,
                           void *dst, void *meta, void *fp_x, void *stream);

/* The same quantizer with the producer of its input fused in, so that the normalised / activated matrix never
 * goes to HBM.  No counterpart in the reference, which quantizes whatever tensor the decoder layer hands to the linear
 * (experiments/qlinear.py:114-117); these cover the two producers of a Llama decoder layer (the groups of
 * experiments/llama.py:402-407): the RMSNorm in front of q/k/v and of gate/up, and SiLU(gate) * up in front of
 * down_proj.  Outputs exactly as quik_asym_quantize_u16 on the produced matrix:
 *   rmsnorm:   y[r,c] = T(float(x[r,c]) * rsqrt(mean_c(x[r,:]^2) + eps)) * norm_weight[c]   (fp32 statistics, rounded
 *              to T, multiplied by the weight in T: the arithmetic of LlamaRMSNorm)
 *   silu_mul:  y[r,c] = T(silu(float(gate[r,c]))) * up[r,c]                                  (both roundings as
 *              torch's F.silu(gate) * up)
 * x, gate, up [rows, cols] dtype; norm_weight [cols] dtype. */
int quik_rmsnorm_quantize_u16(const void *x, const void *norm_weight, float eps, int dtype, int rows, int cols,
                              const uint16_t *int_indices, int num_int,
                              const uint16_t *fp_indices, int num_fp, int bits, int wide,
                              void *dst, void *meta, void *fp_x, void *stream);
int quik_silu_mul_quantize_u16(const void *gate, const void *up, int dtype, int rows, int cols,
                               const uint16_t *int_indices, int num_int,
                               const uint16_t *fp_indices, int num_fp, int bits, int wide,
                               void *dst, void *meta, void *fp_x, void *stream);

/* quik.asymmetric.find_meta (src/asymmetric/asymmetric.cpp:40-44, asymmetric.cu:263-338):
 * meta[2r] = T(fmaxf((max_r - min_r) / (2^bits - 1), 1e-6f)), meta[2r+1] = min_r. */
int quik_asym_find_meta(const void *src, int dtype, int rows, int cols, int bits,
                        void *meta, void *stream);

/* quik.asymmetric.quantizeOld (src/asymmetric/asymmetric.cpp:8-14, asymmetric.cu:13-117):
 * quantize an already gathered matrix with a given meta; dst as in quik_asym_quantize with
 * ceil(cols/2) bytes per row for bits=4. */
int quik_asym_quantize_old(const void *src, int dtype, const void *meta, int rows, int cols,
                           int bits, void *dst, void *stream);

/* quik.asymmetric.dequantize (src/asymmetric/asymmetric.cpp:27-38, asymmetric.cu:119-233):
 * out[r,c] = T(float(x[r,c]) * (s_r * sc_c) + ((z_r + 2^(bits-1) * s_r) * wred_c + float(y[r,c])))
 * in fp32 with one final rounding.  x int32 [rows, cols]; meta [2*rows]; scale_col [cols];
 * w_reduced [cols]; y, out [rows, cols] of dtype. */
int quik_asym_dequantize(const int32_t *x, const void *meta, const void *scale_col,
                         const void *w_reduced, const void *y, void *out, int dtype,
                         int rows, int cols, int bits, void *stream);

/* ==== symmetric ops ========================================================================
 * quik.symmetric.quantize (src/symmetric/symmetric.cpp:9-21, symmetric.cu:6-78), fp16 only:
 * q = rn(src / scale[row]) without clamping; bits=4 packs two nibbles per byte. */
int quik_sym_quantize(const void *src, const void *scale, int rows, int cols, int bits,
                      void *dst, void *stream);
/* quik.symmetric.dequantize (src/symmetric/symmetric.cpp:23-42, symmetric.cu:80-152), fp16:
 * out = hmul(hmul(half(x), scale_row[r]), scale_col[c]) + y; x_bits 8 (int8), 16 (fp16), 32 (int32). */
int quik_sym_dequantize(const void *x, int x_bits, const void *scale_row, const void *scale_col,
                        const void *y, void *out, int rows, int cols, void *stream);

/* ==== integer GEMM =========================================================================
 * quik.matmul.int8Matmul (src/matmul/matmul.cpp:43-48, matmul.cu:98-136):
 * C[m,n] = sum_k A[m,k] * B[n,k], int8 x int8 -> exact int32.  A [M,K], B [N,K], C [M,N].
 * Requires K % 16 == 0 and 16-byte aligned A, B. */
int quik_int8_matmul(const int8_t *A, const int8_t *B, int32_t *C, int M, int N, int K,
                     void *stream);

/* quik.matmul.int4Matmul (src/matmul/matmul.cpp:8-13, matmul.cu:17-55): the same contraction on
 * packed int4 operands, A uint8 [M,K/2], B uint8 [N,K/2] (K counts int4 elements, K % 32 == 0).
 * The operands are widened to int8 in `scratch` (device memory, at least
 * quik_int4_matmul_scratch_bytes(M,N,K) bytes, 256-byte aligned) and fed to the int8 engine. */
size_t quik_int4_matmul_scratch_bytes(int M, int N, int K);
int quik_int4_matmul(const uint8_t *A, const uint8_t *B, int32_t *C, int M, int N, int K,
                     void *scratch, size_t scratch_bytes, void *stream);

/* The same int4 GEMM for callers that cannot hand over scratch memory.  (It has no counterpart in the
 * reference, whose operators allocate through torch.)  Some hosts of this library are not free to call
 * cudaMalloc or an allocating torch routine at the moment they need the product: a serving loop that has
 * given every free byte of the device to its own pool, or a thread that must not trigger the device-wide
 * synchronisation an allocation can imply.  For them the widened operands are kept in a fixed array
 * inside the library image, QUIK_NOALLOC_SCRATCH_BYTES per GPU that loads the library, held until the
 * process exits.  The call performs no allocation and no free of any kind.
 *   - Limit: quik_int4_matmul_scratch_bytes(M, N, K) must not exceed QUIK_NOALLOC_SCRATCH_BYTES
 *     (e.g. (M + N) * K <= 16 Mi); larger problems return QUIK_ERR_TOO_LARGE and launch nothing.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents; every call
 *     rewrites the part it uses, so nothing needs clearing, but two calls that overlap in time on the
 *     GPU (different streams) race on it.  Serialise them.
 * Inputs, output, shapes and result are exactly those of quik_int4_matmul. */
#define QUIK_NOALLOC_SCRATCH_BYTES (16u << 20)
int quik_int4_matmul_fixed_scratch(const uint8_t *A, const uint8_t *B, int32_t *C, int M, int N, int K,
                                   void *stream);

/* Widen packed int4 [rows, cols/2] to int8 [rows, cols] (layout rule of include/int4.h:78-98). */
int quik_unpack_int4(const uint8_t *src, int8_t *dst, int rows, int cols, void *stream);

/* Rotary position embedding in place on the q and k projections of a decoder block (the step between the
 * q/k/v layers and attention; the reference leaves it to transformers' LlamaAttention, which computes
 * x * cos + rotate_half(x) * sin elementwise — this call gives the same bits in one pass).
 * q [tokens, q_heads*head_dim], k [tokens, k_heads*head_dim] row-major, cos_table / sin_table [tokens, head_dim/2]
 * (the angle of position t, pair j: the two halves of a head share it), all of `dtype`; head_dim % 16 == 0;
 * pointers 16-byte aligned. */
int quik_rotary_inplace(void *q, void *k, const void *cos_table, const void *sin_table, int dtype, int tokens,
                        int q_heads, int k_heads, int head_dim, void *stream);

/* ==== fused GEMM + dequantize ==============================================================
 * quik.asymmetric.int4FusedDequantize / int8FusedDequantize
 * (src/asymmetric/asymmetric.cpp:46-88, src/asymmetric/fused_dequantize.cu:9-119) and, with
 * zero_row = w_reduced = NULL, quik.symmetric.int4FusedDequantize / int8FusedDequantize
 * (src/symmetric/symmetric.cpp:44-70, src/symmetric/fused_dequantize.cu:9-107):
 *   out = half(acc * scale_row * scale_col + (zero_row + shift_value * scale_row) * w_reduced + y)
 * evaluated in fp32 with one final rounding (the reference rounds every operation to fp16).
 * A, B: int8 [M,K] / [N,K] when bits == 8; packed int4 when bits == 4 (then scratch as for
 * quik_int4_matmul).  scale_row, zero_row [M]; scale_col, w_reduced [N]; y, out [M,N]; fp16. */
int quik_fused_dequantize(const void *A, const void *B, int bits,
                          const void *scale_row, const void *scale_col, float shift_value,
                          const void *zero_row, const void *w_reduced, const void *y, void *out,
                          int M, int N, int K, void *scratch, size_t scratch_bytes, void *stream);

/* ==== the fused layer ======================================================================
 * Replaces the body of MixedQLinear.forward after the quantizer (experiments/qlinear.py:122-145:
 * F.linear on the outlier columns, int4Matmul / int8Matmul, asymmetric.dequantize) by one launch:
 *   out[m,n] = T( float(sum_k q[m,k] * w[n,k]) * (s_m * sw_n)
 *                 + ((z_m + 2^(bits-1) * s_m) * wred_n + sum_j fp_x[m,j] * fp_w[n,j] + bias_n) )
 *   q        int8 [M, K_int]  activation codes, one per byte (quik_asym_quantize_u16 wide=1), or,
 *            when q_packed != 0, the reference layout (uint8 [M, K_int/2] for bits=4)
 *   w        int8 [N, K_int]  weight codes, one per byte; or packed when w_packed != 0
 *   meta     [2*M] dtype (scale, zero) per row;  scale_col, w_reduced [N] dtype
 *   fp_x     [M, F] dtype, fp_w [N, F] dtype (F may be 0: both NULL);  bias [N] dtype or NULL
 *   out      [M, N] dtype
 * 4-bit layers choose the engine by the operand layout:
 *   q one per byte, w one per byte   tensor-core GEMM (any M);
 *   q packed,       w one per byte   tensor-core GEMM whose token operand is widened on chip on its way into tensor
 *                                    memory (any M, K_int % 32 == 0; engine TCGEN05_TS only);
 *   q one per byte, w packed         weight streaming on tcgen05 (M <= QUIK_STREAM_M_MAX, K_int % 32 == 0): the
 *                                    packed weights are widened on chip on their way to the tensor cores;
 *   q packed,       w packed         weight streaming on mma.sync, direct loads or TMA ring by QUIK_CFG_SMALL_M
 *                                    (M <= QUIK_SMALL_M_MAX, K_int % 32 == 0).
 * The tensor-core engines use `out` as scratch while they run (the rounded outlier product + bias is parked there
 * before the dequantize step, as the reference's F.linear output is rounded, experiments/qlinear.py:124): `out` must
 * not alias any input.
 * K_int % 16 == 0, F % 8 == 0. */
#define QUIK_SMALL_M_MAX 16
/* most tokens the tcgen05 weight-streaming engine takes (q one code per byte, w in storage format) */
#define QUIK_STREAM_M_MAX 128
int quik_mixed_linear(const void *q, int q_packed, const void *w, int w_packed,
                      const void *meta, const void *scale_col, const void *w_reduced,
                      const void *fp_x, const void *fp_w, const void *bias, void *out,
                      int dtype, int M, int N, int K_int, int F, int bits, void *stream);

/* ==== tensor-parallel output assembly ======================================================
 * Strided device-to-device copy (rows x width_bytes, independent pitches) issued on `stream`; runs on
 * the copy engines.  Source or destination may be memory of a peer GPU mapped into this process
 * (symmetric memory / IPC).  Used to pull the [M, N/g] output slabs of the other ranks into the local
 * [M, N] result without occupying SMs.  No counterpart in the reference, which has no multi-GPU path
 * for the layer (experiments/llama.py:295-326 places whole layers on GPUs). */
int quik_copy_2d(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows,
                 void *stream);

/* The same copy as a kernel on `ctas` CTAs of 128 threads (0 = 64) with 16-byte accesses: width, pitches and pointers must be multiples
 * of 16 bytes.  Peer memory is read with plain (cache-volatile) loads over NVLink. */
int quik_copy_2d_sm(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows,
                    int ctas, void *stream);

/* quik_mixed_linear with a row pitch for `out` (in elements, >= N): the layer writes its N columns
 * into a wider row-major matrix, e.g. its column range of a tensor-parallel [M, N_total] result. */
int quik_mixed_linear_ld(const void *q, int q_packed, const void *w, int w_packed,
                         const void *meta, const void *scale_col, const void *w_reduced,
                         const void *fp_x, const void *fp_w, const void *bias, void *out, long long out_pitch,
                         int dtype, int M, int N, int K_int, int F, int bits, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QUIK_B200_H_ */
