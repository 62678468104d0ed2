// extern "C" entry points of libquik_b200: argument validation and dispatch to the kernels.
// The checks mirror the reference's TORCH_CHECKs (QUIK src/asymmetric/asymmetric.cpp:16-44,
// src/asymmetric/asymmetric.cu:185-196,519-524, src/matmul/matmul.cpp:8-48) as status codes.
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace quik {
namespace {
thread_local char g_err[256] = "";
// Process-wide settings of quik_config_set: single words, read once per launch.  They are meant to be set before the
// layers run; changing one while other threads launch gives each launch the old or the new value, never a mix.
std::atomic<int> g_engine{QUIK_ENGINE_AUTO};
std::atomic<int> g_small_m{1};
std::atomic<int> g_stream_preload{1};
std::atomic<int> g_stream_ring{2};
std::atomic<int> g_pdl{1};
}  // namespace

void set_cuda_error(cudaError_t e, const char *where) {
  snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
}

bool pdl_enabled() { return g_pdl != 0; }
void set_stream_preload(int on) { g_stream_preload = on; }
int get_stream_preload() { return g_stream_preload; }
void set_stream_ring(int mode) { g_stream_ring = mode; }
int get_stream_ring() { return g_stream_ring; }

int num_sms() {
  static std::atomic<int> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = cached[dev].load();
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n);
  }
  return n;
}

static bool dtype_ok(int dtype) { return dtype == QUIK_F16 || dtype == QUIK_BF16; }

static int run_int8_gemm(const int8_t *A, const int8_t *B, int M, int N, int K, const Epilogue &ep,
                         cudaStream_t st) {
  const int engine = g_engine.load();
  if (engine == QUIK_ENGINE_MMA_SYNC) return launch_gemm_mma_sync(A, B, M, N, K, ep, st);
  if (engine == QUIK_ENGINE_TCGEN05_TS) return launch_gemm_tcgen05_ts(A, 0, B, M, N, K, ep, st);
  return launch_gemm_tcgen05(A, B, M, N, K, ep, st);
}

}  // namespace quik

using namespace quik;

extern "C" {

const char *quik_version(void) { return "quik_b200 0.1 (sm_100a)"; }

const char *quik_strerror(int status) {
  switch (status) {
    case QUIK_OK: return "ok";
    case QUIK_ERR_NULL: return "a required pointer is NULL";
    case QUIK_ERR_BITS: return "bits argument must be either 4 or 8";
    case QUIK_ERR_SHAPE: return "invalid sizes (column counts must add up, integer columns even / multiple of 16 or 32)";
    case QUIK_ERR_ALIGN: return "pointer or row pitch is not 16-byte aligned";
    case QUIK_ERR_DTYPE: return "unsupported element type";
    case QUIK_ERR_CUDA: return "CUDA call failed";
    case QUIK_ERR_SCRATCH: return "scratch buffer missing or too small";
    case QUIK_ERR_UNSUPPORTED: return "configuration not supported by this build";
    case QUIK_ERR_DEVICE_WAIT: return "a bounded on-device wait ran out";
    case QUIK_ERR_TOO_LARGE: return "operands need more scratch than the library's fixed scratch area holds";
    default: return "unknown status";
  }
}

const char *quik_last_cuda_error(void) { return g_err; }

int quik_config_set(int key, int value) {
  if (key == QUIK_CFG_GEMM_ENGINE) {
    if (value < QUIK_ENGINE_AUTO || value > QUIK_ENGINE_TCGEN05_TS) return QUIK_ERR_UNSUPPORTED;
    g_engine = value;
    return QUIK_OK;
  }
  if (key == QUIK_CFG_TILE_N) {
    if (value != 0 && (value < 32 || value > 256 || value % 16 != 0)) return QUIK_ERR_UNSUPPORTED;
    set_tile_n(value);
    return QUIK_OK;
  }
  if (key == QUIK_CFG_SMALL_M) {
    if (value < 0 || value > 4) return QUIK_ERR_UNSUPPORTED;
    g_small_m = value;
    return QUIK_OK;
  }
  if (key == QUIK_CFG_PDL) {
    g_pdl = value ? 1 : 0;
    return QUIK_OK;
  }
  if (key == QUIK_CFG_CTA_PAIR) {
    if (value < 0 || value > 2) return QUIK_ERR_UNSUPPORTED;
    set_cta_pair(value);
    return QUIK_OK;
  }
  if (key == QUIK_CFG_MMA_ISSUERS) {
    if (value < 1 || value > 2) return QUIK_ERR_UNSUPPORTED;
    set_mma_issuers(value);
    return QUIK_OK;
  }
  if (key == QUIK_CFG_L2_HINT) {
    set_l2_hint(value);
    return QUIK_OK;
  }
  if (key == QUIK_CFG_STREAM_RING) {
    if (value < 0 || value > 2) return QUIK_ERR_UNSUPPORTED;
    g_stream_ring = value;
    return QUIK_OK;
  }
  if (key == QUIK_CFG_STREAM_PRELOAD) {
    if (value < 0 || value > 2) return QUIK_ERR_UNSUPPORTED;
    g_stream_preload = value;
    return QUIK_OK;
  }
  return QUIK_ERR_UNSUPPORTED;
}

int quik_config_get(int key) {
  if (key == QUIK_CFG_SMALL_M) return g_small_m;
  if (key == QUIK_CFG_PDL) return g_pdl;
  if (key == QUIK_CFG_CTA_PAIR) return get_cta_pair();
  if (key == QUIK_CFG_MMA_ISSUERS) return get_mma_issuers();
  if (key == QUIK_CFG_L2_HINT) return get_l2_hint();
  if (key == QUIK_CFG_STREAM_PRELOAD) return g_stream_preload;
  if (key == QUIK_CFG_STREAM_RING) return g_stream_ring;
  if (key == QUIK_CFG_GEMM_ENGINE) return g_engine;
  if (key == QUIK_CFG_TILE_N) return get_tile_n();
  return QUIK_ERR_UNSUPPORTED;
}

int quik_device_status(int clear) { return device_status_read(clear); }

int quik_gemm_plan(int M, int N, int K_int, int F, int *ctas, int *block_n) {
  if (M <= 0 || N <= 0 || K_int <= 0 || F < 0 || !ctas || !block_n) return QUIK_ERR_SHAPE;
  const int kblocks = (K_int + 127) / 128 + (F + 63) / 64;
  if (g_engine.load() == QUIK_ENGINE_TCGEN05_TS) choose_tile_ts(M, N, kblocks, ctas, block_n);
  else choose_tile(M, N, kblocks, ctas, block_n);
  return QUIK_OK;
}

int quik_selftest_bounded_wait(unsigned int limit_us, int *device_result, void *stream) {
  if (limit_us == 0 || limit_us > 1000000u) return QUIK_ERR_SHAPE;
  return launch_bounded_wait_selftest(limit_us, device_result, static_cast<cudaStream_t>(stream));
}

int quik_debug_counters(void *device_buffer) {
  set_debug_counters(device_buffer);
  return QUIK_OK;
}

static int check_quantize_args(const void *src, int dtype, int rows, int cols, const void *int_idx, int num_int,
                               const void *fp_idx, int num_fp, int bits, void *dst, void *meta, void *fp_x) {
  if (bits != 4 && bits != 8) return QUIK_ERR_BITS;
  if (!dtype_ok(dtype)) return QUIK_ERR_DTYPE;
  if (rows < 0 || cols <= 0 || num_int <= 0 || num_fp < 0) return QUIK_ERR_SHAPE;
  if (num_int + num_fp != cols) return QUIK_ERR_SHAPE;   // asymmetric.cu:519-521
  if (num_int % 2 != 0) return QUIK_ERR_SHAPE;           // asymmetric.cu:522-524
  if (cols > 65536) return QUIK_ERR_UNSUPPORTED;
  if (rows == 0) return QUIK_OK;
  if (!src || !int_idx || !dst || !meta) return QUIK_ERR_NULL;
  if (num_fp > 0 && (!fp_idx || !fp_x)) return QUIK_ERR_NULL;
  return QUIK_OK;
}

int quik_asym_quantize(const void *src, int dtype, int rows, int cols, const int64_t *int_indices, int num_int,
                       const int64_t *fp_indices, int num_fp, int bits, void *dst, void *meta, void *fp_x,
                       void *stream) {
  int rc = check_quantize_args(src, dtype, rows, cols, int_indices, num_int, fp_indices, num_fp, bits, dst, meta, fp_x);
  if (rc != QUIK_OK) return rc;
  return launch_asym_quantize(src, dtype, rows, cols, int_indices, num_int, fp_indices, num_fp, 8, bits, 0, dst,
                              meta, fp_x, static_cast<cudaStream_t>(stream));
}

int quik_asym_quantize_u16(const void *src, int dtype, int rows, int cols, const uint16_t *int_indices, int num_int,
                           const uint16_t *fp_indices, int num_fp, int bits, int wide, void *dst, void *meta,
                           void *fp_x, void *stream) {
  int rc = check_quantize_args(src, dtype, rows, cols, int_indices, num_int, fp_indices, num_fp, bits, dst, meta, fp_x);
  if (rc != QUIK_OK) return rc;
  return launch_asym_quantize(src, dtype, rows, cols, int_indices, num_int, fp_indices, num_fp, 2, bits, wide, dst,
                              meta, fp_x, static_cast<cudaStream_t>(stream));
}

int quik_rmsnorm_quantize_u16(const void *x, const void *norm_weight, float eps, int dtype, int rows, int cols,
                              const uint16_t *int_indices, int num_int, const uint16_t *fp_indices, int num_fp, int bits,
                              int wide, void *dst, void *meta, void *fp_x, void *stream) {
  int rc = check_quantize_args(x, dtype, rows, cols, int_indices, num_int, fp_indices, num_fp, bits, dst, meta, fp_x);
  if (rc != QUIK_OK) return rc;
  if (rows > 0 && !norm_weight) return QUIK_ERR_NULL;
  return launch_asym_quantize_fused(1, x, norm_weight, eps, dtype, rows, cols, int_indices, num_int, fp_indices, num_fp,
                                    bits, wide, dst, meta, fp_x, static_cast<cudaStream_t>(stream));
}

int quik_silu_mul_quantize_u16(const void *gate, const void *up, int dtype, int rows, int cols,
                               const uint16_t *int_indices, int num_int, const uint16_t *fp_indices, int num_fp, int bits,
                               int wide, void *dst, void *meta, void *fp_x, void *stream) {
  int rc = check_quantize_args(gate, dtype, rows, cols, int_indices, num_int, fp_indices, num_fp, bits, dst, meta, fp_x);
  if (rc != QUIK_OK) return rc;
  if (rows > 0 && !up) return QUIK_ERR_NULL;
  return launch_asym_quantize_fused(2, gate, up, 0.f, dtype, rows, cols, int_indices, num_int, fp_indices, num_fp, bits,
                                    wide, dst, meta, fp_x, static_cast<cudaStream_t>(stream));
}

int quik_asym_find_meta(const void *src, int dtype, int rows, int cols, int bits, void *meta, void *stream) {
  if (bits != 4 && bits != 8) return QUIK_ERR_BITS;
  if (!dtype_ok(dtype)) return QUIK_ERR_DTYPE;
  if (rows < 0 || cols <= 0) return QUIK_ERR_SHAPE;
  if (rows == 0) return QUIK_OK;
  if (!src || !meta) return QUIK_ERR_NULL;
  return launch_find_meta(src, dtype, rows, cols, bits, meta, static_cast<cudaStream_t>(stream));
}

int quik_asym_quantize_old(const void *src, int dtype, const void *meta, int rows, int cols, int bits, void *dst,
                           void *stream) {
  if (bits != 4 && bits != 8) return QUIK_ERR_BITS;
  if (!dtype_ok(dtype)) return QUIK_ERR_DTYPE;
  if (rows < 0 || cols < 0) return QUIK_ERR_SHAPE;
  if (rows == 0 || cols == 0) return QUIK_OK;
  if (!src || !meta || !dst) return QUIK_ERR_NULL;
  return launch_quantize_old(src, dtype, meta, rows, cols, bits, dst, static_cast<cudaStream_t>(stream));
}

int quik_asym_dequantize(const int32_t *x, const void *meta, const void *scale_col, const void *w_reduced,
                         const void *y, void *out, int dtype, int rows, int cols, int bits, void *stream) {
  if (bits != 4 && bits != 8) return QUIK_ERR_BITS;
  if (!dtype_ok(dtype)) return QUIK_ERR_DTYPE;
  if (rows < 0 || cols < 0) return QUIK_ERR_SHAPE;
  if (rows == 0 || cols == 0) return QUIK_OK;
  if (!x || !meta || !scale_col || !w_reduced || !y || !out) return QUIK_ERR_NULL;
  return launch_asym_dequantize(x, meta, scale_col, w_reduced, y, out, dtype, rows, cols, bits,
                                static_cast<cudaStream_t>(stream));
}

int quik_sym_quantize(const void *src, const void *scale, int rows, int cols, int bits, void *dst, void *stream) {
  if (bits != 4 && bits != 8) return QUIK_ERR_BITS;
  if (rows < 0 || cols < 0) return QUIK_ERR_SHAPE;
  if (rows == 0 || cols == 0) return QUIK_OK;
  if (!src || !scale || !dst) return QUIK_ERR_NULL;
  return launch_sym_quantize(src, scale, rows, cols, bits, dst, static_cast<cudaStream_t>(stream));
}

int quik_sym_dequantize(const void *x, int x_bits, const void *scale_row, const void *scale_col, const void *y,
                        void *out, int rows, int cols, void *stream) {
  if (x_bits != 8 && x_bits != 16 && x_bits != 32) return QUIK_ERR_BITS;
  if (rows < 0 || cols < 0) return QUIK_ERR_SHAPE;
  if (rows == 0 || cols == 0) return QUIK_OK;
  if (!x || !scale_row || !scale_col || !y || !out) return QUIK_ERR_NULL;
  return launch_sym_dequantize(x, x_bits, scale_row, scale_col, y, out, rows, cols,
                               static_cast<cudaStream_t>(stream));
}

int quik_int8_matmul(const int8_t *A, const int8_t *B, int32_t *C, int M, int N, int K, void *stream) {
  if (M < 0 || N < 0 || K <= 0 || K % 16 != 0) return QUIK_ERR_SHAPE;
  if (M == 0 || N == 0) return QUIK_OK;
  if (!A || !B || !C) return QUIK_ERR_NULL;
  if (!aligned16(A) || !aligned16(B)) return QUIK_ERR_ALIGN;
  Epilogue ep{};
  ep.mode = 0;
  ep.C = C;
  return run_int8_gemm(A, B, M, N, K, ep, static_cast<cudaStream_t>(stream));
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

size_t quik_int4_matmul_scratch_bytes(int M, int N, int K) {
  if (M < 0 || N < 0 || K < 0) return 0;
  return align256((size_t)M * K) + align256((size_t)N * K);
}

int quik_unpack_int4(const uint8_t *src, int8_t *dst, int rows, int cols, void *stream) {
  if (rows < 0 || cols < 0 || cols % 2 != 0) return QUIK_ERR_SHAPE;
  if (rows == 0 || cols == 0) return QUIK_OK;
  if (!src || !dst) return QUIK_ERR_NULL;
  return launch_unpack_int4(src, dst, rows, cols, static_cast<cudaStream_t>(stream));
}

int quik_rotary_inplace(void *q, void *k, const void *cos_table, const void *sin_table, int dtype, int tokens,
                        int q_heads, int k_heads, int head_dim, void *stream) {
  if (tokens < 0 || q_heads < 0 || k_heads < 0 || head_dim <= 0 || head_dim % 16 != 0) return QUIK_ERR_SHAPE;
  if (dtype != QUIK_F16 && dtype != QUIK_BF16) return QUIK_ERR_DTYPE;
  if (tokens == 0 || q_heads + k_heads == 0) return QUIK_OK;
  if (!cos_table || !sin_table || (q_heads && !q) || (k_heads && !k)) return QUIK_ERR_NULL;
  if (!aligned16(cos_table) || !aligned16(sin_table) || (q_heads && !aligned16(q)) || (k_heads && !aligned16(k)))
    return QUIK_ERR_ALIGN;
  return launch_rotary(q, k, cos_table, sin_table, dtype, tokens, q_heads, k_heads, head_dim,
                       static_cast<cudaStream_t>(stream));
}

// Brings packed int4 operands into the form the selected engine takes: the engine with the token operand in tensor
// memory reads A packed and widens it on chip, so only B is widened into scratch; the others need both one per byte.
// Returns the engine call's status.
static int run_int4_gemm(const uint8_t *A, const uint8_t *B, int M, int N, int K, void *scratch, size_t scratch_bytes,
                         const Epilogue &ep, cudaStream_t st) {
  if (!scratch || scratch_bytes < quik_int4_matmul_scratch_bytes(M, N, K)) return QUIK_ERR_SCRATCH;
  if ((reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return QUIK_ERR_ALIGN;
  int8_t *a8 = static_cast<int8_t *>(scratch);
  int8_t *b8 = a8 + align256((size_t)M * K);
  const int engine = g_engine.load();
  const bool on_chip = engine == QUIK_ENGINE_TCGEN05_TS && aligned16(A);
  int rc = launch_unpack_int4(B, b8, N, K, st);
  if (rc != QUIK_OK) return rc;
  if (on_chip) return launch_gemm_tcgen05_ts(A, 1, b8, M, N, K, ep, st);
  rc = launch_unpack_int4(A, a8, M, K, st);
  if (rc != QUIK_OK) return rc;
  return run_int8_gemm(a8, b8, M, N, K, ep, st);
}

int quik_int4_matmul(const uint8_t *A, const uint8_t *B, int32_t *C, int M, int N, int K, void *scratch,
                     size_t scratch_bytes, void *stream) {
  if (M < 0 || N < 0 || K <= 0 || K % 32 != 0) return QUIK_ERR_SHAPE;
  if (M == 0 || N == 0) return QUIK_OK;
  if (!A || !B || !C) return QUIK_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Epilogue ep{};
  ep.mode = 0;
  ep.C = C;
  return run_int4_gemm(A, B, M, N, K, scratch, scratch_bytes, ep, st);
}

int quik_fused_dequantize(const void *A, const void *B, int bits, const void *scale_row, const void *scale_col,
                          float shift_value, const void *zero_row, const void *w_reduced, const void *y, void *out,
                          int M, int N, int K, void *scratch, size_t scratch_bytes, void *stream) {
  if (bits != 4 && bits != 8) return QUIK_ERR_BITS;
  if (M < 0 || N < 0 || K <= 0 || K % (bits == 4 ? 32 : 16) != 0) return QUIK_ERR_SHAPE;
  if (M == 0 || N == 0) return QUIK_OK;
  if (!A || !B || !scale_row || !scale_col || !y || !out) return QUIK_ERR_NULL;
  if ((zero_row == nullptr) != (w_reduced == nullptr)) return QUIK_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (bits == 8 && (!aligned16(A) || !aligned16(B))) return QUIK_ERR_ALIGN;
  Epilogue ep{};
  ep.mode = 1;
  ep.dtype = QUIK_F16;
  ep.out = out;
  ep.scale_row = scale_row;
  ep.zero_row = zero_row;
  ep.scale_col = scale_col;
  ep.w_reduced = w_reduced;
  ep.y = y;
  ep.shift_value = shift_value;
  if (bits == 4)
    return run_int4_gemm(static_cast<const uint8_t *>(A), static_cast<const uint8_t *>(B), M, N, K, scratch, scratch_bytes,
                         ep, st);
  return run_int8_gemm(static_cast<const int8_t *>(A), static_cast<const int8_t *>(B), M, N, K, ep, st);
}

int quik_mixed_linear(const void *q, int q_packed, const void *w, int w_packed, const void *meta,
                      const void *scale_col, const void *w_reduced, const void *fp_x, const void *fp_w,
                      const void *bias, void *out, int dtype, int M, int N, int K_int, int F, int bits,
                      void *stream) {
  return quik_mixed_linear_ld(q, q_packed, w, w_packed, meta, scale_col, w_reduced, fp_x, fp_w, bias, out, N, dtype, M, N,
                              K_int, F, bits, stream);
}

int quik_mixed_linear_ld(const void *q, int q_packed, const void *w, int w_packed, const void *meta,
                         const void *scale_col, const void *w_reduced, const void *fp_x, const void *fp_w,
                         const void *bias, void *out, long long out_pitch, int dtype, int M, int N, int K_int, int F,
                         int bits, void *stream) {
  if (out_pitch < N) return QUIK_ERR_SHAPE;
  if (bits != 4 && bits != 8) return QUIK_ERR_BITS;
  if (!dtype_ok(dtype)) return QUIK_ERR_DTYPE;
  if (M < 0 || N < 0 || K_int <= 0 || F < 0 || K_int % 16 != 0 || F % 8 != 0) return QUIK_ERR_SHAPE;
  if (M == 0 || N == 0) return QUIK_OK;
  if (!q || !w || !meta || !scale_col || !w_reduced || !out) return QUIK_ERR_NULL;
  if (F > 0 && (!fp_x || !fp_w)) return QUIK_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int small_m = g_small_m.load();
  Epilogue ep{};
  ep.mode = 1;
  ep.dtype = dtype;
  ep.out = out;
  ep.ldo = out_pitch;
  ep.meta = meta;
  ep.scale_col = scale_col;
  ep.w_reduced = w_reduced;
  ep.bias = bias;
  ep.shift_value = bits == 4 ? 8.0f : 128.0f;
  ep.fp_a = F > 0 ? fp_x : nullptr;
  ep.fp_b = F > 0 ? fp_w : nullptr;
  ep.F = F;
  if (bits == 4 && q_packed && !w_packed) {
    // packed token codes against weights one per byte: tensor-core GEMM that widens the tokens on chip
    const int engine = g_engine.load();
    if (engine != QUIK_ENGINE_TCGEN05_TS) return QUIK_ERR_UNSUPPORTED;
    if (K_int % 32 != 0) return QUIK_ERR_SHAPE;
    return launch_gemm_tcgen05_ts(q, 1, static_cast<const int8_t *>(w), M, N, K_int, ep, st);
  }
  if (bits == 4 && w_packed) {
    // packed int4 weights: weight-streaming engines (few tokens only)
    if (K_int % 32 != 0) return QUIK_ERR_SHAPE;
    if (q_packed) {
      // mma.sync engines, both operands packed.  Automatic mode: layers of >= 16 MiB of packed weights go
      // through the TMA-fed ring (it streams faster), smaller ones to the direct-load kernel (it starts faster).
      const bool ring = small_m == 4 || (small_m == 1 && (size_t)N * (size_t)K_int / 2 >= ((size_t)16 << 20));
      return ring ? launch_stream_w_mma(q, w, 4, M, N, K_int, ep, st) : launch_small_m(q, w, 4, M, N, K_int, ep, st);
    }
    return launch_stream_w(q, w, 4, M, N, K_int, ep, st);                   // tcgen05, token codes one per byte
  }
  // one code per byte: int8 layers with few tokens also stream their weights.  Automatic mode, by the size of the
  // weights (measured on 7B and 70B down projections): >= 128 MiB tcgen05 (0.91 of the HBM rate), >= 32 MiB mma.sync
  // behind the TMA ring (0.87 on the large layer, the fastest on the 45 MiB one), below that mma.sync with direct
  // loads (shortest start-up).
  if (bits == 8 && M <= QUIK_SMALL_M_MAX && small_m != 0) {
    const size_t wbytes = (size_t)N * (size_t)K_int;
    int engine = small_m;
    if (engine == 1) engine = wbytes >= ((size_t)128 << 20) ? 3 : (wbytes >= ((size_t)32 << 20) ? 4 : 2);
    if (engine == 3) return launch_stream_w(q, w, 8, M, N, K_int, ep, st);
    if (engine == 4) return launch_stream_w_mma(q, w, 8, M, N, K_int, ep, st);
    return launch_small_m(q, w, 8, M, N, K_int, ep, st);
  }
  // 17 to 128 tokens: the tcgen05 streaming engine takes them at the cost of 16 (the tensor-core GEMM would leave
  // most SMs idle at these sizes)
  if (bits == 8 && M <= QUIK_STREAM_M_MAX && small_m != 0) return launch_stream_w(q, w, 8, M, N, K_int, ep, st);
  return run_int8_gemm(static_cast<const int8_t *>(q), static_cast<const int8_t *>(w), M, N, K_int, ep, st);
}

int quik_copy_2d(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows,
                 void *stream) {
  if (rows == 0 || width_bytes == 0) return QUIK_OK;
  if (!dst || !src) return QUIK_ERR_NULL;
  if (dst_pitch < width_bytes || src_pitch < width_bytes) return QUIK_ERR_SHAPE;
  QUIK_CUDA_TRY(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDeviceToDevice,
                                  static_cast<cudaStream_t>(stream)));
  return QUIK_OK;
}

int quik_copy_2d_sm(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows,
                    int ctas, void *stream) {
  if (rows == 0 || width_bytes == 0) return QUIK_OK;
  if (!dst || !src) return QUIK_ERR_NULL;
  if (dst_pitch < width_bytes || src_pitch < width_bytes || ctas < 0) return QUIK_ERR_SHAPE;
  if (width_bytes % 16 != 0 || dst_pitch % 16 != 0 || src_pitch % 16 != 0 || !aligned16(dst) || !aligned16(src))
    return QUIK_ERR_ALIGN;
  return launch_peer_copy_2d(dst, dst_pitch, src, src_pitch, width_bytes, rows, ctas, static_cast<cudaStream_t>(stream));
}

// ---- int4 GEMM without any caller-provided or freshly allocated scratch -----------------------
// The widened operands live in this fixed device array.  It is part of the library image: every GPU
// that loads the library carries these bytes until the process exits.
static __device__ __align__(256) unsigned char g_fixed_scratch[QUIK_NOALLOC_SCRATCH_BYTES];

namespace {
std::mutex g_fixed_mutex;
void *g_fixed_ptr[kMaxDevices] = {};      // device address of g_fixed_scratch, looked up once per device

// In host code `g_fixed_scratch` is only a handle for the runtime, not a device address; the address
// that kernels may use has to be asked for, with the device in question current.
int fixed_scratch_for_current_device(void **out) {
  int dev = -1;
  QUIK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return QUIK_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_fixed_mutex);
  if (g_fixed_ptr[dev] == nullptr) {
    void *ptr = nullptr;
    QUIK_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_fixed_scratch));
    if (ptr == nullptr) return QUIK_ERR_CUDA;
    g_fixed_ptr[dev] = ptr;
  }
  *out = g_fixed_ptr[dev];
  return QUIK_OK;
}
}  // namespace

int quik_int4_matmul_fixed_scratch(const uint8_t *A, const uint8_t *B, int32_t *C, int M, int N, int K,
                                   void *stream) {
  if (M < 0 || N < 0 || K <= 0 || K % 32 != 0) return QUIK_ERR_SHAPE;
  if (M == 0 || N == 0) return QUIK_OK;           // an empty product needs no scratch, whatever the other size
  if (quik_int4_matmul_scratch_bytes(M, N, K) > (size_t)QUIK_NOALLOC_SCRATCH_BYTES) return QUIK_ERR_TOO_LARGE;
  if (!A || !B || !C) return QUIK_ERR_NULL;
  void *scratch = nullptr;
  int rc = fixed_scratch_for_current_device(&scratch);
  if (rc != QUIK_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the part of the array that a call uses is rewritten in full by that call, so nothing has to be cleared first
  Epilogue ep{};
  ep.mode = 0;
  ep.C = C;
  return run_int4_gemm(A, B, M, N, K, scratch, QUIK_NOALLOC_SCRATCH_BYTES, ep, st);
}

}  // extern "C"
