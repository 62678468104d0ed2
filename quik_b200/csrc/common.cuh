// Shared helpers for the quik_b200 CUDA sources: status codes, dtype traits, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/quik_b200.h"

namespace quik {

// ---- host-side error plumbing -------------------------------------------------------------
void set_cuda_error(cudaError_t e, const char *where);   // abi.cu
int num_sms();                                           // abi.cu (cached per device)

#define QUIK_CUDA_TRY(expr)                                        \
  do {                                                             \
    cudaError_t _e = (expr);                                       \
    if (_e != cudaSuccess) {                                       \
      ::quik::set_cuda_error(_e, #expr);                           \
      return QUIK_ERR_CUDA;                                        \
    }                                                              \
  } while (0)

inline int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_cuda_error(e, what);
    return QUIK_ERR_CUDA;
  }
  return QUIK_OK;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- per-device launch state ----------------------------------------------------------------
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) and occupancy answers hold for the device that was
// current when they were made.  A process may drive several GPUs (one layer per device, as the reference's
// llama_multigpu does, experiments/llama.py:295-326) and several host threads, so every launcher keeps
// this state per device ordinal behind a mutex.  One object per kernel instantiation (a function-local static).
constexpr int kMaxDevices = 64;
struct PerDeviceSmem {
  std::mutex mu;
  size_t opted[kMaxDevices] = {};     // bytes of dynamic shared memory opted in to on that device
  int blocks_per_sm[kMaxDevices] = {};
};
// Makes sure `kern` may be launched with `smem` bytes of dynamic shared memory on the current device; when
// `threads` > 0 also reports how many of its blocks fit on one SM (cached per device and size).
template <typename Kern>
int ensure_smem(PerDeviceSmem &st, Kern kern, size_t smem, int threads = 0, int *blocks_per_sm = nullptr) {
  int dev = 0;
  QUIK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return QUIK_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(st.mu);
  if (st.opted[dev] != smem + 1) {       // + 1: a kernel without dynamic shared memory is still recorded
    if (smem > 48 * 1024)
      QUIK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int occ = 0;
    if (threads > 0) {
      QUIK_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, threads, smem));
      if (occ < 1) return QUIK_ERR_UNSUPPORTED;
    }
    st.blocks_per_sm[dev] = occ;
    st.opted[dev] = smem + 1;
  }
  if (blocks_per_sm) *blocks_per_sm = st.blocks_per_sm[dev];
  return QUIK_OK;
}

// ---- launches with programmatic dependent launch ----------------------------------------------
// The layer's kernels (quantizer, GEMM, weight-streaming engines) are launched so that a kernel may start
// while its predecessor in the stream is still running: it sets up (barriers, TMEM, descriptors), asks L2 to
// prefetch its weights (a prefetch returns nothing to the SM and L2 is coherent, so this is safe whoever
// writes that memory) and only then waits for the predecessor to complete (pdl_wait) before its first global
// load or store.  Every kernel launched through LaunchCfg must call pdl_wait() before that point.
// QUIK_CFG_PDL = 0 restores plain stream order.
bool pdl_enabled();                                      // abi.cu

struct LaunchCfg {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attrs[2];
  LaunchCfg(dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster_x = 1) : cfg{} {
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    unsigned n = 0;
    if (cluster_x > 1) {
      attrs[n].id = cudaLaunchAttributeClusterDimension;
      attrs[n].val.clusterDim.x = (unsigned)cluster_x;
      attrs[n].val.clusterDim.y = 1;
      attrs[n].val.clusterDim.z = 1;
      ++n;
    }
    if (pdl_enabled()) {
      attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attrs[n].val.programmaticStreamSerializationAllowed = 1;
      ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
  }
};

#ifdef __CUDACC__
// dependents of this grid may be launched (they still wait for its completion in pdl_wait)
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// all grids this one depends on have completed and their writes are visible
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

// ---- device status word (bounded waits report here); lives in gemm_tcgen05.cu ---------------
int device_status_read(int clear);   // synchronises the device
// tile shape the tcgen05 GEMM uses for an M x N problem of `kblocks` 128-byte k-blocks: CTAs per tile (1, 2) and width
void choose_tile(int M, int N, int kblocks, int *ctas_out, int *bn_out);
void set_tile_n(int n);               // 0 = by shape, else a multiple of 16 in [32, 256]
int get_tile_n();
void set_cta_pair(int mode);           // 0 = by shape, 1 = never, 2 = always
void set_mma_issuers(int n);           // 1 or 2 threads issue the integer products of a tile (shared-memory operand engine)
int get_mma_issuers();
void set_l2_hint(int on);               // token-operand loads of the tiled GEMM carry an L2 evict-last hint
int get_l2_hint();
void set_stream_preload(int on);        // weight-streaming engines load their first weight tiles before waiting for the predecessor
int get_stream_preload();
void set_stream_ring(int mode);         // ring depth policy of the mma.sync streaming engine (QUIK_CFG_STREAM_RING)
int get_stream_ring();
int get_cta_pair();
void set_debug_counters(void *buf);    // device buffer of 16 x uint64 per CTA, or NULL
unsigned long long *get_debug_counters();

// ---- dtype traits ---------------------------------------------------------------------------
template <typename T> struct Traits;
template <> struct Traits<__half> {
  using T2 = __half2;
  static constexpr bool kIsHalf = true;
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half(v); }
  static __device__ __forceinline__ int to_int_rn(__half v) { return __half2int_rn(v); }
};
template <> struct Traits<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static constexpr bool kIsHalf = false;
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ int to_int_rn(__nv_bfloat16 v) { return __bfloat162int_rn(v); }
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- launchers implemented in the individual .cu files ---------------------------------------
int launch_asym_quantize(const void *src, int dtype, int rows, int cols, const void *int_idx,
                         int num_int, const void *fp_idx, int num_fp, int idx_bytes, int bits,
                         int wide, void *dst, void *meta, void *fp_x, cudaStream_t st);
// quantizer with the producer of X fused in (quantize.cu): prod 1 = RMSNorm (aux = weight vector), 2 = SiLU(src) * aux
int launch_asym_quantize_fused(int prod, const void *src, const void *aux, float eps, int dtype, int rows, int cols,
                               const void *int_idx, int num_int, const void *fp_idx, int num_fp, int bits, int wide,
                               void *dst, void *meta, void *fp_x, cudaStream_t st);
int launch_find_meta(const void *src, int dtype, int rows, int cols, int bits, void *meta,
                     cudaStream_t st);
int launch_quantize_old(const void *src, int dtype, const void *meta, int rows, int cols, int bits,
                        void *dst, cudaStream_t st);
int launch_sym_quantize(const void *src, const void *scale, int rows, int cols, int bits, void *dst,
                        cudaStream_t st);
int launch_asym_dequantize(const int32_t *x, const void *meta, const void *scale_col,
                           const void *w_reduced, const void *y, void *out, int dtype, int rows,
                           int cols, int bits, cudaStream_t st);
int launch_sym_dequantize(const void *x, int x_bits, const void *scale_row, const void *scale_col,
                          const void *y, void *out, int rows, int cols, cudaStream_t st);
int launch_unpack_int4(const uint8_t *src, int8_t *dst, int rows, int cols, cudaStream_t st);
int launch_peer_copy_2d(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes,
                        size_t rows, int ctas, cudaStream_t st);
int launch_rotary(void *q, void *k, const void *cos_t, const void *sin_t, int dtype, int tokens, int q_heads,
                  int k_heads, int head_dim, cudaStream_t st);
int launch_bounded_wait_selftest(unsigned int limit_us, int *result, cudaStream_t st);   // selftest.cu

// Epilogue description shared by the GEMM engines.
struct Epilogue {
  int mode;                 // 0: int32 C; 1: dequantize to `out`
  int dtype;                // QUIK_F16 / QUIK_BF16 of every floating operand
  int32_t *C;               // mode 0
  void *out;                // mode 1, [M, N]
  long long ldo;            // row pitch of `out` in elements; 0 = N (dense)
  const void *meta;         // interleaved (scale, zero) per row, or NULL when scale_row is given
  const void *scale_row;    // [M] (fused-op form) or NULL
  const void *zero_row;     // [M] or NULL (symmetric)
  const void *scale_col;    // [N]
  const void *w_reduced;    // [N] or NULL (symmetric)
  const void *bias;         // [N] or NULL
  const void *y;            // [M, N] addend or NULL
  float shift_value;        // 8 / 128 or caller-given
  const void *fp_a;         // [M, F] outlier activations or NULL
  const void *fp_b;         // [N, F] outlier weights or NULL
  int F;
};

int launch_gemm_tcgen05(const int8_t *A, const int8_t *B, int M, int N, int K, const Epilogue &ep,
                        cudaStream_t st);
int launch_gemm_mma_sync(const int8_t *A, const int8_t *B, int M, int N, int K, const Epilogue &ep,
                         cudaStream_t st);
// tcgen05 GEMM with the A operand in tensor memory (gemm_tcgen05_ts.cu): A int8 [M, K], or packed int4 [M, K/2]
// widened on chip when a_packed != 0 (K counts codes); B int8 [N, K]
int launch_gemm_tcgen05_ts(const void *A, int a_packed, const int8_t *B, int M, int N, int K, const Epilogue &ep,
                           cudaStream_t st);
void choose_tile_ts(int M, int N, int kblocks, int *ctas_out, int *bn_out);
int launch_small_m(const void *q, const void *w, int bits, int M, int N, int K_int,
                   const Epilogue &ep, cudaStream_t st);
// TMA-fed mma.sync weight streaming (stream_w_mma.cu): q and w in the reference's storage format
int launch_stream_w_mma(const void *q, const void *w, int bits, int M, int N, int K_int, const Epilogue &ep,
                        cudaStream_t st);
// tcgen05 weight streaming (stream_w.cu): q one code per byte, w packed int4 (bits 4) or int8 (bits 8)
int launch_stream_w(const void *q, const void *w, int bits, int M, int N, int K_int, const Epilogue &ep,
                    cudaStream_t st);

}  // namespace quik
