// int8 x int8 -> int32 GEMM on the Blackwell tensor cores (tcgen05.mma kind::i8) with TMA-fed
// shared-memory tiles, TMEM accumulators and a fused dequantize epilogue that can also add an
// fp16/bf16 "outlier" GEMM (tcgen05.mma kind::f16 into a second TMEM accumulator).
//
// Computes, per 128 x BLOCK_N output tile (QUIK experiments/qlinear.py:122-145 in one launch):
//   acc_i[m,n] = sum_k A[m,k] * B[n,k]            (int8 operands, exact int32)   matmul.cu:98-136
//   acc_f[m,n] = sum_j FA[m,j] * FB[n,j]          (fp16/bf16 operands, fp32)     qlinear.py:124
//   out = T( acc_i * (s_m * sc_n) + ((z_m + shift * s_m) * wred_n + (acc_f + bias_n + y[m,n])) )
//                                                                                asymmetric.cu:134-146
// or stores acc_i as int32 (mode 0).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0    TMA producer: cp.async.bulk.tensor.2d loads of the A / B k-blocks (128 bytes of K
//             per row, 128B swizzle) into a ring of shared-memory stages, completion on mbarriers.
//   warp 1    allocates TMEM; one elected lane issues tcgen05.mma (M=128, N=BLOCK_N, K=32 bytes)
//             from shared-memory descriptors and commits each stage back to the producer.
//   warps 2-5 epilogue: tcgen05.ld the accumulators (32 lanes x 32 columns per warp and step),
//             apply the dequantize arithmetic in fp32 and store 16-byte vectors.
// Outlier k-blocks (64 fp16 values = 128 bytes per row) travel through the same ring before the
// integer k-blocks of a tile.  With BLOCK_N = 256 the integer-only kernel double-buffers the
// accumulator (2 x 256 TMEM columns) so the epilogue of tile i overlaps the MMAs of tile i+1.
// Every wait is bounded: when a limit is hit the kernel records it in a device status word,
// all roles leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace quik {

__device__ unsigned int g_device_status = 0;

namespace {

constexpr int BLOCK_M = 128;
constexpr int STAGE_K_BYTES = 128;           // one 128B-swizzle row of K per stage
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s per wait
int g_tile_n = 0;                                             // 0 = choose by shape

struct GemmParams {
  int M, N;
  int num_m_tiles, num_tiles;
  int int_kb, fp_kb;              // k-blocks per tile: integer (128 B each) and outlier (64 elems)
  uint32_t idesc_int, idesc_fp;   // tcgen05 instruction descriptors
  int mode;                       // 0: int32 C, 1: dequantize
  int32_t *C;
  void *out;
  const void *row_scale;          // element (row * row_stride)
  const void *row_zero;           // may be NULL
  int row_stride;
  const void *scale_col, *w_reduced, *bias, *y;
  float shift_value;
  int vec_out;                    // 16-byte stores allowed (pitch and base aligned)
  int vec_y;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the CTA is aborting (this or another wait ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  uint32_t spins = 0;
  unsigned long long t0 = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++spins) & 0xFFu) == 0) {
      if (*abort_flag) return false;
      const unsigned long long now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicOr(&g_device_status, 1u);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; `accumulate` = 0 overwrites D.
__device__ __forceinline__ void mma_i8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major tile stored as rows of 128 bytes with the 128B
// swizzle (what a TMA box of 128 bytes x rows writes): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);       // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                        // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                        // layout: 128-byte swizzle
  return d;
}

template <typename T> __device__ __forceinline__ float ldf(const void *p, size_t i) {
  return Traits<T>::to_float(static_cast<const T *>(p)[i]);
}

// ---------------------------------------------------------------------------------------------
template <typename T, int BLOCK_N, bool HAS_FP>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_fa, const __grid_constant__ CUtensorMap tmap_fb,
                    const GemmParams p) {
  constexpr int A_BYTES = BLOCK_M * STAGE_K_BYTES;
  constexpr int B_BYTES = BLOCK_N * STAGE_K_BYTES;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int STAGES = (BLOCK_N == 256) ? 4 : 6;
  constexpr int ACC_COLS = BLOCK_N * (HAS_FP ? 2 : 1);        // TMEM columns per accumulator stage
  constexpr int ACC_STAGES = (TMEM_COLS / ACC_COLS) >= 2 ? 2 : 1;

  extern __shared__ unsigned char smem_dyn[];
  // 128B-swizzled tiles need 1024-byte alignment
  unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char *aux = tiles + STAGES * STAGE_BYTES;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(aux);               // [STAGES]
  uint64_t *empty_bar = full_bar + STAGES;                             // [STAGES]
  uint64_t *tmem_full = empty_bar + STAGES;                            // [ACC_STAGES]
  uint64_t *tmem_empty = tmem_full + ACC_STAGES;                       // [ACC_STAGES]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + ACC_STAGES);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // per-column epilogue vectors, one private copy per epilogue warp (no cross-warp barrier needed)
  float *s_vec = reinterpret_cast<float *>(aux + 256);                 // [4][3][BLOCK_N], 16-byte aligned

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      mbar_init(smem_u32(tmem_full + s), 1);
      mbar_init(smem_u32(tmem_empty + s), 128);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    if (HAS_FP) {
      prefetch_tmap(&tmap_fa);
      prefetch_tmap(&tmap_fb);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nkb = p.int_kb + (HAS_FP ? p.fp_kb : 0);

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.num_m_tiles) * BLOCK_M;
        const int n0 = (tile / p.num_m_tiles) * BLOCK_N;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(smem_u32(empty_bar + stage), phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t fb = smem_u32(full_bar + stage);
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          mbar_expect_tx(fb, STAGE_BYTES);
          if (HAS_FP && kb < p.fp_kb) {
            tma_load_2d(sa, &tmap_fa, fb, kb * 64, m0);
            tma_load_2d(sb, &tmap_fb, fb, kb * 64, n0);
          } else {
            const int k0 = (kb - (HAS_FP ? p.fp_kb : 0)) * STAGE_K_BYTES;
            tma_load_2d(sa, &tmap_a, fb, k0, m0);
            tma_load_2d(sb, &tmap_b, fb, k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(smem_u32(tmem_empty + acc), acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_int = tmem_base + acc * ACC_COLS;
        const uint32_t d_fp = d_int + BLOCK_N;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
          const bool is_fp = HAS_FP && kb < p.fp_kb;
          const int kb_local = is_fp ? kb : kb - (HAS_FP ? p.fp_kb : 0);
#pragma unroll
          for (int k = 0; k < STAGE_K_BYTES / 32; ++k) {
            // +32 bytes of K inside the swizzled row = +2 in the 16-byte start-address field
            const uint32_t accumulate = (kb_local > 0 || k > 0) ? 1u : 0u;
            if (is_fp) mma_f16(d_fp, da + 2 * k, db + 2 * k, p.idesc_fp, accumulate);
            else mma_i8(d_int, da + 2 * k, db + 2 * k, p.idesc_int, accumulate);
          }
          mma_commit(smem_u32(empty_bar + stage));          // stage reusable once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(smem_u32(tmem_full + acc));               // accumulator complete -> epilogue
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ================= epilogue (warps 2..5) =================
    const int sub = warp & 3;                 // TMEM lane quarter this warp may read
    float *s_scol = s_vec + (warp - 2) * 3 * BLOCK_N;
    float *s_wred = s_scol + BLOCK_N;
    float *s_bias = s_wred + BLOCK_N;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
      const int m0 = (tile % p.num_m_tiles) * BLOCK_M;
      const int n0 = (tile / p.num_m_tiles) * BLOCK_N;
      if (p.mode == 1) {
        __syncwarp();                         // previous tile's vector reads are done
        for (int c = lane; c < BLOCK_N; c += 32) {
          const int col = n0 + c;
          const bool in = col < p.N;
          s_scol[c] = in ? ldf<T>(p.scale_col, col) : 0.f;
          s_wred[c] = (in && p.w_reduced) ? ldf<T>(p.w_reduced, col) : 0.f;
          s_bias[c] = (in && p.bias) ? ldf<T>(p.bias, col) : 0.f;
        }
        __syncwarp();
      }
      // warp-uniform outcome: tcgen05.ld below is warp-collective
      const bool ready = mbar_wait(smem_u32(tmem_full + acc), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) break;
      tc_fence_after();

      const int row = m0 + sub * 32 + lane;
      const bool row_ok = row < p.M;
      float srow = 0.f, zs = 0.f;
      if (p.mode == 1 && row_ok) {
        srow = ldf<T>(p.row_scale, (size_t)row * p.row_stride);
        const float zrow = p.row_zero ? ldf<T>(p.row_zero, (size_t)row * p.row_stride) : 0.f;
        zs = __fadd_rn(zrow, __fmul_rn(p.shift_value, srow));
      }
      const uint32_t t_int = tmem_base + ((uint32_t)(sub * 32) << 16) + acc * ACC_COLS;

#pragma unroll 1
      for (int c0 = 0; c0 < BLOCK_N; c0 += 32) {
        uint32_t v[32];
        uint32_t f[32];
        __syncwarp();                          // tcgen05.ld is warp-collective: reconverge first
        tmem_ld32(t_int + c0, v);
        if (HAS_FP) tmem_ld32(t_int + BLOCK_N + c0, f);
        tmem_ld_wait();
        const int col0 = n0 + c0;
        const bool full_chunk = col0 + 32 <= p.N;
        const size_t off = (size_t)row * p.N + col0;
        if (!row_ok || col0 >= p.N) {
          // nothing to store for this thread
        } else if (p.mode == 0) {
          if (full_chunk && p.vec_out) {
            int4 *dst = reinterpret_cast<int4 *>(p.C + off);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              dst[j] = make_int4((int)v[4 * j], (int)v[4 * j + 1], (int)v[4 * j + 2], (int)v[4 * j + 3]);
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) p.C[off + j] = (int)v[j];
          }
        } else {
          float o[32];
          T yv[32];
          const bool has_y = p.y != nullptr;
          if (has_y) {
            if (full_chunk && p.vec_y) {
              const uint4 *ys = reinterpret_cast<const uint4 *>(static_cast<const T *>(p.y) + off);
#pragma unroll
              for (int j = 0; j < 4; ++j) reinterpret_cast<uint4 *>(yv)[j] = __ldg(ys + j);
            } else {
              for (int j = 0; j < 32; ++j)
                yv[j] = (col0 + j < p.N) ? static_cast<const T *>(p.y)[off + j] : Traits<T>::from_float(0.f);
            }
          }
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 sc4 = reinterpret_cast<const float4 *>(s_scol + c0)[j4];
            const float4 wr4 = reinterpret_cast<const float4 *>(s_wred + c0)[j4];
            const float4 bi4 = reinterpret_cast<const float4 *>(s_bias + c0)[j4];
            const float sc[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
            const float wr[4] = {wr4.x, wr4.y, wr4.z, wr4.w};
            const float bi[4] = {bi4.x, bi4.y, bi4.z, bi4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = 4 * j4 + e;
              float add = HAS_FP ? __uint_as_float(f[j]) : 0.f;
              add = __fadd_rn(add, bi[e]);
              if (has_y) add = __fadd_rn(add, Traits<T>::to_float(yv[j]));
              add = __fadd_rn(__fmul_rn(zs, wr[e]), add);
              o[j] = __fadd_rn(__fmul_rn((float)(int)v[j], __fmul_rn(srow, sc[e])), add);
            }
          }
          T *dst = static_cast<T *>(p.out) + off;
          if (full_chunk && p.vec_out) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 pk;
              T *pe = reinterpret_cast<T *>(&pk);
#pragma unroll
              for (int e = 0; e < 8; ++e) pe[e] = Traits<T>::from_float(o[8 * j + e]);
              reinterpret_cast<uint4 *>(dst)[j] = pk;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dst[j] = Traits<T>::from_float(o[j]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(tmem_empty + acc));
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---- teardown: every thread arrives here, also after an aborted wait
  if (*abort_flag) {
    // let bulk copies that are still in flight land before shared memory is released
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements; box = 128 bytes of a row x box_rows.
int make_tmap(CUtensorMap *map, const void *base, CUtensorMapDataType dt, int elem_bytes, int rows, int cols,
              int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return QUIK_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(STAGE_K_BYTES / elem_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return QUIK_ERR_CUDA;
  }
  return QUIK_OK;
}

// tcgen05 instruction descriptor: dense, K-major A and B, M = 128.
uint32_t make_idesc(int c_format, int ab_format, int n) {
  uint32_t d = 0;
  d |= (uint32_t)c_format << 4;      // accumulator: 1 = F32, 2 = S32
  d |= (uint32_t)ab_format << 7;     // A format
  d |= (uint32_t)ab_format << 10;    // B format
  d |= (uint32_t)(n >> 3) << 17;     // N / 8
  d |= (uint32_t)(BLOCK_M >> 4) << 24;   // M / 16
  return d;
}

template <int BLOCK_N>
constexpr size_t smem_bytes() {
  constexpr int stages = (BLOCK_N == 256) ? 4 : 6;
  return 1024 /*align slack*/ + (size_t)stages * (BLOCK_M + BLOCK_N) * STAGE_K_BYTES +
         256 /*barriers, TMEM slot, abort flag*/ + 4 * 3 * BLOCK_N * 4 /*epilogue vectors*/;
}

template <typename T, int BLOCK_N, bool HAS_FP>
int launch_t(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tfa, const CUtensorMap &tfb,
             const GemmParams &p, cudaStream_t st) {
  auto kern = gemm_tcgen05_kernel<T, BLOCK_N, HAS_FP>;
  constexpr size_t smem = smem_bytes<BLOCK_N>();
  static bool configured = false;   // per instantiation; the attribute is per function and idempotent
  if (!configured) {
    QUIK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const int grid = p.num_tiles < num_sms() ? p.num_tiles : num_sms();
  kern<<<grid, NUM_THREADS, smem, st>>>(ta, tb, tfa, tfb, p);
  return check_launch("gemm_tcgen05_kernel");
}

}  // namespace

void set_tile_n(int n) { g_tile_n = n; }
int get_tile_n() { return g_tile_n; }

int device_status_read(int clear) {
  unsigned int v = 0;
  QUIK_CUDA_TRY(cudaDeviceSynchronize());
  QUIK_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(v)));
  if (clear && v) {
    unsigned int z = 0;
    QUIK_CUDA_TRY(cudaMemcpyToSymbol(g_device_status, &z, sizeof(z)));
  }
  return v ? QUIK_ERR_DEVICE_WAIT : QUIK_OK;
}

int launch_gemm_tcgen05(const int8_t *A, const int8_t *B, int M, int N, int K, const Epilogue &ep,
                        cudaStream_t st) {
  if (M == 0 || N == 0) return QUIK_OK;
  if (K % 16 != 0 || K <= 0) return QUIK_ERR_SHAPE;
  if (!aligned16(A) || !aligned16(B)) return QUIK_ERR_ALIGN;
  const bool has_fp = ep.mode == 1 && ep.fp_a != nullptr && ep.F > 0;
  if (has_fp && (ep.F % 8 != 0 || !aligned16(ep.fp_a) || !aligned16(ep.fp_b))) return QUIK_ERR_ALIGN;

  // Narrow tiles when wide ones would leave SMs idle.
  const int m_tiles = (M + BLOCK_M - 1) / BLOCK_M;
  const int tiles256 = m_tiles * ((N + 255) / 256);
  int block_n = (N <= 128) ? 128 : (tiles256 >= num_sms() ? 256 : 128);
  if (g_tile_n == 128 || g_tile_n == 256) block_n = g_tile_n;

  GemmParams p{};
  p.M = M;
  p.N = N;
  p.num_m_tiles = m_tiles;
  p.num_tiles = m_tiles * ((N + block_n - 1) / block_n);
  p.int_kb = (K + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
  p.fp_kb = has_fp ? (ep.F + 63) / 64 : 0;
  p.idesc_int = make_idesc(2, 1, block_n);                              // S32 accumulate, signed 8-bit operands
  p.idesc_fp = make_idesc(1, ep.dtype == QUIK_BF16 ? 1 : 0, block_n);   // F32 accumulate, F16 / BF16 operands
  p.mode = ep.mode;
  p.C = ep.C;
  p.out = ep.out;
  if (ep.meta) {
    const size_t eb = 2;
    p.row_scale = ep.meta;
    p.row_zero = static_cast<const unsigned char *>(ep.meta) + eb;
    p.row_stride = 2;
  } else {
    p.row_scale = ep.scale_row;
    p.row_zero = ep.zero_row;
    p.row_stride = 1;
  }
  p.scale_col = ep.scale_col;
  p.w_reduced = ep.w_reduced;
  p.bias = ep.bias;
  p.y = ep.y;
  p.shift_value = ep.shift_value;
  if (ep.mode == 0) p.vec_out = (N % 4 == 0) && aligned16(ep.C);
  else p.vec_out = (N % 8 == 0) && aligned16(ep.out);
  p.vec_y = ep.y && (N % 8 == 0) && aligned16(ep.y);

  CUtensorMap ta, tb, tfa, tfb;
  int rc;
  if ((rc = make_tmap(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, BLOCK_M)) != QUIK_OK) return rc;
  if ((rc = make_tmap(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, block_n)) != QUIK_OK) return rc;
  if (has_fp) {
    const CUtensorMapDataType fdt = ep.dtype == QUIK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if ((rc = make_tmap(&tfa, ep.fp_a, fdt, 2, M, ep.F, BLOCK_M)) != QUIK_OK) return rc;
    if ((rc = make_tmap(&tfb, ep.fp_b, fdt, 2, N, ep.F, block_n)) != QUIK_OK) return rc;
  } else {
    tfa = ta;
    tfb = tb;
  }

#define QUIK_LAUNCH(T)                                                                     \
  do {                                                                                     \
    if (block_n == 256) {                                                                  \
      return has_fp ? launch_t<T, 256, true>(ta, tb, tfa, tfb, p, st)                      \
                    : launch_t<T, 256, false>(ta, tb, tfa, tfb, p, st);                    \
    }                                                                                      \
    return has_fp ? launch_t<T, 128, true>(ta, tb, tfa, tfb, p, st)                        \
                  : launch_t<T, 128, false>(ta, tb, tfa, tfb, p, st);                      \
  } while (0)
  if (ep.dtype == QUIK_BF16) QUIK_LAUNCH(__nv_bfloat16);
  QUIK_LAUNCH(__half);
#undef QUIK_LAUNCH
}

}  // namespace quik
