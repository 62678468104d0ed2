// Tiled tcgen05 GEMM with the token operand in tensor memory.
//
// Same product, fused epilogue and tile schedule as gemm_tcgen05.cu (QUIK experiments/qlinear.py:122-145 in one
// launch: int GEMM of src/matmul/matmul.cu:17-55,98-136, outlier F.linear, dequantize of
// src/asymmetric/asymmetric.cu:134-146), but the A operand (the activation codes, or the outlier activations) does not
// go from shared memory to the tensor core through a shared-memory descriptor.  Four warps move every k-block of A from
// its shared-memory stage into a small ring of tensor-memory slots (tcgen05.st), and the products are issued in the
// form that reads A from tensor memory and only B through a descriptor.  Two things follow:
//   * one thread issues tcgen05.mma of this form at the tensor pipe's full rate (128 cycles for 128 x 256 x 32 bytes
//     per SM), whereas with both operands in shared memory one thread needs ~217 cycles per instruction whatever its
//     size (measured), which bounded the other kernel;
//   * 4-bit activation codes travel packed (the reference layout, two per byte, include/int4.h:78-98) from HBM
//     through L2 into shared memory -- half the bytes -- and are widened to signed bytes on their way into tensor
//     memory (each byte = 16 x code; the factor is shifted out of the exact int32 sums in the epilogue).
//
// Roles of a CTA (448 threads): warp 0 TMA producer, warp 1 TMEM allocation + MMA issue, warps 2-5 operand transfer
// (one per tensor-memory lane quarter), warps 6-13 epilogue (gemm_epilogue.cuh).  Tensor memory (512 columns): two
// accumulator regions of block_n columns, then the operand ring (32 columns = 128 bytes of K per row and slot).
// Every wait is bounded (tcgen05_ptx.cuh): a wait that runs out sets the device status word, all roles leave their
// loops, tensor memory is released and the kernel returns.
#include <cuda.h>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tcgen05_ptx.cuh"

namespace quik {
namespace {

constexpr int TS_THREADS = 448;
constexpr int TS_MAX_N = 224;                 // 2 x 224 accumulator columns + 2 operand slots = 512
constexpr int TS_HALF_CAP = 128;              // most columns per epilogue warp
constexpr int TS_A_BYTES = BLOCK_M * STAGE_K_BYTES;           // room for an unpacked k-block of A (packed: first half)
constexpr int TS_MAX_SLOTS = 4;
constexpr int TS_AUX_BYTES = ((512 + 8 * 3 * TS_HALF_CAP * 4) + 1023) / 1024 * 1024;
constexpr int ts_stage_bytes(int ctas) { return TS_A_BYTES + (TS_MAX_N / ctas) * STAGE_K_BYTES; }
constexpr int ts_num_stages(int ctas) {
  const int n = (SMEM_LIMIT - 1024 - TS_AUX_BYTES - 8 * EPI_BUF_BYTES) / ts_stage_bytes(ctas);
  return n > 8 ? 8 : n;
}
constexpr size_t ts_smem_bytes(int ctas) {
  return 1024 + (size_t)ts_num_stages(ctas) * ts_stage_bytes(ctas) + TS_AUX_BYTES + 8 * EPI_BUF_BYTES;
}

// The k-blocks of a CTA in issue order: outlier blocks of tile 0; then per tile j the first half of its integer
// blocks, the outlier blocks of tile j + 1, the second half of its integer blocks (so that the drain of tile j + 1 and
// the epilogue of tile j hide behind integer products).  fn(j, fp, kb) returns false to stop.
template <bool HAS_FP, typename Fn>
__device__ __forceinline__ void for_each_block(int n_local, int int_kb, int fp_kb, Fn fn) {
  const int int_half = (int_kb + 1) / 2;
  bool ok = true;
  auto range = [&](int j, bool fp, int kb0, int kb1) {
    for (int kb = kb0; kb < kb1 && ok; ++kb) ok = fn(j, fp, kb);
  };
  if (HAS_FP && n_local > 0) range(0, true, 0, fp_kb);
  for (int j = 0; j < n_local && ok; ++j) {
    range(j, false, 0, int_half);
    if (HAS_FP && j + 1 < n_local) range(j + 1, true, 0, fp_kb);
    range(j, false, int_half, int_kb);
  }
}

template <typename T, bool HAS_FP, int CTAS, bool A_PACKED>
__global__ void __launch_bounds__(TS_THREADS, 1)
gemm_tcgen05_ts_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_fa, const __grid_constant__ CUtensorMap tmap_fb,
                       const GemmParams p) {
  constexpr int STAGE_BYTES = ts_stage_bytes(CTAS);
  constexpr int STAGES = ts_num_stages(CTAS);
  constexpr int TILE_M = BLOCK_M * CTAS;
  constexpr int A_INT_BYTES = A_PACKED ? TS_A_BYTES / 2 : TS_A_BYTES;     // bytes of one integer k-block of A
  const int bn = p.block_n;
  const int b_rows = bn / CTAS;                               // B rows this CTA loads per k-block
  const uint32_t b_tx = (uint32_t)(b_rows * STAGE_K_BYTES) * CTAS;          // B bytes of the whole pair per k-block
  const int slots = p.a_slots;
  const uint32_t a_col0 = 2 * bn;                             // first column of the operand ring

  extern __shared__ unsigned char smem_dyn[];
  unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char *aux = tiles + STAGES * STAGE_BYTES;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(aux);               // [STAGES] B of the stage has landed (pair leader)
  uint64_t *a_bar = full_bar + STAGES;                                 // [STAGES] A of the stage has landed (this CTA)
  uint64_t *empty_bar = a_bar + STAGES;                                // [STAGES] stage consumed (this CTA)
  uint64_t *a_full = empty_bar + STAGES;                               // [4] operand slot written (pair leader)
  uint64_t *a_empty = a_full + TS_MAX_SLOTS;                           // [4] operand slot consumed (this CTA)
  uint64_t *acc_full = a_empty + TS_MAX_SLOTS;                         // [2] integer product complete
  uint64_t *acc_empty = acc_full + 2;                                  // [2] region free again
  uint64_t *fp_full = acc_empty + 2;                                   // [2] outlier product complete
  uint64_t *fp_drained = fp_full + 2;                                  // [2] outlier product parked
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(fp_drained + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float *s_vec = reinterpret_cast<float *>(aux + 512);                 // [8][3][TS_HALF_CAP]
  unsigned char *s_out = aux + TS_AUX_BYTES;                           // [8][32 x 64 bytes]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(a_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), 1 + 4);                     // MMA commit + the four transfer warps
    }
    for (int s = 0; s < TS_MAX_SLOTS; ++s) {
      mbar_init(smem_u32(a_full + s), 4 * CTAS);                     // transfer warps of the whole pair
      mbar_init(smem_u32(a_empty + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(acc_full + s), 1);
      mbar_init(smem_u32(acc_empty + s), NUM_EPI_THREADS * CTAS);    // epilogue threads of the whole pair
      mbar_init(smem_u32(fp_full + s), 1);
      mbar_init(smem_u32(fp_drained + s), NUM_EPI_THREADS * CTAS);
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
    tmem_alloc<CTAS>(smem_u32(tmem_slot), 512);
    tmem_relinquish<CTAS>();
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();          // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                                 // set-up done; everything below reads or writes global memory

  const int rank = CTAS == 2 ? (int)cluster_ctarank() : 0;
  const int unit = (int)blockIdx.x / CTAS, num_units = (int)gridDim.x / CTAS;    // a unit = CTA or CTA pair
  const int n_local = (p.num_tiles - unit + num_units - 1) / num_units;           // tiles of this unit

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for_each_block<HAS_FP>(n_local, p.int_kb, p.fp_kb, [&](int j, bool fp, int kb) {
        const int tile = unit + j * num_units;
        const int m0 = (tile % p.num_m_tiles) * TILE_M + rank * BLOCK_M;      // this CTA's rows of A
        const int n0 = (tile / p.num_m_tiles) * bn + rank * b_rows;           // this CTA's rows of B
        if (!mbar_wait(smem_u32(empty_bar + stage), phase ^ 1, abort_flag, p.status)) return false;
        const uint32_t fb = smem_u32(full_bar + stage), ab = smem_u32(a_bar + stage);
        const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
        if (rank == 0) mbar_expect_tx(fb, b_tx);
        mbar_expect_tx(ab, fp ? TS_A_BYTES : A_INT_BYTES);
        if (fp) {
          tma_load_2d<1>(sa, &tmap_fa, ab, kb * 64, m0);
          tma_load_2d<CTAS>(sa + TS_A_BYTES, &tmap_fb, fb, kb * 64, n0);
        } else {
          tma_load_2d<1>(sa, &tmap_a, ab, kb * (A_PACKED ? STAGE_K_BYTES / 2 : STAGE_K_BYTES), m0);
          tma_load_2d<CTAS>(sa + TS_A_BYTES, &tmap_b, fb, kb * STAGE_K_BYTES, n0);
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
        return true;
      });
    }
  } else if (warp == 1) {
    // ================= MMA issuer (pair leader only) =================
    if (lane == 0 && rank == 0) {
      int stage = 0, slot = 0;
      uint32_t phase = 0, slot_phase = 0;
      long long w_region = 0, w_full = 0, w_a = 0;
      const long long t_begin = clock64();
      for_each_block<HAS_FP>(n_local, p.int_kb, p.fp_kb, [&](int j, bool fp, int kb) {
        const int r = j & 1;
        const uint32_t use_parity = (uint32_t)(j >> 1) & 1u;
        const uint32_t d = tmem_base + r * bn;
        if (kb == 0) {
          // the region must be free: after the previous tile's epilogue (outlier product, or integer product of
          // an outlier-free layer), or after this tile's drain
          const bool after_drain = HAS_FP && !fp;
          const uint32_t bar = smem_u32((after_drain ? fp_drained : acc_empty) + r);
          const long long t0 = clock64();
          if (!mbar_wait(bar, after_drain ? use_parity : (use_parity ^ 1u), abort_flag, p.status)) return false;
          w_region += clock64() - t0;
        }
        const long long t1 = clock64();
        if (!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag, p.status)) return false;
        const long long t2 = clock64();
        w_full += t2 - t1;
        if (!mbar_wait(smem_u32(a_full + slot), slot_phase, abort_flag, p.status)) return false;
        w_a += clock64() - t2;
        tc_fence_after();
        const uint64_t db = make_smem_desc(smem_u32(tiles + stage * STAGE_BYTES) + TS_A_BYTES);
        const uint32_t a = tmem_base + a_col0 + slot * 32;
#pragma unroll
        for (int k = 0; k < STAGE_K_BYTES / 32; ++k) {
          // 32 bytes of K per instruction: 8 tensor-memory columns of A, +2 in the descriptor's 16-byte address field of B
          const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
          if (fp) mma_f16_ts<CTAS>(d, a + 8 * k, db + 2 * k, p.idesc_fp, accumulate);
          else mma_i8_ts<CTAS>(d, a + 8 * k, db + 2 * k, p.idesc_int, accumulate);
        }
        mma_commit<CTAS>(smem_u32(empty_bar + stage));    // B of the stage reusable once these MMAs retire
        mma_commit<CTAS>(smem_u32(a_empty + slot));       // ... and the operand slot
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
        if (++slot == slots) { slot = 0; slot_phase ^= 1; }
        if (fp && kb == p.fp_kb - 1) mma_commit<CTAS>(smem_u32(fp_full + r));
        if (!fp && kb == p.int_kb - 1) mma_commit<CTAS>(smem_u32(acc_full + r));
        return true;
      });
      if (p.dbg) {
        unsigned long long *dd = p.dbg + (size_t)blockIdx.x * 16;
        dd[0] = (unsigned long long)(clock64() - t_begin);   // MMA thread: issue loop
        dd[1] = (unsigned long long)w_region;                // ... waiting for a free accumulator region
        dd[2] = (unsigned long long)w_full;                  // ... waiting for B operands
        dd[3] = (unsigned long long)n_local;
        dd[8] = (unsigned long long)w_a;                     // ... waiting for A in tensor memory
      }
    }
  } else if (warp < 6) {
    // ================= operand transfer (warps 2..5): shared memory -> registers -> tensor memory =================
    const int q = warp & 3;                   // tensor-memory lane quarter this warp may access
    const int row = q * 32 + lane;            // row of the CTA's A tile this thread moves
    int stage = 0, slot = 0;
    uint32_t phase = 0, slot_phase = 0;
    long long c_full = 0, c_slot = 0;
    for_each_block<HAS_FP>(n_local, p.int_kb, p.fp_kb, [&](int j, bool fp, int kb) {
      const long long t0 = clock64();
      const bool landed = mbar_wait(smem_u32(a_bar + stage), phase, abort_flag, p.status);
      if (!__all_sync(0xffffffffu, landed)) return false;
      c_full += clock64() - t0;
      const unsigned char *sa = tiles + stage * STAGE_BYTES;
      uint32_t v[32];
      if (A_PACKED && !fp) {
        // 64 packed bytes per row under the 64-byte swizzle: 16-byte chunk c sits at chunk position c ^ ((row / 2) % 4)
        const unsigned char *arow = sa + row * 64;
        uint4 pk[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) pk[c] = *reinterpret_cast<const uint4 *>(arow + ((c ^ ((row >> 1) & 3)) << 4));
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          widen8(pk[c].x, v[8 * c + 0], v[8 * c + 1]);
          widen8(pk[c].y, v[8 * c + 2], v[8 * c + 3]);
          widen8(pk[c].z, v[8 * c + 4], v[8 * c + 5]);
          widen8(pk[c].w, v[8 * c + 6], v[8 * c + 7]);
        }
      } else {
        // 128 bytes per row under the 128-byte swizzle: chunk c sits at chunk position c ^ (row % 8)
        const unsigned char *arow = sa + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 w = *reinterpret_cast<const uint4 *>(arow + ((c ^ (row & 7)) << 4));
          v[4 * c + 0] = w.x; v[4 * c + 1] = w.y; v[4 * c + 2] = w.z; v[4 * c + 3] = w.w;
        }
      }
      const long long t1 = clock64();
      const bool free_slot = mbar_wait(smem_u32(a_empty + slot), slot_phase ^ 1u, abort_flag, p.status);
      if (!__all_sync(0xffffffffu, free_slot)) return false;
      c_slot += clock64() - t1;
      tc_fence_after();
      tmem_st32(tmem_base + ((uint32_t)(q * 32) << 16) + a_col0 + slot * 32, v);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 1) mbar_arrive(smem_u32(a_full + slot));
        else mbar_arrive_leader(smem_u32(a_full + slot));
        mbar_arrive(smem_u32(empty_bar + stage));          // this warp no longer reads the stage's A
      }
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
      if (++slot == slots) { slot = 0; slot_phase ^= 1; }
      return true;
    });
    if (p.dbg && warp == 2 && lane == 0) {
      unsigned long long *dd = p.dbg + (size_t)blockIdx.x * 16;
      dd[9] = (unsigned long long)c_full;       // transfer warp: waiting for A in shared memory
      dd[10] = (unsigned long long)c_slot;      // ... waiting for a free tensor-memory slot
    }
  } else {
    // ================= epilogue (warps 6..13): gemm_epilogue.cuh =================
    EpilogueWarp<T, HAS_FP, CTAS> ew(p, tmem_base, bn, unit, num_units, rank, warp - 6, warp & 3, lane, s_vec, TS_HALF_CAP,
                                     s_out, acc_full, acc_empty, fp_full, fp_drained, abort_flag);
    ew.run(n_local);
    if (p.dbg && warp == 6 && lane == 0) ew.write_counters((int)blockIdx.x);
  }

  // ---- teardown: every thread arrives here, also after an aborted wait
  if (*abort_flag) {
    // let bulk copies that are still in flight land before shared memory is released
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();          // no CTA leaves while its peer may still address it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, 512);
  }
}

// Largest number of CTA pairs that can be resident at once (0 if pairs cannot be launched).
template <typename Kern>
int ts_max_pairs(Kern kern, size_t smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * num_sms());
  cfg.blockDim = dim3(TS_THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

template <typename T, bool HAS_FP, int CTAS, bool A_PACKED>
int ts_launch_t(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tfa, const CUtensorMap &tfb,
                const GemmParams &p, cudaStream_t st) {
  auto kern = gemm_tcgen05_ts_kernel<T, HAS_FP, CTAS, A_PACKED>;
  constexpr size_t smem = ts_smem_bytes(CTAS);
  static std::mutex mu;
  static int cached[kMaxDevices];       // resident units per device: 0 = not asked yet, -1 = cannot launch
  int dev = 0;
  QUIK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return QUIK_ERR_UNSUPPORTED;
  int resident;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
      QUIK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      const int n = CTAS == 1 ? num_sms() : ts_max_pairs(kern, smem);
      cached[dev] = n > 0 ? n : -1;
    }
    resident = cached[dev];
  }
  if (resident <= 0) return QUIK_ERR_UNSUPPORTED;
  const int units = p.num_tiles < resident ? p.num_tiles : resident;
  LaunchCfg lc(dim3(CTAS * units), dim3(TS_THREADS), smem, st, CTAS);
  QUIK_CUDA_TRY(cudaLaunchKernelEx(&lc.cfg, kern, ta, tb, tfa, tfb, p));
  return check_launch("gemm_tcgen05_ts_kernel");
}

// Tile width for this engine.  The tensor pipe is busy 2 * block_n cycles per CTA and k-block, so unlike the kernel
// with both operands in shared memory a narrower tile costs proportionally less: the width that leaves the fewest idle
// tile slots in the last wave wins, wider first on ties (fewer loads of A per output column).
void ts_choose_tile(int M, int N, int kblocks, int forced_n, int pair_mode, int *ctas_out, int *bn_out) {
  const int sms = num_sms();
  const int n16 = (N + 15) & ~15;
  double best = 0.0;
  bool have = false;
  for (int ctas = 2; ctas >= 1; --ctas) {
    if (ctas == 2 && (pair_mode == 1 || (pair_mode == 0 && M <= BLOCK_M))) continue;
    if (ctas == 1 && pair_mode == 2) continue;
    const int units = ctas == 2 ? sms / 2 : sms;
    const int tile_m = BLOCK_M * ctas;
    for (int bn = TS_MAX_N; bn >= 32; bn -= 16) {
      int cand = bn;
      if (forced_n) {
        if (bn != TS_MAX_N) break;
        cand = forced_n > TS_MAX_N ? TS_MAX_N : forced_n;
      }
      if (cand > n16) cand = n16 < 32 ? 32 : n16;
      const long long tiles = (long long)((M + tile_m - 1) / tile_m) * ((N + cand - 1) / cand);
      const long long waves = (tiles + units - 1) / units;
      const double mma = 2.0 * cand, feed = (BLOCK_M / 2 + cand / ctas) * (double)STAGE_K_BYTES / 64.0;
      const double cost = (double)waves * (kblocks * (mma > feed ? mma : feed) + 3000.0);
      if (!have || cost < best) {
        have = true;
        best = cost;
        *ctas_out = ctas;
        *bn_out = cand;
      }
    }
  }
}

}  // namespace

// A: [M, K] int8 codes, or (a_packed) [M, K/2] packed int4 codes (K counts codes); B: [N, K] int8.
int launch_gemm_tcgen05_ts(const void *A, int a_packed, const int8_t *B, int M, int N, int K, const Epilogue &ep,
                           cudaStream_t st) {
  if (M == 0 || N == 0) return QUIK_OK;
  if (K <= 0 || K % (a_packed ? 32 : 16) != 0) return QUIK_ERR_SHAPE;
  if (!aligned16(A) || !aligned16(B)) return QUIK_ERR_ALIGN;
  const bool has_fp = ep.mode == 1 && ep.fp_a != nullptr && ep.F > 0;
  if (has_fp && (ep.F % 8 != 0 || !aligned16(ep.fp_a) || !aligned16(ep.fp_b))) return QUIK_ERR_ALIGN;

  GemmParams p{};
  p.int_kb = (K + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
  p.fp_kb = has_fp ? (ep.F + 63) / 64 : 0;
  int ctas = 1, block_n = 128;
  ts_choose_tile(M, N, p.int_kb + p.fp_kb, get_tile_n(), get_cta_pair(), &ctas, &block_n);
  const int tile_m = BLOCK_M * ctas;
  const int m_tiles = (M + tile_m - 1) / tile_m;
  fill_epilogue_params(p, ep, M, N);
  if (p.status == nullptr) return QUIK_ERR_CUDA;
  p.block_n = block_n;
  p.split_n = split_columns(block_n);
  p.num_m_tiles = m_tiles;
  p.num_tiles = m_tiles * ((N + block_n - 1) / block_n);
  p.idesc_int = make_idesc(2, 1, tile_m, block_n);
  p.idesc_fp = make_idesc(1, ep.dtype == QUIK_BF16 ? 1 : 0, tile_m, block_n);
  p.acc_shift = a_packed ? 4 : 0;
  const int free_slots = (512 - 2 * block_n) / 32;
  p.a_slots = free_slots > TS_MAX_SLOTS ? TS_MAX_SLOTS : free_slots;

  CUtensorMap ta, tb, tfa, tfb;
  int rc;
  if (a_packed) rc = make_tmap(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K / 2, BLOCK_M, STAGE_K_BYTES / 2);
  else rc = make_tmap(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, BLOCK_M);
  if (rc != QUIK_OK) return rc;
  if ((rc = make_tmap(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, block_n / ctas)) != QUIK_OK) return rc;
  if (has_fp) {
    const CUtensorMapDataType fdt = ep.dtype == QUIK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if ((rc = make_tmap(&tfa, ep.fp_a, fdt, 2, M, ep.F, BLOCK_M)) != QUIK_OK) return rc;
    if ((rc = make_tmap(&tfb, ep.fp_b, fdt, 2, N, ep.F, block_n / ctas)) != QUIK_OK) return rc;
  } else {
    tfa = ta;
    tfb = tb;
  }
#define QUIK_TS_P(T, F, C)                                                                        \
  do {                                                                                            \
    return a_packed ? ts_launch_t<T, F, C, true>(ta, tb, tfa, tfb, p, st)                         \
                    : ts_launch_t<T, F, C, false>(ta, tb, tfa, tfb, p, st);                       \
  } while (0)
#define QUIK_TS_C(T, C)                                                                           \
  do {                                                                                            \
    if (has_fp) QUIK_TS_P(T, true, C);                                                            \
    QUIK_TS_P(T, false, C);                                                                       \
  } while (0)
#define QUIK_TS(T)                                                                                \
  do {                                                                                            \
    if (ctas == 2) QUIK_TS_C(T, 2);                                                               \
    QUIK_TS_C(T, 1);                                                                              \
  } while (0)
  if (ep.dtype == QUIK_BF16) QUIK_TS(__nv_bfloat16);
  QUIK_TS(__half);
#undef QUIK_TS_P
#undef QUIK_TS_C
#undef QUIK_TS
}

// Tile shape this engine would use (diagnostics).
void choose_tile_ts(int M, int N, int kblocks, int *ctas_out, int *bn_out) {
  ts_choose_tile(M, N, kblocks, get_tile_n(), get_cta_pair(), ctas_out, bn_out);
}

}  // namespace quik
