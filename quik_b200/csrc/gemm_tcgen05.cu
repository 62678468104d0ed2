// int8 x int8 -> int32 GEMM on the Blackwell tensor cores (tcgen05.mma kind::i8) with TMA-fed
// shared-memory tiles, TMEM accumulators and a fused dequantize epilogue that can also add an
// fp16/bf16 "outlier" GEMM (tcgen05.mma kind::f16 into a second TMEM accumulator).
//
// Computes, per 128 x block_n output tile (QUIK experiments/qlinear.py:122-145 in one launch):
//   acc_i[m,n] = sum_k A[m,k] * B[n,k]            (int8 operands, exact int32)   matmul.cu:98-136
//   acc_f[m,n] = sum_j FA[m,j] * FB[n,j]          (fp16/bf16 operands, fp32)     qlinear.py:124
//   out = T( acc_i * (s_m * sc_n) + ((z_m + shift * s_m) * wred_n + (acc_f + bias_n + y[m,n])) )
//                                                                                asymmetric.cu:134-146
// or stores acc_i as int32 (mode 0).
//
// Structure (one persistent CTA per SM or one CTA pair per two SMs, 320 threads per CTA):
//   warp 0    TMA producer: cp.async.bulk.tensor.2d loads of the A / B k-blocks (128 bytes of K
//             per row, 128B swizzle) into a ring of shared-memory stages, completion on mbarriers.
//   warp 1    allocates TMEM; one elected lane issues tcgen05.mma (M=128 or 256, N=block_n, K=32
//             bytes) from shared-memory descriptors and commits each stage back to the producer.
//   warps 2-9 epilogue: tcgen05.ld the accumulators (32 lanes x 32 columns per warp and step),
//             apply the dequantize arithmetic in fp32 and store through a shared-memory transpose.
// Outlier k-blocks (64 fp16 values = 128 bytes per row) travel through the same ring as the integer
// k-blocks; TMEM holds two accumulator regions so the epilogue of tile i overlaps the MMAs of tile
// i+1 (schedule in the comment above the kernel).
// The tile width block_n is a launch parameter (any multiple of 16 up to the kernel's capacity CAP_N,
// which fixes the shared-memory and TMEM plan): the host picks it per problem so that the tiles fill
// whole waves of CTAs (choose_tile below).
// Every wait is bounded: when a limit is hit the kernel records it in a device status word,
// all roles leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tcgen05_ptx.cuh"

namespace quik {

__device__ unsigned int g_device_status = 0;

namespace {

constexpr int NUM_THREADS = 352;              // TMA warp + MMA warp + 8 epilogue warps + second MMA warp
constexpr int SECOND_ISSUER_WARP = 10;
// Process-wide tuning knobs (quik_config_set): plain words, meant to be set once before the layers run; a
// launch reads each of them once.
std::atomic<int> g_tile_n{0};                                 // 0 = choose by shape, else a multiple of 16 in [32, 256]
std::atomic<int> g_cta_pair{0};                               // 0 = by shape, 1 = never, 2 = always
std::atomic<int> g_l2_hint{0};                                // 1 = token-operand loads carry an L2 evict-last hint
std::atomic<int> g_issuers{1};                                // threads that issue the integer products of a tile (1 or 2)
std::atomic<unsigned long long *> g_dbg{nullptr};             // diagnostic counters (device memory), off by default

// Shared-memory plan after the 1024-byte aligned ring of stages: 256 bytes of barriers etc. and the
// per-warp epilogue vectors (rounded to 1024 together), then one output staging chunk per epilogue
// warp (32 rows x 64 bytes).
constexpr int AUX_BYTES(int cap_n) { return ((256 + 8 * 3 * (cap_n / 2) * 4) + 1023) / 1024 * 1024; }
constexpr int stage_bytes(int cap_n, int ctas) { return (BLOCK_M + cap_n / ctas) * STAGE_K_BYTES; }
// Ring depth: as many stages as fit (at most 8).
constexpr int num_stages(int cap_n, int ctas) {
  const int n = (SMEM_LIMIT - 1024 - AUX_BYTES(cap_n) - 8 * EPI_BUF_BYTES) / stage_bytes(cap_n, ctas);
  return n > 8 ? 8 : n;
}

// ---------------------------------------------------------------------------------------------
// Work of one CTA = its tiles t_0, t_1, ... (tile index blockIdx.x + j * gridDim.x).  TMEM holds
// two accumulator regions (CAP_N columns apart); tile j uses region j & 1 for BOTH of its products,
// one after the other:
//   FP(t_j):  outlier k-blocks -> region (f32), drained by the epilogue warps, which round
//             (product + bias) to T and park it in the tile's place in `out` (it stays in L2);
//   INT(t_j): integer k-blocks -> same region (s32), then the final epilogue reads the parked
//             value back (same thread, same address), applies the dequantize arithmetic and
//             overwrites it.
// The MMA issue order is FP(t_0), then for every j: first half of INT(t_j), FP(t_{j+1}), second half
// of INT(t_j).  FP(t_{j+1}) and its drain therefore run in the shadow of INT(t_j), and the epilogue of
// t_j in the shadow of INT(t_{j+1}): the tensor pipe never waits for an epilogue in steady state
// although int32 and fp32 accumulators cannot share a region at the same time.
//
// CTAS == 2: two CTAs on neighbouring SMs (a cluster of 2) work on one 256 x block_n tile.  Each
// loads its own 128 rows of A and only its half of the B rows, so a CTA moves a third less operand
// data per multiply-accumulate than alone.  The leader (cluster rank 0) issues the MMAs for the pair
// and owns the barriers that count loads and region releases; commits reach both CTAs.
template <typename T, int CAP_N, bool HAS_FP, int CTAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_fa, const __grid_constant__ CUtensorMap tmap_fb,
                    const GemmParams p) {
  constexpr int A_BYTES = BLOCK_M * STAGE_K_BYTES;
  constexpr int STAGE_BYTES = stage_bytes(CAP_N, CTAS);      // room for the widest tile; narrower ones use less of it
  constexpr int STAGES = num_stages(CAP_N, CTAS);
  constexpr int TMEM_ALLOC = 2 * CAP_N;                       // two accumulator regions, CAP_N columns apart
  constexpr int HALF_CAP = CAP_N / 2;                         // most columns per epilogue warp
  constexpr int TILE_M = BLOCK_M * CTAS;
  const int bn = p.block_n;
  const int b_rows = bn / CTAS;                               // B rows this CTA loads per k-block
  const uint32_t stage_tx = (uint32_t)(A_BYTES + b_rows * STAGE_K_BYTES) * CTAS;   // bytes of the whole pair

  extern __shared__ unsigned char smem_dyn[];
  // 128B-swizzled tiles need 1024-byte alignment
  unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char *aux = tiles + STAGES * STAGE_BYTES;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(aux);               // [STAGES]
  uint64_t *empty_bar = full_bar + STAGES;                             // [STAGES]
  uint64_t *acc_full = empty_bar + STAGES;                             // [2] integer product complete
  uint64_t *acc_empty = acc_full + 2;                                  // [2] region free again
  uint64_t *fp_full = acc_empty + 2;                                   // [2] outlier product complete
  uint64_t *fp_drained = fp_full + 2;                                  // [2] outlier product parked
  uint64_t *int_started = fp_drained + 2;                              // [2] first integer k-block of the tile complete
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(int_started + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // per-column epilogue vectors, one private copy per epilogue warp (no cross-warp barrier needed)
  float *s_vec = reinterpret_cast<float *>(aux + 256);                 // [8][3][HALF_CAP], 16-byte aligned
  // output staging: [8 warps][32 rows x 64 bytes], 1024-byte aligned
  unsigned char *s_out = tiles + STAGES * STAGE_BYTES + AUX_BYTES(CAP_N);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), p.issuers);                 // every issuing thread commits the stage
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(int_started + s), 1);
      mbar_init(smem_u32(acc_full + s), p.issuers);
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
    tmem_alloc<CTAS>(smem_u32(tmem_slot), TMEM_ALLOC);
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
  const int int_half = (p.int_kb + 1) / 2;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // The token operand A is read again by every column tile of the launch and fits in L2: its lines are marked to
      // be evicted last, so that data streaming through L2 meanwhile (the weights, the outputs, a tensor-parallel
      // rank's peer copies) does not push it out.
      const uint64_t keep = l2_policy_evict_last();
      const bool hint = p.l2_hint != 0;
      // one k-block range of one product of tile j into the ring
      auto feed = [&](int j, bool fp, int kb0, int kb1) {
        const int tile = unit + j * num_units;
        const int m0 = (tile % p.num_m_tiles) * TILE_M + rank * BLOCK_M;      // this CTA's rows of A
        const int n0 = (tile / p.num_m_tiles) * bn + rank * b_rows;           // this CTA's rows of B
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
          if (!mbar_wait(smem_u32(empty_bar + stage), phase ^ 1, abort_flag, p.status)) { ok = false; break; }
          const uint32_t fb = smem_u32(full_bar + stage);
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          if (rank == 0) mbar_expect_tx(fb, stage_tx);
          if (fp) {
            tma_load_2d<CTAS>(sa, &tmap_fa, fb, kb * 64, m0);
            tma_load_2d<CTAS>(sa + A_BYTES, &tmap_fb, fb, kb * 64, n0);
          } else {
            if (hint) tma_load_2d_policy<CTAS>(sa, &tmap_a, fb, kb * STAGE_K_BYTES, m0, keep);
            else tma_load_2d<CTAS>(sa, &tmap_a, fb, kb * STAGE_K_BYTES, m0);
            tma_load_2d<CTAS>(sa + A_BYTES, &tmap_b, fb, kb * STAGE_K_BYTES, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      };
      if (HAS_FP && n_local > 0) feed(0, true, 0, p.fp_kb);
      for (int j = 0; j < n_local && ok; ++j) {
        feed(j, false, 0, int_half);
        if (HAS_FP && j + 1 < n_local) feed(j + 1, true, 0, p.fp_kb);
        feed(j, false, int_half, p.int_kb);
      }
    }
  } else if (warp == 1 || warp == SECOND_ISSUER_WARP) {
    // ================= MMA issuers (pair leader only) =================
    // One thread issues tcgen05.mma with both operands in shared memory no faster than every ~217 cycles (measured,
    // whatever the instruction's size), the tensor pipe needs 128 for the largest one; two threads together reach
    // ~153 in isolation.  Inside this kernel the second thread gains 1-2 % only (the GPU runs into its power limit and
    // lowers the clock instead), so one thread is the default and two are an option (QUIK_CFG_MMA_ISSUERS).
    // With p.issuers == 2 the threads share the integer k-blocks of a tile: thread 0 takes the 32-byte slices
    // 0 and 2 of each block, thread 1 the slices 1 and 3, both into the tile's accumulator.  Integer sums do not
    // depend on the order of their terms, and the tensor pipe applies the multiply-accumulates of one accumulator one
    // after the other whoever issued them (no update is lost: tests/test_gpu_b_matmul.py holds exact products of
    // long sums against the oracle for this mode).  What does need an order is kept on thread 0: the first block of a
    // tile (its first instruction overwrites the accumulator; thread 1 waits until that block is complete before its
    // first instruction of the tile) and the outlier product (floating point: one fixed order).
    const int me = warp == 1 ? 0 : 1;
    if (lane == 0 && rank == 0 && me < p.issuers) {
      const bool shared_work = p.issuers == 2;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long w_region = 0, w_full = 0;
      const long long t_begin = clock64();
      auto issue = [&](int j, bool fp, int kb0, int kb1) {
        const int r = j & 1;
        const uint32_t use_parity = (uint32_t)(j >> 1) & 1u;
        const uint32_t d = tmem_base + r * CAP_N;
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
          if (kb == 0 && me == 0) {
            // the region must be free: after the previous tile's epilogue (outlier product, or
            // integer product of an outlier-free layer), or after this tile's drain
            const bool after_drain = HAS_FP && !fp;
            const uint32_t bar = smem_u32((after_drain ? fp_drained : acc_empty) + r);
            const long long t0 = clock64();
            if (!mbar_wait(bar, after_drain ? use_parity : (use_parity ^ 1u), abort_flag, p.status)) { ok = false; break; }
            w_region += clock64() - t0;
            tc_fence_after();
          }
          if (!fp && kb == 1 && me == 1) {
            if (!mbar_wait(smem_u32(int_started + r), use_parity, abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
          }
          const long long t1 = clock64();
          if (!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag, p.status)) { ok = false; break; }
          w_full += clock64() - t1;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
          const bool alone = !shared_work || fp || kb == 0;       // thread 0 issues the whole block
          if (!alone || me == 0) {
#pragma unroll
            for (int k = 0; k < STAGE_K_BYTES / 32; ++k) {
              if (!alone && (k & 1) != me) continue;
              // +32 bytes of K inside the swizzled row = +2 in the 16-byte start-address field
              const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
              if (fp) mma_f16<CTAS>(d, da + 2 * k, db + 2 * k, p.idesc_fp, accumulate);
              else mma_i8<CTAS>(d, da + 2 * k, db + 2 * k, p.idesc_int, accumulate);
            }
          }
          if (shared_work && me == 0 && !fp && kb == 0) mma_commit<CTAS>(smem_u32(int_started + r));
          mma_commit<CTAS>(smem_u32(empty_bar + stage));    // stage reusable once these MMAs retire (every issuer arrives)
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (fp && kb == p.fp_kb - 1 && me == 0) mma_commit<CTAS>(smem_u32(fp_full + r));
          if (!fp && kb == p.int_kb - 1) mma_commit<CTAS>(smem_u32(acc_full + r));
        }
      };
      if (HAS_FP && n_local > 0) issue(0, true, 0, p.fp_kb);
      for (int j = 0; j < n_local && ok; ++j) {
        issue(j, false, 0, int_half);
        if (HAS_FP && j + 1 < n_local) issue(j + 1, true, 0, p.fp_kb);
        issue(j, false, int_half, p.int_kb);
      }
      if (p.dbg && me == 0) {
        unsigned long long *d = p.dbg + (size_t)blockIdx.x * 16;
        d[0] = (unsigned long long)(clock64() - t_begin);   // MMA thread: issue loop
        d[1] = (unsigned long long)w_region;                // ... waiting for a free accumulator region
        d[2] = (unsigned long long)w_full;                  // ... waiting for operands
        d[3] = (unsigned long long)n_local;
      }
    }
  } else {
    // ================= epilogue (warps 2..9): gemm_epilogue.cuh =================
    EpilogueWarp<T, HAS_FP, CTAS> ew(p, tmem_base, CAP_N, unit, num_units, rank, warp - 2, warp & 3, lane, s_vec,
                                     HALF_CAP, s_out, acc_full, acc_empty, fp_full, fp_drained, abort_flag);
    ew.run(n_local);
    if (p.dbg && warp == 2 && lane == 0) ew.write_counters((int)blockIdx.x);
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
    tmem_dealloc<CTAS>(tmem_base, TMEM_ALLOC);
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

}  // namespace

int make_tmap(CUtensorMap *map, const void *base, CUtensorMapDataType dt, int elem_bytes, int rows, int cols,
              int box_rows, int box_row_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return QUIK_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(box_row_bytes / elem_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = box_row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return QUIK_ERR_CUDA;
  }
  return QUIK_OK;
}

// m = 128 (one CTA) or 256 (CTA pair)
uint32_t make_idesc(int c_format, int ab_format, int m, int n) {
  uint32_t d = 0;
  d |= (uint32_t)c_format << 4;      // accumulator: 1 = F32, 2 = S32
  d |= (uint32_t)ab_format << 7;     // A format
  d |= (uint32_t)ab_format << 10;    // B format
  d |= (uint32_t)(n >> 3) << 17;     // N / 8
  d |= (uint32_t)(m >> 4) << 24;     // M / 16
  return d;
}

unsigned int *device_status_word() {
  void *p = nullptr;
  if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return static_cast<unsigned int *>(p);
}

namespace {

constexpr size_t smem_bytes(int cap_n, int ctas) {
  return 1024 /*align slack*/ + (size_t)num_stages(cap_n, ctas) * stage_bytes(cap_n, ctas) + AUX_BYTES(cap_n) +
         8 * EPI_BUF_BYTES;
}

// Largest number of CTA pairs that can be resident at once (0 if pairs cannot be launched).
template <typename Kern>
int max_pairs(Kern kern, size_t smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * num_sms());
  cfg.blockDim = dim3(NUM_THREADS);
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

// Units (CTAs, or CTA pairs) of one kernel instantiation that are resident at once on the current device.
// The shared-memory opt-in and the occupancy answer belong to a device, so they are kept per device ordinal.
template <typename T, int CAP_N, bool HAS_FP, int CTAS>
int resident_units(int *out) {
  static std::mutex mu;
  static int cached[kMaxDevices];       // 0 = not asked yet, -1 = cannot launch
  int dev = 0;
  QUIK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return QUIK_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    auto kern = gemm_tcgen05_kernel<T, CAP_N, HAS_FP, CTAS>;
    constexpr size_t smem = smem_bytes(CAP_N, CTAS);
    QUIK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int n = CTAS == 1 ? num_sms() : max_pairs(kern, smem);
    cached[dev] = n > 0 ? n : -1;
  }
  *out = cached[dev];
  return QUIK_OK;
}

template <typename T, int CAP_N, bool HAS_FP, int CTAS>
int launch_t(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tfa, const CUtensorMap &tfb,
             const GemmParams &p, cudaStream_t st) {
  auto kern = gemm_tcgen05_kernel<T, CAP_N, HAS_FP, CTAS>;
  constexpr size_t smem = smem_bytes(CAP_N, CTAS);
  int resident = 0;
  const int rc = resident_units<T, CAP_N, HAS_FP, CTAS>(&resident);
  if (rc != QUIK_OK) return rc;
  if (resident <= 0) return QUIK_ERR_UNSUPPORTED;
  const int units = p.num_tiles < resident ? p.num_tiles : resident;
  LaunchCfg lc(dim3(CTAS * units), dim3(NUM_THREADS), smem, st, CTAS);
  QUIK_CUDA_TRY(cudaLaunchKernelEx(&lc.cfg, kern, ta, tb, tfa, tfb, p));
  return check_launch("gemm_tcgen05_kernel");
}

// ---- tile shape per problem -------------------------------------------------------------------
// A launch is a number of waves of equally sized tiles over the resident units (CTAs or CTA pairs).  Measured on the
// Llama-2 shapes (7B at 2048 tokens, 70B at 4096, and their column shards for 2/4/8 GPUs): the time of a tile hardly
// depends on its width -- a tcgen05.mma with both operands in shared memory occupies its issuing thread ~217 cycles
// whatever its N -- so per k-block a tile costs about kBlockClk + kColClk * block_n cycles.  A narrower tile is
// therefore almost as expensive as the widest one and only pays where it saves a whole wave; among widths with the
// same number of waves the narrowest wins by a little.
constexpr double kBlockClk = 366.0;
constexpr double kColClk = 0.45;
constexpr double kTileFixedClk = 1500.0;

double tile_cost(int M, int N, int kblocks, int ctas, int bn, int units) {
  const int tile_m = BLOCK_M * ctas;
  const long long tiles = (long long)((M + tile_m - 1) / tile_m) * ((N + bn - 1) / bn);
  const long long waves = (tiles + units - 1) / units;
  return (double)waves * (kblocks * (kBlockClk + kColClk * bn) + kTileFixedClk);
}

}  // namespace

void choose_tile(int M, int N, int kblocks, int *ctas_out, int *bn_out) {
  const int forced_n = g_tile_n.load(), pair_mode = g_cta_pair.load();
  const int sms = num_sms();
  const int n16 = (N + 15) & ~15;
  double best = 0.0;
  int best_ctas = 1, best_bn = 128;
  bool have = false;
  for (int ctas = 2; ctas >= 1; --ctas) {
    if (ctas == 2 && (pair_mode == 1 || (pair_mode == 0 && M <= BLOCK_M))) continue;
    if (ctas == 1 && pair_mode == 2) continue;
    const int units = ctas == 2 ? sms / 2 : sms;
    for (int bn = 256; bn >= 32; bn -= 16) {
      int cand = bn;
      if (forced_n) {
        if (bn != 256) break;                       // one candidate only
        cand = forced_n;
      }
      if (cand > n16) cand = n16 < 32 ? 32 : n16;   // a tile wider than the matrix only wastes columns
      const double c = tile_cost(M, N, kblocks, ctas, cand, units);
      if (!have || c < best) {
        have = true;
        best = c;
        best_ctas = ctas;
        best_bn = cand;
      }
    }
  }
  *ctas_out = best_ctas;
  *bn_out = best_bn;
}

void set_tile_n(int n) { g_tile_n.store(n); }
int get_tile_n() { return g_tile_n.load(); }
void set_debug_counters(void *buf) { g_dbg.store(static_cast<unsigned long long *>(buf)); }
unsigned long long *get_debug_counters() { return g_dbg.load(); }
void set_l2_hint(int on) { g_l2_hint.store(on ? 1 : 0); }
int get_l2_hint() { return g_l2_hint.load(); }
void set_mma_issuers(int n) { g_issuers.store(n); }
int get_mma_issuers() { return g_issuers.load(); }
void set_cta_pair(int mode) { g_cta_pair.store(mode); }
int get_cta_pair() { return g_cta_pair.load(); }

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

  GemmParams p{};
  p.int_kb = (K + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
  p.fp_kb = has_fp ? (ep.F + 63) / 64 : 0;
  int ctas = 1, block_n = 128;
  choose_tile(M, N, p.int_kb + p.fp_kb, &ctas, &block_n);
  const int tile_m = BLOCK_M * ctas;
  const int m_tiles = (M + tile_m - 1) / tile_m;
  const int cap_n = block_n <= 128 ? 128 : 256;

  fill_epilogue_params(p, ep, M, N);
  if (p.status == nullptr) return QUIK_ERR_CUDA;
  p.block_n = block_n;
  p.split_n = split_columns(block_n);
  p.num_m_tiles = m_tiles;
  p.num_tiles = m_tiles * ((N + block_n - 1) / block_n);
  p.idesc_int = make_idesc(2, 1, tile_m, block_n);                              // S32 accumulate, signed 8-bit operands
  p.idesc_fp = make_idesc(1, ep.dtype == QUIK_BF16 ? 1 : 0, tile_m, block_n);   // F32 accumulate, F16 / BF16 operands
  p.acc_shift = 0;
  // two issuing threads only for long sums: a thread can run at most one ring of stages ahead of the other, which must
  // stay well inside one tile for the per-tile barriers that both arrive on
  p.issuers = (g_issuers.load() >= 2 && p.int_kb >= 16) ? 2 : 1;
  p.l2_hint = g_l2_hint.load();

  CUtensorMap ta, tb, tfa, tfb;
  int rc;
  if ((rc = make_tmap(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, BLOCK_M)) != QUIK_OK) return rc;
  if ((rc = make_tmap(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, block_n / ctas)) != QUIK_OK) return rc;
  if (has_fp) {
    const CUtensorMapDataType fdt = ep.dtype == QUIK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if ((rc = make_tmap(&tfa, ep.fp_a, fdt, 2, M, ep.F, BLOCK_M)) != QUIK_OK) return rc;
    if ((rc = make_tmap(&tfb, ep.fp_b, fdt, 2, N, ep.F, block_n / ctas)) != QUIK_OK) return rc;
  } else {
    tfa = ta;
    tfb = tb;
  }
#define QUIK_LAUNCH_C(T, C)                                                                \
  do {                                                                                     \
    if (cap_n == 256) {                                                                    \
      return has_fp ? launch_t<T, 256, true, C>(ta, tb, tfa, tfb, p, st)                   \
                    : launch_t<T, 256, false, C>(ta, tb, tfa, tfb, p, st);                 \
    }                                                                                      \
    return has_fp ? launch_t<T, 128, true, C>(ta, tb, tfa, tfb, p, st)                     \
                  : launch_t<T, 128, false, C>(ta, tb, tfa, tfb, p, st);                   \
  } while (0)
#define QUIK_LAUNCH(T)                                                                     \
  do {                                                                                     \
    if (ctas == 2) QUIK_LAUNCH_C(T, 2);                                                    \
    QUIK_LAUNCH_C(T, 1);                                                                   \
  } while (0)
  if (ep.dtype == QUIK_BF16) QUIK_LAUNCH(__nv_bfloat16);
  QUIK_LAUNCH(__half);
#undef QUIK_LAUNCH_C
#undef QUIK_LAUNCH
}

}  // namespace quik
