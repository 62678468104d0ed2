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
#include "tcgen05_ptx.cuh"

namespace quik {

__device__ unsigned int g_device_status = 0;

namespace {

constexpr int BLOCK_M = 128;
constexpr int STAGE_K_BYTES = 128;           // one 128B-swizzle row of K per stage
constexpr int NUM_THREADS = 320;              // TMA warp + MMA warp + 8 epilogue warps
constexpr int NUM_EPI_THREADS = 256;
// Process-wide tuning knobs (quik_config_set): plain words, meant to be set once before the layers run; a
// launch reads each of them once.
std::atomic<int> g_tile_n{0};                                 // 0 = choose by shape, else a multiple of 16 in [32, 256]
std::atomic<int> g_cta_pair{0};                               // 0 = by shape, 1 = never, 2 = always
std::atomic<unsigned long long *> g_dbg{nullptr};             // diagnostic counters (device memory), off by default

// Shared-memory plan after the 1024-byte aligned ring of stages: 256 bytes of barriers etc. and the
// per-warp epilogue vectors (rounded to 1024 together), then one output staging chunk per epilogue
// warp (32 rows x 64 bytes).
constexpr int EPI_BUF_BYTES = 32 * 64;
constexpr int AUX_BYTES(int cap_n) { return ((256 + 8 * 3 * (cap_n / 2) * 4) + 1023) / 1024 * 1024; }
constexpr int stage_bytes(int cap_n, int ctas) { return (BLOCK_M + cap_n / ctas) * STAGE_K_BYTES; }
constexpr int SMEM_LIMIT = 227 * 1024;
// Ring depth: as many stages as fit (at most 8).
constexpr int num_stages(int cap_n, int ctas) {
  const int n = (SMEM_LIMIT - 1024 - AUX_BYTES(cap_n) - 8 * EPI_BUF_BYTES) / stage_bytes(cap_n, ctas);
  return n > 8 ? 8 : n;
}

struct GemmParams {
  int M, N;
  int block_n;                    // tile width: multiple of 16, <= CAP_N
  int split_n;                    // columns of a tile that the first four epilogue warps take (multiple of 32 or block_n)
  int num_m_tiles, num_tiles;
  int int_kb, fp_kb;              // k-blocks per tile: integer (128 B each) and outlier (64 elems)
  uint32_t idesc_int, idesc_fp;   // tcgen05 instruction descriptors
  int mode;                       // 0: int32 C, 1: dequantize
  int32_t *C;
  void *out;
  long long ldo;                  // row pitch of `out` in elements (>= N)
  const void *row_scale;          // element (row * row_stride)
  const void *row_zero;           // may be NULL
  int row_stride;
  const void *scale_col, *w_reduced, *bias, *y;
  float shift_value;
  int vec_out;                    // 16-byte stores allowed (pitch and base aligned)
  int vec_y;
  unsigned long long *dbg;         // optional per-CTA cycle counters (16 per CTA), NULL = off
};

// mbarrier / TMA / TMEM / tcgen05 wrappers: tcgen05_ptx.cuh
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  return mbar_wait(bar, parity, abort_flag, &g_device_status);
}

template <typename T> __device__ __forceinline__ float ldf(const void *p, size_t i) {
  return Traits<T>::to_float(static_cast<const T *>(p)[i]);
}

// 32 consecutive values of type T: 16-byte vector access when `vec`, scalar with a column guard
// otherwise.
template <typename T>
__device__ __forceinline__ void load_row32(const T *src, bool vec, int ncols_left, T (&v)[32]) {
  if (vec) {
#pragma unroll
    for (int j = 0; j < 4; ++j) reinterpret_cast<uint4 *>(v)[j] = reinterpret_cast<const uint4 *>(src)[j];
  } else {
    for (int j = 0; j < 32; ++j) v[j] = (j < ncols_left) ? src[j] : Traits<T>::from_float(0.f);
  }
}
// eight fp32 values -> eight values of type T in one 16-byte word
template <typename T>
__device__ __forceinline__ uint4 pack8(const float *o) {
  uint4 pk;
  T *pe = reinterpret_cast<T *>(&pk);
#pragma unroll
  for (int e = 0; e < 8; ++e) pe[e] = Traits<T>::from_float(o[e]);
  return pk;
}
template <typename T>
__device__ __forceinline__ void store_row32(T *dst, bool vec, int ncols_left, const float (&o)[32]) {
  if (vec) {
#pragma unroll
    for (int j = 0; j < 4; ++j) reinterpret_cast<uint4 *>(dst)[j] = pack8<T>(o + 8 * j);
  } else {
    for (int j = 0; j < 32; ++j)
      if (j < ncols_left) dst[j] = Traits<T>::from_float(o[j]);
  }
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
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(fp_drained + 2);
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
      mbar_init(smem_u32(empty_bar + s), 1);
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
      // one k-block range of one product of tile j into the ring
      auto feed = [&](int j, bool fp, int kb0, int kb1) {
        const int tile = unit + j * num_units;
        const int m0 = (tile % p.num_m_tiles) * TILE_M + rank * BLOCK_M;      // this CTA's rows of A
        const int n0 = (tile / p.num_m_tiles) * bn + rank * b_rows;           // this CTA's rows of B
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
          if (!mbar_wait(smem_u32(empty_bar + stage), phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t fb = smem_u32(full_bar + stage);
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          if (rank == 0) mbar_expect_tx(fb, stage_tx);
          if (fp) {
            tma_load_2d<CTAS>(sa, &tmap_fa, fb, kb * 64, m0);
            tma_load_2d<CTAS>(sa + A_BYTES, &tmap_fb, fb, kb * 64, n0);
          } else {
            tma_load_2d<CTAS>(sa, &tmap_a, fb, kb * STAGE_K_BYTES, m0);
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
  } else if (warp == 1) {
    // ================= MMA issuer (pair leader only) =================
    if (lane == 0 && rank == 0) {
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
          if (kb == 0) {
            // the region must be free: after the previous tile's epilogue (outlier product, or
            // integer product of an outlier-free layer), or after this tile's drain
            const bool after_drain = HAS_FP && !fp;
            const uint32_t bar = smem_u32((after_drain ? fp_drained : acc_empty) + r);
            const long long t0 = clock64();
            if (!mbar_wait(bar, after_drain ? use_parity : (use_parity ^ 1u), abort_flag)) { ok = false; break; }
            w_region += clock64() - t0;
            tc_fence_after();
          }
          const long long t1 = clock64();
          if (!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag)) { ok = false; break; }
          w_full += clock64() - t1;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < STAGE_K_BYTES / 32; ++k) {
            // +32 bytes of K inside the swizzled row = +2 in the 16-byte start-address field
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            if (fp) mma_f16<CTAS>(d, da + 2 * k, db + 2 * k, p.idesc_fp, accumulate);
            else mma_i8<CTAS>(d, da + 2 * k, db + 2 * k, p.idesc_int, accumulate);
          }
          mma_commit<CTAS>(smem_u32(empty_bar + stage));    // stage reusable once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (fp && kb == p.fp_kb - 1) mma_commit<CTAS>(smem_u32(fp_full + r));
          if (!fp && kb == p.int_kb - 1) mma_commit<CTAS>(smem_u32(acc_full + r));
        }
      };
      if (HAS_FP && n_local > 0) issue(0, true, 0, p.fp_kb);
      for (int j = 0; j < n_local && ok; ++j) {
        issue(j, false, 0, int_half);
        if (HAS_FP && j + 1 < n_local) issue(j + 1, true, 0, p.fp_kb);
        issue(j, false, int_half, p.int_kb);
      }
      if (p.dbg) {
        unsigned long long *d = p.dbg + (size_t)blockIdx.x * 16;
        d[0] = (unsigned long long)(clock64() - t_begin);   // MMA thread: issue loop
        d[1] = (unsigned long long)w_region;                // ... waiting for a free accumulator region
        d[2] = (unsigned long long)w_full;                  // ... waiting for operands
        d[3] = (unsigned long long)n_local;
      }
    }
  } else {
    // ================= epilogue (warps 2..9) =================
    // Warp (sub, half) owns rows [32*sub, 32*sub+32) of the tile and the columns [cb, cb + cn): the first
    // split_n columns for half 0, the rest for half 1.  It walks them 32 at a time; the last step of a range
    // whose length is not a multiple of 32 holds 16 valid columns (`valid` below), the rest is ignored.
    const int e = warp - 2;
    const int sub = warp & 3;                 // TMEM lane quarter this warp may read
    const int half = e >> 2;                  // which part of the tile's columns
    const int cb = half ? p.split_n : 0;
    const int cn = half ? bn - p.split_n : p.split_n;
    const int cn32 = (cn + 31) & ~31;
    float *s_scol = s_vec + e * 3 * HALF_CAP;
    float *s_wred = s_scol + HALF_CAP;
    float *s_bias = s_wred + HALF_CAP;
    unsigned char *s_stage = s_out + e * EPI_BUF_BYTES;   // staging of one 32 x 32 output chunk
    bool ok = true;
    long long e_wait_fp = 0, e_wait_acc = 0, e_drain = 0, e_finish = 0;

    // Where the outlier product of (this warp, tile) is parked inside the tile's place in `out`.
    // Every full 32 x 32 chunk is parked inside its own 32-row x 64-byte block (so the final store of one
    // chunk never touches the parked data of another), but permuted: the jj-th 16-byte piece of lane
    // L goes to row 8*jj + L/4, piece L%4 of the block, so one warp instruction writes 8 rows x 64
    // contiguous bytes (whole sectors) instead of 32 rows x 16 bytes.  The same lane reads its pieces
    // back from the same addresses; nobody else looks at them.  Chunks that touch the matrix edge or hold
    // fewer than 32 valid columns keep the plain row-per-lane layout with guards.
    auto parked_piece = [&](T *sub_base, int c0, int jj) -> uint4 * {   // sub_base = &out[first row of warp][n0]
      return reinterpret_cast<uint4 *>(sub_base + (size_t)(8 * jj + (lane >> 2)) * p.ldo + c0) + (lane & 3);
    };

    // park T(outlier product + bias) of tile j in `out`
    auto drain = [&](int j) {
      const int tile = unit + j * num_units;
      const int m0 = (tile % p.num_m_tiles) * TILE_M + rank * BLOCK_M + sub * 32;   // first row of this warp
      const int n0 = (tile / p.num_m_tiles) * bn + cb;
      const int lim = min(p.N - n0, cn);       // valid columns from n0 on (<= 0: none)
      const int r = j & 1;
      __syncwarp();
      for (int c = lane; c < cn32; c += 32)
        s_bias[c] = (c < lim && p.bias) ? ldf<T>(p.bias, n0 + c) : 0.f;
      __syncwarp();
      const long long tw = clock64();
      const bool ready = mbar_wait(smem_u32(fp_full + r), (uint32_t)(j >> 1) & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) { ok = false; return; }
      const long long tw1 = clock64();
      e_wait_fp += tw1 - tw;
      tc_fence_after();
      const int row = m0 + lane;
      const bool rows_in = m0 + 32 <= p.M;
      T *sub_base = static_cast<T *>(p.out) + (size_t)m0 * p.ldo + n0;
      const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + r * CAP_N + cb;
#pragma unroll 1
      for (int c0 = 0; c0 < cn; c0 += 32) {
        uint32_t f[32];
        float o[32];
        __syncwarp();                          // tcgen05.ld is warp-collective
        tmem_ld32(taddr + c0, f);
        tmem_ld_wait();
        const int valid = lim - c0;            // warp-uniform
        if (valid <= 0) continue;
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(f[i]) + s_bias[c0 + i];
        if (p.vec_out && rows_in && valid >= 32) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) *parked_piece(sub_base, c0, jj) = pack8<T>(o + 8 * jj);
        } else if (row < p.M) {
          T *dst = static_cast<T *>(p.out) + (size_t)row * p.ldo + n0 + c0;
          if (p.vec_out) {                     // valid is a multiple of 8 here
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
              if (8 * jj < valid) reinterpret_cast<uint4 *>(dst)[jj] = pack8<T>(o + 8 * jj);
          } else {
            store_row32<T>(dst, false, valid, o);
          }
        }
      }
      tc_fence_before();
      if (CTAS == 1) mbar_arrive(smem_u32(fp_drained + r));
      else mbar_arrive_leader(smem_u32(fp_drained + r));
      e_drain += clock64() - tw1;
    };

    auto finish = [&](int j) {
      const int tile = unit + j * num_units;
      const int m0 = (tile % p.num_m_tiles) * TILE_M + rank * BLOCK_M + sub * 32;   // first row of this warp
      const int n0 = (tile / p.num_m_tiles) * bn + cb;
      const int lim = min(p.N - n0, cn);
      const int r = j & 1;
      if (p.mode == 1) {
        __syncwarp();                         // previous readers of the vectors are done
        for (int c = lane; c < cn32; c += 32) {
          const int col = n0 + c;
          const bool in = c < lim;
          s_scol[c] = in ? ldf<T>(p.scale_col, col) : 0.f;
          s_wred[c] = (in && p.w_reduced) ? ldf<T>(p.w_reduced, col) : 0.f;
          s_bias[c] = (in && p.bias && !HAS_FP) ? ldf<T>(p.bias, col) : 0.f;   // with outliers the drain added it
        }
        __syncwarp();
      }
      const int row = m0 + lane;
      const bool row_ok = row < p.M;
      const bool rows_in = m0 + 32 <= p.M;
      T *sub_base = static_cast<T *>(p.out) + (size_t)m0 * p.ldo + n0;
      const T *my_row = static_cast<const T *>(p.out) + (size_t)row * p.ldo + n0;
      // The parked outlier product of the first 32 columns is fetched before waiting for the integer
      // product, the following ones one step ahead, so their L2 latency stays off the critical path.
      uint4 pk_next[4];
      auto prefetch_parked = [&](int c0) {
        if (!HAS_FP || p.mode != 1 || !p.vec_out) return;
        const int valid = lim - c0;
        if (rows_in && valid >= 32) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) pk_next[jj] = *parked_piece(sub_base, c0, jj);
        } else if (row_ok) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            if (8 * jj < valid) pk_next[jj] = reinterpret_cast<const uint4 *>(my_row + c0)[jj];
        }
      };
      prefetch_parked(0);
      const long long tw = clock64();
      const bool ready = mbar_wait(smem_u32(acc_full + r), (uint32_t)(j >> 1) & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) { ok = false; return; }
      const long long tw1 = clock64();
      e_wait_acc += tw1 - tw;
      tc_fence_after();
      float srow = 0.f, zs = 0.f;
      if (p.mode == 1 && row_ok) {
        srow = ldf<T>(p.row_scale, (size_t)row * p.row_stride);
        const float zrow = p.row_zero ? ldf<T>(p.row_zero, (size_t)row * p.row_stride) : 0.f;
        zs = fmaf(p.shift_value, srow, zrow);
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + r * CAP_N + cb;
#pragma unroll 1
      for (int c0 = 0; c0 < cn; c0 += 32) {
        uint32_t v[32];
        uint4 pk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pk[i] = pk_next[i];
        __syncwarp();                          // tcgen05.ld is warp-collective: reconverge first
        tmem_ld32(taddr + c0, v);
        if (c0 + 32 < cn) prefetch_parked(c0 + 32);
        tmem_ld_wait();
        const int valid = lim - c0;            // warp-uniform
        if (valid <= 0) continue;
        const int col0 = n0 + c0;
        const size_t off = (size_t)row * p.N + col0;
        if (p.mode == 0) {
          if (!row_ok) continue;
          if (p.vec_out) {                     // valid is a multiple of 4 here
            int4 *dst = reinterpret_cast<int4 *>(p.C + off);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (4 * i < valid) dst[i] = make_int4((int)v[4 * i], (int)v[4 * i + 1], (int)v[4 * i + 2], (int)v[4 * i + 3]);
          } else {
            for (int i = 0; i < 32; ++i)
              if (i < valid) p.C[off + i] = (int)v[i];
          }
          continue;
        }
        float o[32];   // addend first, result later
        if (HAS_FP) {
          if (p.vec_out) {
            const T *pe = reinterpret_cast<const T *>(pk);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = Traits<T>::to_float(pe[i]);   // pieces beyond `valid` are never stored
          } else {
            for (int i = 0; i < 32; ++i)
              o[i] = (row_ok && i < valid) ? Traits<T>::to_float(my_row[c0 + i]) : 0.f;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = s_bias[c0 + i];
        }
        if (p.y != nullptr && row_ok) {
          T yv[32];
          load_row32<T>(static_cast<const T *>(p.y) + off, valid >= 32 && p.vec_y, valid, yv);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] += Traits<T>::to_float(yv[i]);
        }
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 sc4 = reinterpret_cast<const float4 *>(s_scol + c0)[i4];
          const float4 wr4 = reinterpret_cast<const float4 *>(s_wred + c0)[i4];
          const float sc[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
          const float wr[4] = {wr4.x, wr4.y, wr4.z, wr4.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int i = 4 * i4 + q;
            // out = acc * (s_row * s_col) + ((zero + shift * s_row) * w_red + addend), fused multiply-adds
            o[i] = fmaf((float)(int)v[i], srow * sc[q], fmaf(zs, wr[q], o[i]));
          }
        }
        if (p.vec_out) {
          // Transpose through shared memory so that one warp instruction stores 8 rows x 64 contiguous
          // bytes (whole sectors) instead of 32 rows x 16 bytes: lane i writes its row as four 16-byte
          // pieces (swizzled against bank conflicts), lane L then stores piece L%4 of rows 8k + L/4.
          __syncwarp();                        // the previous chunk has been read out of the buffer
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            *reinterpret_cast<uint4 *>(s_stage + lane * 64 + ((jj ^ ((lane >> 1) & 3)) << 4)) = pack8<T>(o + 8 * jj);
          __syncwarp();
          const int pc = lane & 3;
          const bool col_ok = 8 * pc + 8 <= valid;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int rr = 8 * k + (lane >> 2);
            const uint4 piece = *reinterpret_cast<const uint4 *>(s_stage + rr * 64 + ((pc ^ ((rr >> 1) & 3)) << 4));
            if (col_ok && m0 + rr < p.M)
              *(reinterpret_cast<uint4 *>(static_cast<T *>(p.out) + (size_t)(m0 + rr) * p.ldo + col0) + pc) = piece;
          }
        } else if (row_ok) {
          store_row32<T>(static_cast<T *>(p.out) + (size_t)row * p.ldo + col0, false, valid, o);
        }
      }
      tc_fence_before();
      if (CTAS == 1) mbar_arrive(smem_u32(acc_empty + r));
      else mbar_arrive_leader(smem_u32(acc_empty + r));
      e_finish += clock64() - tw1;
    };

    if (HAS_FP && n_local > 0) drain(0);
    for (int j = 0; j < n_local && ok; ++j) {
      if (HAS_FP && j + 1 < n_local) drain(j + 1);
      if (!ok) break;
      finish(j);
    }
    if (p.dbg && warp == 2 && lane == 0) {
      unsigned long long *d = p.dbg + (size_t)blockIdx.x * 16;
      d[4] = (unsigned long long)e_wait_fp;     // epilogue warp: waiting for an outlier product
      d[5] = (unsigned long long)e_wait_acc;    // ... waiting for an integer product
      d[6] = (unsigned long long)e_drain;       // ... parking outlier products
      d[7] = (unsigned long long)e_finish;      // ... final epilogues
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
// A launch is a number of waves of equally sized tiles over the resident units (CTAs or CTA pairs).  The time
// of a tile is set by the slower of the tensor pipe (2 * block_n cycles per CTA and 128-byte k-block) and the
// operand feed ((128 + block_n / ctas) rows of 128 bytes per CTA and k-block at kFeedBytesPerClk), so the
// widest pair tile is the cheapest per multiply-accumulate, but a last wave that is mostly empty can cost more
// than narrower tiles that fill their waves.  The model picks the (pair or single, block_n) with the smallest
// waves x tile time; kFeedBytesPerClk and kTileFixedClk are fitted to measured sweeps over the Llama-2 shapes.
constexpr double kFeedBytesPerClk = 43.0;
constexpr double kTileFixedClk = 1500.0;

double tile_cost(int M, int N, int kblocks, int ctas, int bn, int units) {
  const int tile_m = BLOCK_M * ctas;
  const long long tiles = (long long)((M + tile_m - 1) / tile_m) * ((N + bn - 1) / bn);
  const long long waves = (tiles + units - 1) / units;
  const double mma = 2.0 * bn;
  const double feed = (BLOCK_M + bn / ctas) * (double)STAGE_K_BYTES / kFeedBytesPerClk;
  return (double)waves * (kblocks * (mma > feed ? mma : feed) + kTileFixedClk);
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

  p.M = M;
  p.N = N;
  p.block_n = block_n;
  p.split_n = ((block_n / 2 + 31) & ~31) < block_n ? ((block_n / 2 + 31) & ~31) : block_n;
  p.num_m_tiles = m_tiles;
  p.num_tiles = m_tiles * ((N + block_n - 1) / block_n);
  p.idesc_int = make_idesc(2, 1, tile_m, block_n);                              // S32 accumulate, signed 8-bit operands
  p.idesc_fp = make_idesc(1, ep.dtype == QUIK_BF16 ? 1 : 0, tile_m, block_n);   // F32 accumulate, F16 / BF16 operands
  p.mode = ep.mode;
  p.C = ep.C;
  p.out = ep.out;
  p.ldo = ep.ldo > 0 ? ep.ldo : N;
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
  else p.vec_out = (N % 8 == 0) && (p.ldo % 8 == 0) && aligned16(ep.out);
  p.vec_y = ep.y && (N % 8 == 0) && aligned16(ep.y);
  p.dbg = g_dbg.load();

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
