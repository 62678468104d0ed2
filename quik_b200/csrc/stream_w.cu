// Weight-streaming fused layer for few tokens (M <= 128) on the tcgen05 tensor cores.
//
// With few tokens the layer (QUIK experiments/qlinear.py:122-145) is bound by reading the weights
// once from HBM, so the kernel is built around the weight stream and keeps the weights in their storage
// format: packed int4 (two codes per byte, low nibble first, QUIK include/int4.h:78-98) or int8.
//
// The product is computed transposed, out^T[n, m] = sum_k W[n, k] * Xq[m, k]: 128 weight rows are the
// M = 128 operand of tcgen05.mma, the tokens (zero-padded to NTOK = 16, 32, 64 or 128) its N operand, so one
// instruction consumes 128 x 32 weight codes.  Per CTA (one 128-row slab of W, one share of K):
//   warp 0      TMA producer: k-blocks of W (128 rows x 128 bytes, 128B swizzle) and of the token codes /
//               outlier values (NTOK rows x 128 bytes) into a ring of shared-memory stages.
//   warps 2-9   int4 only: each thread takes 64 packed bytes of "its" weight row from shared memory, widens
//               the 128 nibbles to signed bytes that carry 16 x the code (shift, two masks and two byte
//               permutes per 8 codes, natural k order) and writes them with tcgen05.st into a ring of TMEM
//               slots: the widened weights never touch shared or global memory.
//   warps 1,10  one lane each issues every second tcgen05.mma of a k-block (kind::i8 with A read from TMEM (int4)
//               or from the shared-memory stage (int8), B always from shared memory) into its own s32 accumulator;
//               warp 1 also issues kind::f16 for the outlier columns.  Accumulators (NTOK columns each) live in TMEM.
//   warps 2-9   epilogue: tcgen05.ld of the accumulators, split-K reduction, dequantize arithmetic of
//               QUIK src/asymmetric/asymmetric.cu:134-146, stores of out[m, n] (64 contiguous bytes per warp
//               and token).
// K is split over the CTAs of a thread-block cluster (1, 2, 4 or 8) when the layer has too few 128-row slabs
// to fill the GPU: the non-leading CTAs add their exact int32 partial sums into the leader's shared memory
// with red.shared::cluster (integer addition: the result does not depend on the order), the leader alone
// handles the outlier product, so the floating-point arithmetic has one fixed order.
// Every mbarrier wait is bounded; a wait that runs out sets the device status word, all roles leave their
// loops, the cluster barriers are still passed by every thread, TMEM is released and the kernel returns.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05_ptx.cuh"

namespace quik {
namespace {

constexpr int SW_THREADS = 352;                    // TMA warp, MMA warp, 8 widen/epilogue warps, second MMA warp
constexpr int SW_ISSUERS = 2;                      // one thread issues a small tcgen05.mma every ~60 ns at best: two share the work
constexpr int SW_ROWS = 128;                       // weight rows per CTA (the MMA's M)
constexpr int SW_W_BYTES = SW_ROWS * 128;          // one k-block of W: 128 bytes per row
constexpr int SW_A_COLS = 64;                      // 256 int8 codes per row = 64 32-bit columns
constexpr int SW_ACCS = 2;                         // one s32 accumulator per issuing thread, summed at the end
constexpr int SW_AUX_BYTES = 2048;

// Sizes that depend on NTOK, the MMA's N: the number of tokens (16, 32, 64 or 128; tokens beyond M read as zero).  A
// tcgen05.mma costs the same for every N up to 64, so up to 64 tokens ride along with the weight stream for free.
template <int NTOK> struct SwCfg {
  static constexpr int X_BYTES = NTOK * 128;                        // one 128-byte k-block of the token operand
  static constexpr int STAGE_BYTES = SW_W_BYTES + 2 * X_BYTES;      // int4: 256 codes of W need two token blocks
  static constexpr int CTAS_PER_SM = NTOK <= 32 ? 2 : 1;
  static constexpr int STAGES = (NTOK == 128 || NTOK == 32) ? 3 : 5;
  static constexpr int A_SLOTS = (NTOK == 128 || NTOK == 32) ? 2 : 3;   // TMEM ring of widened W k-blocks
  static constexpr int D_INT = A_SLOTS * SW_A_COLS;                 // TMEM column of the first s32 accumulator
  static constexpr int D_FP = D_INT + SW_ACCS * NTOK;               // ... of the f32 accumulator
  static constexpr int TMEM_COLS = NTOK <= 32 ? 256 : 512;          // NTOK 16, 32: two CTAs per SM share the 512 columns
  static constexpr int RED_BYTES = NTOK * SW_ROWS * 4;
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + RED_BYTES + SW_AUX_BYTES;
  static_assert(D_FP + NTOK <= TMEM_COLS, "TMEM plan");
  static_assert(SMEM <= (227 * 1024) / CTAS_PER_SM - 1024 * (CTAS_PER_SM - 1), "shared-memory plan");
};

struct StreamParams {
  int M, N;
  int nk, nf;                     // k-blocks of the integer part (128 bytes of a W row each) and of the outliers
  int splits;                     // CTAs that share one slab (= cluster size)
  int prefetch_blocks;            // k-blocks per CTA to prefetch into L2 before waiting for the predecessor
  uint32_t idesc_int, idesc_fp;
  const void *meta, *scale_col, *w_reduced, *bias;
  void *out;
  long long ldo;
  float shift_value;
  unsigned int *status;
  unsigned long long *dbg;        // optional cycle counters (16 per CTA), NULL = off
};

template <typename T, int BITS, int NTOK>
__global__ void __launch_bounds__(SW_THREADS, SwCfg<NTOK>::CTAS_PER_SM)
stream_w_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                const __grid_constant__ CUtensorMap tm_fw, const __grid_constant__ CUtensorMap tm_fx,
                const StreamParams p) {
  using Cfg = SwCfg<NTOK>;
  constexpr int SW_TOKENS = NTOK, SW_X_BYTES = Cfg::X_BYTES, SW_STAGE_BYTES = Cfg::STAGE_BYTES, SW_STAGES = Cfg::STAGES;
  constexpr int SW_A_SLOTS = Cfg::A_SLOTS, SW_D_INT = Cfg::D_INT, SW_D_FP = Cfg::D_FP, SW_TMEM_COLS = Cfg::TMEM_COLS;
  constexpr int SW_RED_BYTES = Cfg::RED_BYTES;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  int *red = reinterpret_cast<int *>(tiles + SW_STAGES * SW_STAGE_BYTES);     // [token][row], leader only
  unsigned char *aux = reinterpret_cast<unsigned char *>(red) + SW_RED_BYTES;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(aux);       // [STAGES] stage loaded
  uint64_t *empty_bar = full_bar + SW_STAGES;                   // [STAGES] stage consumed
  uint64_t *a_full = empty_bar + SW_STAGES;                     // [A_SLOTS] widened block written to TMEM
  uint64_t *a_empty = a_full + SW_A_SLOTS;                      // [A_SLOTS] ... consumed by the MMAs
  uint64_t *acc_full = a_empty + SW_A_SLOTS;                    // all MMAs of this CTA complete
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float *s_srow = reinterpret_cast<float *>(aux + 256);         // [NTOK] token scale
  float *s_zs = s_srow + SW_TOKENS;                             // [NTOK] zero + shift * scale

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool worker = warp >= 2 && warp < 10;                     // widening + epilogue warps
  const int issuer = warp == 1 ? 0 : (warp == 10 ? 1 : -1);       // MMA-issuing warps
  const int S = p.splits;
  const int rank = S > 1 ? (int)cluster_ctarank() : 0;
  const int n0 = ((int)blockIdx.x / S) * SW_ROWS;
  // Blocks of the slab in one sequence: outlier blocks first (so that they all fall to rank 0, which the
  // host guarantees by its choice of S), then the integer blocks; rank r takes an equal contiguous share.
  const int total = p.nk + p.nf;
  const int c0 = (int)(((long long)rank * total) / S), c1 = (int)(((long long)(rank + 1) * total) / S);
  const int nb = c1 - c0;
  const int n_fp = c0 < p.nf ? (c1 < p.nf ? c1 : p.nf) - c0 : 0;   // leading outlier blocks of this CTA
  const int n_int = nb - n_fp;
  const int kb_first = c0 + n_fp - p.nf;                           // first integer k-block

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < SW_STAGES; ++s) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), SW_ISSUERS + (BITS == 4 ? 8 : 0));   // MMA commits (+ the 8 widening warps)
    }
    for (int s = 0; s < SW_A_SLOTS; ++s) {
      mbar_init(smem_u32(a_full + s), 8);
      mbar_init(smem_u32(a_empty + s), SW_ISSUERS);
    }
    mbar_init(smem_u32(acc_full), SW_ISSUERS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_x);
    if (p.nf > 0) {
      prefetch_tmap(&tm_fw);
      prefetch_tmap(&tm_fx);
    }
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_slot), SW_TMEM_COLS);
    tmem_relinquish<1>();
  }
  if (warp == 0) {
    // ask L2 for this CTA's first weight tiles while the producer of the token codes may still run
    const int npre = nb < p.prefetch_blocks ? nb : p.prefetch_blocks;
    for (int i = lane; i < npre; i += 32) {
      if (i < n_fp) tma_prefetch_2d(&tm_fw, (c0 + i) * 64, n0);
      else tma_prefetch_2d(&tm_w, (kb_first + i - n_fp) * 128, n0);
    }
  }
  pdl_wait();      // first global access below
  if (worker) {
    const int te = threadIdx.x - 64;
    if (S > 1 && rank == 0)
      for (int i = te; i < SW_TOKENS * SW_ROWS; i += 256) red[i] = 0;
    if (te < SW_TOKENS) {
      float s = 0.f, z = 0.f;
      if (te < p.M) {
        s = Traits<T>::to_float(static_cast<const T *>(p.meta)[2 * te]);
        z = Traits<T>::to_float(static_cast<const T *>(p.meta)[2 * te + 1]);
      }
      s_srow[te] = s;
      s_zs[te] = fmaf(p.shift_value, s, z);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The leader's reduction buffer is zeroed: every thread arrives at the cluster barrier now (the TMA warp after
  // its first loads are under way); it is waited for before the first remote add.
  if (S > 1 && warp != 0) cluster_arrive();

  // epilogue vectors of this thread's weight row, fetched while the weights stream
  // (kept in storage format until the end: converting here would wait for the loads, which take microseconds
  // while the weight stream saturates HBM)
  T ep_scol = Traits<T>::from_float(0.f), ep_wred = ep_scol, ep_bias = ep_scol;
  if (worker && rank == 0) {
    const int n = n0 + (warp & 3) * 32 + lane;
    if (n < p.N) {
      ep_scol = static_cast<const T *>(p.scale_col)[n];
      ep_wred = static_cast<const T *>(p.w_reduced)[n];
      if (p.bias) ep_bias = static_cast<const T *>(p.bias)[n];
    }
  }

  if (warp == 0) {
    // ================= TMA producer =================
    auto issue = [&](int i, int stage) {
      const uint32_t fb = smem_u32(full_bar + stage);
      const uint32_t sw = smem_u32(tiles + stage * SW_STAGE_BYTES);
      if (i < n_fp) {
        const int fbk = c0 + i;
        mbar_expect_tx(fb, SW_W_BYTES + SW_X_BYTES);
        tma_load_2d<1>(sw, &tm_fw, fb, fbk * 64, n0);
        tma_load_2d<1>(sw + SW_W_BYTES, &tm_fx, fb, fbk * 64, 0);
      } else {
        const int kb = kb_first + (i - n_fp);
        if (BITS == 4) {
          mbar_expect_tx(fb, SW_W_BYTES + 2 * SW_X_BYTES);
          tma_load_2d<1>(sw, &tm_w, fb, kb * 128, n0);                     // 128 packed bytes = 256 codes
          tma_load_2d<1>(sw + SW_W_BYTES, &tm_x, fb, kb * 256, 0);
          tma_load_2d<1>(sw + SW_W_BYTES + SW_X_BYTES, &tm_x, fb, kb * 256 + 128, 0);
        } else {
          mbar_expect_tx(fb, SW_W_BYTES + SW_X_BYTES);
          tma_load_2d<1>(sw, &tm_w, fb, kb * 128, n0);
          tma_load_2d<1>(sw + SW_W_BYTES, &tm_x, fb, kb * 128, 0);
        }
      }
    };
    // One lane feeds the ring in order.  (Requesting the first STAGES blocks of every CTA at once was measured
    // slower: the burst completes as a whole, so the first block arrives later and nothing overlaps it.)
    int i = 0;
    if (lane == 0 && nb > 0) issue(i++, 0);
    __syncwarp();
    if (S > 1) cluster_arrive();
    if (lane == 0) {
      int stage = i % SW_STAGES;
      uint32_t phase = 0;
      for (; i < nb; ++i) {
        if (!mbar_wait(smem_u32(empty_bar + stage), phase ^ 1, abort_flag, p.status)) break;
        issue(i, stage);
        if (++stage == SW_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (issuer >= 0) {
    // ================= MMA issuers: issuer i takes every second instruction of a k-block, starting with i;
    // the two never share an accumulator (no order is defined between MMAs of different threads)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long w_full = 0, w_a = 0;
      const long long t_begin = clock64();
      for (int i = 0; i < nb && ok; ++i) {
        const long long t0 = clock64();
        if (!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag, p.status)) break;
        w_full += clock64() - t0;
        const uint32_t sw = smem_u32(tiles + stage * SW_STAGE_BYTES);
        const uint64_t dw = make_smem_desc(sw);
        const uint64_t dx = make_smem_desc(sw + SW_W_BYTES);
        if (i < n_fp) {
          tc_fence_after();
          if (issuer == 0)                 // one f32 accumulator, one fixed summation order
#pragma unroll
            for (int k = 0; k < 4; ++k)    // 16 values (32 bytes) of K per instruction
              mma_f16<1>(tmem_base + SW_D_FP, dw + 2 * k, dx + 2 * k, p.idesc_fp, (i > 0 || k > 0) ? 1u : 0u);
        } else if (BITS == 8) {
          tc_fence_after();
          const int ii = i - n_fp;
#pragma unroll
          for (int kk = 0; kk < 4 / SW_ISSUERS; ++kk) {
            const int k = kk * SW_ISSUERS + issuer;
            mma_i8<1>(tmem_base + SW_D_INT + SW_TOKENS * issuer, dw + 2 * k, dx + 2 * k, p.idesc_int, (ii > 0 || kk > 0) ? 1u : 0u);
          }
        } else {
          const int ii = i - n_fp, slot = ii % SW_A_SLOTS;
          const long long t1 = clock64();
          if (!mbar_wait(smem_u32(a_full + slot), (uint32_t)(ii / SW_A_SLOTS) & 1u, abort_flag, p.status)) break;
          w_a += clock64() - t1;
          tc_fence_after();
          const uint64_t dx1 = make_smem_desc(sw + SW_W_BYTES + SW_X_BYTES);
          const uint32_t a = tmem_base + slot * SW_A_COLS;
#pragma unroll
          for (int kk = 0; kk < 8 / SW_ISSUERS; ++kk) {      // 32 codes = 8 TMEM columns of A per instruction
            const int k = kk * SW_ISSUERS + issuer;
            mma_i8_ts<1>(tmem_base + SW_D_INT + SW_TOKENS * issuer, a + 8 * k, (k < 4 ? dx : dx1) + 2 * (k & 3), p.idesc_int,
                      (ii > 0 || kk > 0) ? 1u : 0u);
          }
          mma_commit<1>(smem_u32(a_empty + slot));
        }
        mma_commit<1>(smem_u32(empty_bar + stage));
        if (++stage == SW_STAGES) { stage = 0; phase ^= 1; }
      }
      mma_commit<1>(smem_u32(acc_full));     // also after an aborted loop: the epilogue wait ends either way
      if (p.dbg && issuer == 0) {
        unsigned long long *d = p.dbg + (size_t)blockIdx.x * 16;
        d[0] = (unsigned long long)(clock64() - t_begin);   // MMA thread: issue loop
        d[1] = (unsigned long long)w_full;                  // ... waiting for a loaded stage
        d[2] = (unsigned long long)w_a;                     // ... waiting for widened weights
        d[3] = (unsigned long long)nb;
      }
    }
  } else if (BITS == 4 && worker) {
    // ================= widening warps: packed W (shared memory) -> int8 W (TMEM) =================
    const int q = warp & 3;                   // TMEM lane quarter this warp may access
    const int h = (warp - 2) >> 2;            // which 64 bytes of the 128-byte packed row
    const int row = q * 32 + lane;
    int stage = 0;
    uint32_t phase = 0;
    long long c_full = 0, c_slot = 0, c_st = 0;
    const long long c_begin = clock64();
    for (int i = 0; i < nb; ++i) {
      const long long t0 = clock64();
      if (!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag, p.status)) break;
      c_full += clock64() - t0;
      if (i >= n_fp) {
        const int ii = i - n_fp, slot = ii % SW_A_SLOTS;
        const unsigned char *wrow = tiles + stage * SW_STAGE_BYTES + row * 128;
        uint4 pk[4];
#pragma unroll
        for (int c = 0; c < 4; ++c)      // 16-byte chunk c of the row sits at chunk position c ^ (row % 8)
          pk[c] = *reinterpret_cast<const uint4 *>(wrow + ((((4 * h + c) ^ (row & 7))) << 4));
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          widen8(pk[c].x, v[8 * c + 0], v[8 * c + 1]);
          widen8(pk[c].y, v[8 * c + 2], v[8 * c + 3]);
          widen8(pk[c].z, v[8 * c + 4], v[8 * c + 5]);
          widen8(pk[c].w, v[8 * c + 6], v[8 * c + 7]);
        }
        const long long t1 = clock64();
        if (!mbar_wait(smem_u32(a_empty + slot), ((uint32_t)(ii / SW_A_SLOTS) & 1u) ^ 1u, abort_flag, p.status)) break;
        const long long t2 = clock64();
        c_slot += t2 - t1;
        tc_fence_after();
        tmem_st32(tmem_base + ((uint32_t)(q * 32) << 16) + slot * SW_A_COLS + h * 32, v);
        tmem_st_wait();
        c_st += clock64() - t2;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(a_full + slot));
      } else {
        __syncwarp();
      }
      if (lane == 0) mbar_arrive(smem_u32(empty_bar + stage));   // this warp no longer reads the stage
      if (++stage == SW_STAGES) { stage = 0; phase ^= 1; }
    }
    if (p.dbg && warp == 2 && lane == 0) {
      unsigned long long *d = p.dbg + (size_t)blockIdx.x * 16;
      d[4] = (unsigned long long)(clock64() - c_begin);   // widening warp: whole loop
      d[5] = (unsigned long long)c_full;                  // ... waiting for a loaded stage
      d[6] = (unsigned long long)c_slot;                  // ... waiting for a free TMEM slot
      d[7] = (unsigned long long)c_st;                    // ... tcgen05.st until complete
    }
  }

  // ================= epilogue (warps 2-9) =================
  // Thread (q, lane, h) finishes weight row 32 q + lane for the tokens [h * NTOK / 2, (h + 1) * NTOK / 2), eight at a time.
  bool have = false;
  const int q = warp & 3, h = (warp - 2) >> 2;
  constexpr int CHUNKS = NTOK / 16;                  // 8-token chunks per thread
  const uint32_t lane_base = (uint32_t)(q * 32) << 16;
  auto load_int = [&](int tok0, uint32_t (&acc)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0;
    if (n_int > 0) {
      uint32_t part[8];
#pragma unroll
      for (int r = 0; r < SW_ACCS; ++r) {
        tmem_ld8(tmem_base + lane_base + SW_D_INT + SW_TOKENS * r + tok0, part);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += part[j];
      }
    }
  };
  __syncwarp();
  if (worker) {
    have = mbar_wait(smem_u32(acc_full), 0, abort_flag, p.status) && !*abort_flag;
    have = __all_sync(0xFFFFFFFFu, have);
    tc_fence_after();
  }
  if (S > 1) {
    cluster_wait();                                  // every CTA of the cluster has started; the buffer is zero
    if (worker && rank != 0 && have) {
      const uint32_t base = map_to_rank(smem_u32(red), 0);
#pragma unroll 1
      for (int c = 0; c < CHUNKS; ++c) {
        const int tok0 = h * (NTOK / 2) + 8 * c;
        uint32_t acc_i[8];
        load_int(tok0, acc_i);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          red_add_cluster(base + (uint32_t)(((tok0 + j) * SW_ROWS + q * 32 + lane) * 4), (int)acc_i[j]);
      }
    }
    cluster_arrive();
    cluster_wait();                                  // all partial sums have reached the leader
  }
  if (worker && rank == 0 && have) {
    const int n = n0 + q * 32 + lane;
    const float scol = Traits<T>::to_float(ep_scol), wred = Traits<T>::to_float(ep_wred), bias = Traits<T>::to_float(ep_bias);
    T *out = static_cast<T *>(p.out);
#pragma unroll 1
    for (int c = 0; c < CHUNKS; ++c) {
      const int tok0 = h * (NTOK / 2) + 8 * c;
      if (tok0 >= p.M) break;                        // warp-uniform
      uint32_t acc_i[8], acc_f[8];
      load_int(tok0, acc_i);                         // tcgen05.ld is warp-collective: all lanes, also rows beyond N
#pragma unroll
      for (int j = 0; j < 8; ++j) acc_f[j] = 0;
      if (n_fp > 0) {
        tmem_ld8(tmem_base + lane_base + SW_D_FP + tok0, acc_f);
        tmem_ld_wait();
      }
      if (n < p.N) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = tok0 + j;
          if (m < p.M) {
            int acc = (int)acc_i[j];
            if (S > 1) acc += red[m * SW_ROWS + q * 32 + lane];
            if (BITS == 4) acc >>= 4;                // the weights carried a factor 16; the quotient is exact
            const float add = fmaf(s_zs[m], wred, __uint_as_float(acc_f[j]) + bias);
            out[(size_t)m * p.ldo + n] = Traits<T>::from_float(fmaf((float)acc, s_srow[m] * scol, add));
          }
        }
      }
    }
  }

  // ---- teardown: every thread arrives here, also after an aborted wait
  if (*abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);   // let bulk copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, SW_TMEM_COLS);
  }
}

template <typename T, int BITS, int NTOK>
int launch_t(const CUtensorMap &tw, const CUtensorMap &tx, const CUtensorMap &tfw, const CUtensorMap &tfx,
             const StreamParams &p, int slabs, cudaStream_t st) {
  auto kern = stream_w_kernel<T, BITS, NTOK>;
  static PerDeviceSmem state;
  {
    const int rc = ensure_smem(state, kern, SwCfg<NTOK>::SMEM);
    if (rc != QUIK_OK) return rc;
  }
  LaunchCfg lc(dim3(slabs * p.splits), dim3(SW_THREADS), SwCfg<NTOK>::SMEM, st, p.splits);
  QUIK_CUDA_TRY(cudaLaunchKernelEx(&lc.cfg, kern, tw, tx, tfw, tfx, p));
  return check_launch("stream_w_kernel");
}

}  // namespace

// q: [M, K_int] int8 codes (one per byte); w: [N, K_int/2] packed int4 (bits == 4) or [N, K_int] int8.
int launch_stream_w(const void *q, const void *w, int bits, int M, int N, int K_int, const Epilogue &ep,
                    cudaStream_t st) {
  if (M == 0 || N == 0) return QUIK_OK;
  if (M > QUIK_STREAM_M_MAX) return QUIK_ERR_UNSUPPORTED;
  if (K_int <= 0 || K_int % (bits == 4 ? 32 : 16) != 0) return QUIK_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(w)) return QUIK_ERR_ALIGN;
  const bool has_fp = ep.fp_a != nullptr && ep.F > 0;
  if (has_fp && (ep.F % 8 != 0 || !aligned16(ep.fp_a) || !aligned16(ep.fp_b))) return QUIK_ERR_ALIGN;
  if (ep.meta == nullptr || ep.w_reduced == nullptr || ep.y != nullptr) return QUIK_ERR_UNSUPPORTED;

  const int ntok = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));          // the MMA's N
  const int ctas_per_sm = ntok <= 32 ? 2 : 1;
  const int stages = (ntok == 128 || ntok == 32) ? 3 : 5;
  StreamParams p{};
  p.M = M;
  p.N = N;
  const int w_row_bytes = bits == 4 ? K_int / 2 : K_int;
  p.nk = (w_row_bytes + 127) / 128;
  p.nf = has_fp ? (ep.F + 63) / 64 : 0;
  const int slabs = (N + SW_ROWS - 1) / SW_ROWS;
  // Split K over a cluster while all CTAs still fit on the GPU at once, every CTA keeps at least two k-blocks and
  // the outlier blocks all fall to the first CTA.
  const int total = p.nk + p.nf, slots = ctas_per_sm * num_sms();
  int splits = 1;
  while (splits < 8 && slabs * splits * 2 <= slots && total / (splits * 2) >= (p.nf > 2 ? p.nf : 2)) splits *= 2;
  p.splits = splits;
  p.prefetch_blocks = stages;      // deeper prefetch was measured slower: the requests delay the first real loads
  p.idesc_int = make_idesc(2, 1, SW_ROWS, ntok);
  p.idesc_fp = make_idesc(1, ep.dtype == QUIK_BF16 ? 1 : 0, SW_ROWS, ntok);
  p.meta = ep.meta;
  p.scale_col = ep.scale_col;
  p.w_reduced = ep.w_reduced;
  p.bias = ep.bias;
  p.out = ep.out;
  p.ldo = ep.ldo > 0 ? ep.ldo : N;
  p.shift_value = ep.shift_value;
  p.dbg = get_debug_counters();
  p.status = device_status_word();
  if (p.status == nullptr) return QUIK_ERR_CUDA;

  CUtensorMap tw, tx, tfw, tfx;
  int rc;
  if ((rc = make_tmap(&tw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, w_row_bytes, SW_ROWS)) != QUIK_OK) return rc;
  if ((rc = make_tmap(&tx, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K_int, ntok)) != QUIK_OK) return rc;
  if (has_fp) {
    const CUtensorMapDataType fdt = ep.dtype == QUIK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if ((rc = make_tmap(&tfw, ep.fp_b, fdt, 2, N, ep.F, SW_ROWS)) != QUIK_OK) return rc;
    if ((rc = make_tmap(&tfx, ep.fp_a, fdt, 2, M, ep.F, ntok)) != QUIK_OK) return rc;
  } else {
    tfw = tw;
    tfx = tx;
  }
#define QUIK_SW(T, B)                                                                    \
  do {                                                                                   \
    if (ntok == 16) return launch_t<T, B, 16>(tw, tx, tfw, tfx, p, slabs, st);           \
    if (ntok == 32) return launch_t<T, B, 32>(tw, tx, tfw, tfx, p, slabs, st);           \
    if (ntok == 64) return launch_t<T, B, 64>(tw, tx, tfw, tfx, p, slabs, st);           \
    return launch_t<T, B, 128>(tw, tx, tfw, tfx, p, slabs, st);                          \
  } while (0)
  if (ep.dtype == QUIK_BF16) {
    if (bits == 4) QUIK_SW(__nv_bfloat16, 4);
    QUIK_SW(__nv_bfloat16, 8);
  }
  if (bits == 4) QUIK_SW(__half, 4);
  QUIK_SW(__half, 8);
#undef QUIK_SW
}

}  // namespace quik
