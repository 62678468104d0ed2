// Weight-streaming fused layer for few tokens (M <= 16): TMA-fed shared-memory ring in front of mma.sync.
//
// Same problem and same outer structure as stream_w.cu (one 128-row slab of W per CTA, K split over a
// thread-block cluster, outlier blocks to the cluster's leader, exact split-K reduction with red.shared::cluster),
// but the consumers are the legacy warp-level tensor instructions, which accept this skinny shape (16 tokens x 8
// weight rows x 32 codes per instruction) at a higher rate than tcgen05 accepts 128 x 16 x 32 ones, and which
// take the packed int4 weights after a three-instruction nibble split instead of a trip through TMEM:
//   warp 0      TMA producer: per k-block 128 rows x 128 bytes of W (packed int4: 256 codes, int8: 128 codes,
//               outliers: 64 values) and 16 rows x 128 bytes of the token operand in the same format, 128B swizzle.
//   warps 1-8   warp (rg, kh) owns weight rows [32 rg, 32 rg + 32) and 16-byte chunks [4 kh, 4 kh + 4) of every
//               128-byte row: ldmatrix.x4 (conflict free under the swizzle) hands lane (g, t) word t of row g of
//               each chunk, which is exactly an mma.sync operand register.  int4: each packed word is split into the
//               word of its even codes and the word of its odd codes (bytes = 16 x code), the low and high k halves
//               of one m16n8k32.s8; the same split on the token side keeps the pairing, and the factor 256 is shifted
//               out of the exact sum.  int8 / outliers: two chunks are the two k halves of one instruction.
//               A warp releases a stage as soon as its operands are in registers.
//   end         the two k-half warps of a row group write their int32 and fp32 partial sums into separate tiles in
//               drained stages of the ring; the non-leading CTAs add theirs into the leader's tile
//               (red.shared::cluster; integer addition, order-free); 256 threads of the leader add the tiles (the
//               outlier halves in fixed order), apply the dequantize arithmetic of
//               QUIK src/asymmetric/asymmetric.cu:134-146 and store out[m, n].
// Every mbarrier wait is bounded (device status word, see tcgen05_ptx.cuh).
#include <cuda.h>

#include "common.cuh"
#include "tcgen05_ptx.cuh"

namespace quik {
namespace {

constexpr int SM_THREADS2 = 288;                    // TMA warp + 8 consumer warps
constexpr int SM_ROWS = 128;                        // weight rows per CTA
constexpr int SM_TOKENS = 16;
constexpr int SM_STAGES = 5;                        // ring depth with two CTAs per SM
constexpr int SM_STAGES_DEEP = 11;                  // ... with one CTA per SM (the grid has no more CTAs than SMs)
constexpr int SM_W_BYTES = SM_ROWS * 128;
constexpr int SM_X_BYTES = SM_TOKENS * 128;
constexpr int SM_STAGE_BYTES = SM_W_BYTES + SM_X_BYTES;
constexpr int SM_RED_BYTES = SM_TOKENS * SM_ROWS * 4;
constexpr int SM_AUX_BYTES = 1024;
constexpr size_t sm_smem(int stages) { return 1024 + (size_t)stages * SM_STAGE_BYTES + SM_RED_BYTES + SM_AUX_BYTES; }
static_assert(sm_smem(SM_STAGES_DEEP) <= 227 * 1024 && 2 * sm_smem(SM_STAGES) <= 227 * 1024, "shared-memory plan");
static_assert(2 * SM_STAGES_DEEP * 8 + 4 <= 256, "barriers and the abort flag sit in front of the token scales");

struct MmaStreamParams {
  int M, N;
  int nk, nf;                     // k-blocks (128 bytes of a W row each): integer part, outliers
  int splits;                     // CTAs that share one slab (= cluster size)
  int stages;                     // ring depth (SM_STAGES or SM_STAGES_DEEP)
  int prefetch_blocks;            // k-blocks per CTA to prefetch into L2 before waiting for the predecessor
  int preload;                    // 1: the weight tiles of the first ring fill are loaded before that wait too
  const void *meta, *scale_col, *w_reduced, *bias;
  void *out;
  long long ldo;
  float shift_value;
  unsigned int *status;
  unsigned long long *dbg;        // diagnostics (quik_debug_counters): 16 words per CTA, or nullptr
};

// four 8-row x 16-byte matrices; lanes 8i..8i+7 give the row addresses of matrix i; lane (g, t) receives word t of
// row g of each matrix
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ void mma_fp16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  if (Traits<T>::kIsHalf)
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// eight packed int4 codes -> word of the even codes and word of the odd codes, each byte = 16 x code
__device__ __forceinline__ void split_nibbles(uint32_t w, uint32_t &even16, uint32_t &odd16) {
  even16 = (w << 4) & 0xF0F0F0F0u;
  odd16 = w & 0xF0F0F0F0u;
}

template <typename T, int BITS>
__global__ void __launch_bounds__(SM_THREADS2, 2)
stream_w_mma_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    const __grid_constant__ CUtensorMap tm_fw, const __grid_constant__ CUtensorMap tm_fx,
                    const MmaStreamParams p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  const int STAGES = p.stages;
  int *red = reinterpret_cast<int *>(tiles + STAGES * SM_STAGE_BYTES);     // [token][row] int32 sums of this CTA
  unsigned char *aux = reinterpret_cast<unsigned char *>(red) + SM_RED_BYTES;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(aux);       // [STAGES] stage loaded
  uint64_t *empty_bar = full_bar + SM_STAGES_DEEP;                 // [STAGES] stage read by all 8 consumer warps
  volatile int *abort_flag = reinterpret_cast<volatile int *>(empty_bar + SM_STAGES_DEEP);
  float *s_srow = reinterpret_cast<float *>(aux + 256);         // [16] token scale
  float *s_zs = s_srow + SM_TOKENS;                             // [16] zero + shift * scale
  float *fp_part = reinterpret_cast<float *>(tiles);            // [token][row] outlier sums of the kh = 0 warps; reuses
                                                                // stage 0 after the ring has drained

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.splits;
  const int rank = S > 1 ? (int)cluster_ctarank() : 0;
  const int n0 = ((int)blockIdx.x / S) * SM_ROWS;
  // Blocks of the slab in one sequence: outlier blocks first (they all fall to rank 0, which the host guarantees by
  // its choice of S), then the integer blocks; rank r takes an equal contiguous share.
  const int total = p.nk + p.nf;
  const int c0 = (int)(((long long)rank * total) / S), c1 = (int)(((long long)(rank + 1) * total) / S);
  const int nb = c1 - c0;
  const int n_fp = c0 < p.nf ? (c1 < p.nf ? c1 : p.nf) - c0 : 0;
  const int kb_first = c0 + n_fp - p.nf;

  long long dbg_t[6] = {clock64(), 0, 0, 0, 0, 0};      // written out by thread 32 when diagnostics are on
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), 8);
    }
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
  // The weights are constants of the layer: nothing the predecessor writes.  Before waiting for it (it produces the
  // token codes) the producer thread fills the ring with the weight tiles of its first blocks and the warp asks L2
  // for the tiles after those, so that the weight stream from HBM runs while the predecessor does; the token tiles of
  // the same stages follow after the wait and complete the stages' byte counts.
  const int pre = p.preload ? (nb < STAGES ? nb : STAGES) : 0;
  if (threadIdx.x == 0) {
    const uint64_t once = l2_policy_evict_first();      // the weights are read once
    for (int i = 0; i < pre; ++i) {
      const uint32_t fb = smem_u32(full_bar + i);
      const uint32_t sw = smem_u32(tiles + i * SM_STAGE_BYTES);
      mbar_expect_tx(fb, SM_STAGE_BYTES);
      if (i < n_fp) tma_load_2d_hint(sw, &tm_fw, fb, (c0 + i) * 64, n0, once);
      else tma_load_2d_hint(sw, &tm_w, fb, (kb_first + i - n_fp) * 128, n0, once);
    }
  }
  if (warp == 0) {
    __syncwarp();
    const int first = pre, last = nb < pre + p.prefetch_blocks ? nb : pre + p.prefetch_blocks;
    for (int i = first + lane; i < last; i += 32) {
      if (i < n_fp) tma_prefetch_2d(&tm_fw, (c0 + i) * 64, n0);
      else tma_prefetch_2d(&tm_w, (kb_first + i - n_fp) * 128, n0);
    }
  }
  pdl_wait();      // first global access below
  dbg_t[1] = clock64();
  if (threadIdx.x == 0) {
    for (int i = 0; i < pre; ++i) {      // token tiles of the stages whose weight tiles are already under way
      const uint32_t fb = smem_u32(full_bar + i);
      const uint32_t sx = smem_u32(tiles + i * SM_STAGE_BYTES) + SM_W_BYTES;
      if (i < n_fp) tma_load_2d<1>(sx, &tm_fx, fb, (c0 + i) * 64, 0);
      else tma_load_2d<1>(sx, &tm_x, fb, (kb_first + i - n_fp) * 128, 0);
    }
  }
  if (warp >= 1) {
    const int te = threadIdx.x - 32;
    if (S > 1)       // only a cluster's leader receives remote sums; every CTA zeroes its tile all the same
      for (int i = te; i < SM_TOKENS * SM_ROWS; i += 256) red[i] = 0;
    if (te < SM_TOKENS) {
      float s = 0.f, z = 0.f;
      if (te < p.M) {
        s = Traits<T>::to_float(static_cast<const T *>(p.meta)[2 * te]);
        z = Traits<T>::to_float(static_cast<const T *>(p.meta)[2 * te + 1]);
      }
      s_srow[te] = s;
      s_zs[te] = fmaf(p.shift_value, s, z);
    }
  }
  __syncthreads();
  // The leader's reduction tile is zeroed: every thread arrives at the cluster barrier now (the TMA warp after its
  // first load is under way); it is waited for before the first remote add.
  if (S > 1 && warp != 0) cluster_arrive();

  // epilogue vectors of the weight row this thread finishes, fetched while the weights stream (kept in storage
  // format: converting here would wait for loads that take microseconds while the stream saturates HBM)
  T ep_scol = Traits<T>::from_float(0.f), ep_wred = ep_scol, ep_bias = ep_scol;
  const int ep_row = (threadIdx.x - 32) & (SM_ROWS - 1), ep_half = (threadIdx.x - 32) >> 7;   // valid for warps 1-8
  if (warp >= 1 && rank == 0 && n0 + ep_row < p.N) {
    ep_scol = static_cast<const T *>(p.scale_col)[n0 + ep_row];
    ep_wred = static_cast<const T *>(p.w_reduced)[n0 + ep_row];
    if (p.bias) ep_bias = static_cast<const T *>(p.bias)[n0 + ep_row];
  }

  int ci[4][4];
  float cf[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      ci[i][j] = 0;
      cf[i][j] = 0.f;
    }

  if (warp == 0) {
    // ================= TMA producer =================
    const uint64_t once = l2_policy_evict_first();      // the weights are read once
    auto issue = [&](int i, int stage) {
      const uint32_t fb = smem_u32(full_bar + stage);
      const uint32_t sw = smem_u32(tiles + stage * SM_STAGE_BYTES);
      mbar_expect_tx(fb, SM_STAGE_BYTES);
      if (i < n_fp) {
        tma_load_2d_hint(sw, &tm_fw, fb, (c0 + i) * 64, n0, once);
        tma_load_2d<1>(sw + SM_W_BYTES, &tm_fx, fb, (c0 + i) * 64, 0);
      } else {
        const int kb = kb_first + (i - n_fp);
        tma_load_2d_hint(sw, &tm_w, fb, kb * 128, n0, once);
        tma_load_2d<1>(sw + SM_W_BYTES, &tm_x, fb, kb * 128, 0);
      }
    };
    int i = pre;                          // those stages are complete or under way
    if (lane == 0 && pre == 0 && nb > 0) issue(i++, 0);
    __syncwarp();
    if (S > 1) cluster_arrive();
    if (lane == 0) {
      int stage = i % STAGES;
      uint32_t phase = (uint32_t)((i / STAGES) & 1);
      for (; i < nb; ++i) {
        if (!mbar_wait(smem_u32(empty_bar + stage), phase ^ 1, abort_flag, p.status)) break;
        issue(i, stage);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ================= consumers =================
    const int cw = warp - 1, rg = cw & 3, kh = cw >> 2;
    const int mat = lane >> 3, mrow = lane & 7;           // ldmatrix: this lane addresses row mrow of matrix mat
    // byte offset of chunk (4 kh + mat) in a row r with r % 8 == mrow, under the 128B swizzle
    const uint32_t chunk_off = (uint32_t)(((4 * kh + mat) ^ mrow) << 4);
    int stage = 0;
    uint32_t phase = 0;
    for (int i = 0; i < nb; ++i) {
      if (!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag, p.status)) break;
      if (i == 0) dbg_t[2] = clock64();
      const uint32_t sw = smem_u32(tiles + stage * SM_STAGE_BYTES);
      uint32_t xa[4], xb[4], wv[4][4];
      ldmatrix_x4(xa, sw + SM_W_BYTES + (uint32_t)(mrow * 128) + chunk_off);            // tokens 0-7
      ldmatrix_x4(xb, sw + SM_W_BYTES + (uint32_t)((8 + mrow) * 128) + chunk_off);      // tokens 8-15
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) ldmatrix_x4(wv[nt], sw + (uint32_t)((32 * rg + 8 * nt + mrow) * 128) + chunk_off);
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(empty_bar + stage));       // operands are in registers
      if (i < n_fp) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          mma_fp16<T>(cf[nt], xa[0], xb[0], xa[1], xb[1], wv[nt][0], wv[nt][1]);
          mma_fp16<T>(cf[nt], xa[2], xb[2], xa[3], xb[3], wv[nt][2], wv[nt][3]);
        }
      } else if (BITS == 8) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          mma_s8(ci[nt], xa[0], xb[0], xa[1], xb[1], wv[nt][0], wv[nt][1]);
          mma_s8(ci[nt], xa[2], xb[2], xa[3], xb[3], wv[nt][2], wv[nt][3]);
        }
      } else {
        uint32_t ae[4], ao[4], be[4], bo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          split_nibbles(xa[j], ae[j], ao[j]);
          split_nibbles(xb[j], be[j], bo[j]);
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t we, wo;
            split_nibbles(wv[nt][j], we, wo);
            mma_s8(ci[nt], ae[j], be[j], ao[j], bo[j], we, wo);
          }
      }
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
  }

  // ================= reduction and epilogue =================
  dbg_t[3] = clock64();
  __syncwarp();
  const bool ok = !*abort_flag;
  if (S > 1) cluster_wait();                    // every CTA of the cluster has started: the leader's tile is zero
  __syncthreads();                              // the ring has drained in this CTA: stage 0 may be reused
  // Partial sums leave the registers through shared memory: the two k-half warps of a row group write their 16 x 32
  // sums into separate tiles that reuse drained stages (row pitch 136 words: the paired 8-byte stores of a warp touch
  // every bank once), the finishing thread of a weight row adds the two (and what other CTAs of the cluster sent).
  constexpr int LD = SM_ROWS + 8;
  int *sumA = reinterpret_cast<int *>(tiles + 1 * SM_STAGE_BYTES), *sumB = reinterpret_cast<int *>(tiles + 2 * SM_STAGE_BYTES);
  float *fpA = fp_part, *fpB = reinterpret_cast<float *>(tiles + 3 * SM_STAGE_BYTES);
  if (warp >= 1 && ok) {
    const int cw = warp - 1, rg = cw & 3, kh = cw >> 2, g = lane >> 2, t = lane & 3;
    int *dst = kh ? sumB : sumA;
    float *fdst = kh ? fpB : fpA;
    // accumulator register r of n-tile nt: token g + 8 (r / 2), weight row 32 rg + 8 nt + 2 t + (r % 2)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int row0 = 32 * rg + 8 * nt + 2 * t;
      int v[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) v[r] = BITS == 4 ? (ci[nt][r] >> 8) : ci[nt][r];   // exact: every product carried the factor 256
      *reinterpret_cast<int2 *>(dst + g * LD + row0) = make_int2(v[0], v[1]);
      *reinterpret_cast<int2 *>(dst + (g + 8) * LD + row0) = make_int2(v[2], v[3]);
      if (rank == 0 && p.nf > 0) {
        *reinterpret_cast<float2 *>(fdst + g * LD + row0) = make_float2(cf[nt][0], cf[nt][1]);
        *reinterpret_cast<float2 *>(fdst + (g + 8) * LD + row0) = make_float2(cf[nt][2], cf[nt][3]);
      }
    }
  }
  __syncthreads();
  if (S > 1) {
    if (warp >= 1 && rank != 0 && ok) {         // one pass of remote adds per CTA: its 16 x 128 sums into the leader's tile
      const uint32_t red_base = map_to_rank(smem_u32(red), 0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int m = 8 * ep_half + j;
        red_add_cluster(red_base + (uint32_t)((m * SM_ROWS + ep_row) * 4), sumA[m * LD + ep_row] + sumB[m * LD + ep_row]);
      }
    }
    cluster_arrive();
    cluster_wait();                             // all partial sums have reached the leader
  }
  dbg_t[4] = clock64();
  if (warp >= 1 && rank == 0 && ok) {
    const int n = n0 + ep_row;
    if (n < p.N) {
      const float scol = Traits<T>::to_float(ep_scol), wred = Traits<T>::to_float(ep_wred), bias = Traits<T>::to_float(ep_bias);
      T *out = static_cast<T *>(p.out);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int m = 8 * ep_half + j;
        if (m < p.M) {
          const int acc = sumA[m * LD + ep_row] + sumB[m * LD + ep_row] + (S > 1 ? red[m * SM_ROWS + ep_row] : 0);
          // outlier sums of the two k halves in fixed order
          const float add = fmaf(s_zs[m], wred, (p.nf > 0 ? fpA[m * LD + ep_row] + fpB[m * LD + ep_row] : 0.f) + bias);
          out[(size_t)m * p.ldo + n] = Traits<T>::from_float(fmaf((float)acc, s_srow[m] * scol, add));
        }
      }
    }
  }
  if (p.dbg && threadIdx.x == 32) {
    unsigned long long *d = p.dbg + (size_t)blockIdx.x * 16;
    dbg_t[5] = clock64();
    for (int i = 0; i < 6; ++i) d[i] = (unsigned long long)dbg_t[i];
    d[6] = (unsigned long long)nb;
    d[7] = (unsigned long long)rank;
    d[8] = global_timer_ns();
  }
  if (*abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);   // let bulk copies in flight land
  }
}

template <typename T, int BITS>
int launch_t(const CUtensorMap &tw, const CUtensorMap &tx, const CUtensorMap &tfw, const CUtensorMap &tfx,
             const MmaStreamParams &p, int slabs, cudaStream_t st) {
  auto kern = stream_w_mma_kernel<T, BITS>;
  static PerDeviceSmem state;
  {
    const int rc = ensure_smem(state, kern, sm_smem(SM_STAGES_DEEP));      // the larger of the two ring depths
    if (rc != QUIK_OK) return rc;
  }
  LaunchCfg lc(dim3(slabs * p.splits), dim3(SM_THREADS2), sm_smem(p.stages), st, p.splits);
  QUIK_CUDA_TRY(cudaLaunchKernelEx(&lc.cfg, kern, tw, tx, tfw, tfx, p));
  return check_launch("stream_w_mma_kernel");
}

}  // namespace

// q, w in the reference's storage format: packed int4 [M, K_int/2] / [N, K_int/2] (bits == 4) or int8 (bits == 8).
int launch_stream_w_mma(const void *q, const void *w, int bits, int M, int N, int K_int, const Epilogue &ep,
                        cudaStream_t st) {
  if (M == 0 || N == 0) return QUIK_OK;
  if (M > SM_TOKENS) return QUIK_ERR_UNSUPPORTED;
  if (K_int <= 0 || K_int % (bits == 4 ? 32 : 16) != 0) return QUIK_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(w)) return QUIK_ERR_ALIGN;
  const bool has_fp = ep.fp_a != nullptr && ep.F > 0;
  if (has_fp && (ep.F % 8 != 0 || !aligned16(ep.fp_a) || !aligned16(ep.fp_b))) return QUIK_ERR_ALIGN;
  if (ep.meta == nullptr || ep.w_reduced == nullptr || ep.y != nullptr) return QUIK_ERR_UNSUPPORTED;

  MmaStreamParams p{};
  p.M = M;
  p.N = N;
  const int row_bytes = bits == 4 ? K_int / 2 : K_int;
  p.nk = (row_bytes + 127) / 128;
  p.nf = has_fp ? (ep.F + 63) / 64 : 0;
  const int slabs = (N + SM_ROWS - 1) / SM_ROWS;
  // Split K over a cluster in powers of two (at most 4 CTAs: 8 measured slower, and so did 3: choosing the split by
  // waves x k-blocks per CTA made the 7B qkv and gate+up layers 22.5 / 27.0 us instead of 16.7 / 20.6) while all CTAs still fit on the GPU at once (two per
  // SM), every CTA keeps at least two k-blocks and the outlier blocks all fall to the first CTA.
  const int total = p.nk + p.nf, slots = 2 * num_sms();
  int splits = 1;
  while (splits < 4 && slabs * splits * 2 <= slots && total / (splits * 2) >= (p.nf > 2 ? p.nf : 2)) splits *= 2;
  p.splits = splits;
  // a grid of at most one CTA per SM leaves half of every SM's shared memory unused with the short ring: such layers
  // get the deep one (bytes in flight per CTA / loaded DRAM latency is what a CTA streams at)
  const int ring = get_stream_ring();
  if (ring == 2 && splits > 1 && slabs * splits > num_sms() && slabs * (splits / 2) <= num_sms()) splits /= 2;
  p.splits = splits;
  p.stages = (ring != 1 && slabs * splits <= num_sms()) ? SM_STAGES_DEEP : SM_STAGES;
  p.preload = get_stream_preload();
  // L2 prefetch before the wait.  Without preload: the first ring fill only (deeper was measured slower: the requests
  // delay the first real loads).  With preload the real loads go first, and the prefetch covers the blocks after them
  // up to 64 MiB over the CTAs resident at once (a 7B layer entirely; half of L2 at most).
  {
    const int resident = slabs * splits < slots ? slabs * splits : slots;
    const int deep = (int)(((size_t)64 << 20) / SM_W_BYTES) / (resident > 0 ? resident : 1);
    p.prefetch_blocks = p.preload == 2 ? (deep > SM_STAGES ? deep : SM_STAGES) : (p.preload == 1 ? 0 : SM_STAGES);
  }
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
  if ((rc = make_tmap(&tw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, row_bytes, SM_ROWS)) != QUIK_OK) return rc;
  if ((rc = make_tmap(&tx, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, row_bytes, SM_TOKENS)) != QUIK_OK) return rc;
  if (has_fp) {
    const CUtensorMapDataType fdt = ep.dtype == QUIK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if ((rc = make_tmap(&tfw, ep.fp_b, fdt, 2, N, ep.F, SM_ROWS)) != QUIK_OK) return rc;
    if ((rc = make_tmap(&tfx, ep.fp_a, fdt, 2, M, ep.F, SM_TOKENS)) != QUIK_OK) return rc;
  } else {
    tfw = tw;
    tfx = tx;
  }
  if (ep.dtype == QUIK_BF16)
    return bits == 4 ? launch_t<__nv_bfloat16, 4>(tw, tx, tfw, tfx, p, slabs, st)
                     : launch_t<__nv_bfloat16, 8>(tw, tx, tfw, tfx, p, slabs, st);
  return bits == 4 ? launch_t<__half, 4>(tw, tx, tfw, tfx, p, slabs, st)
                   : launch_t<__half, 8>(tw, tx, tfw, tfx, p, slabs, st);
}

}  // namespace quik
