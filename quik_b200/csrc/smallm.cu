// Weight-streaming kernel for the small-batch regime (M <= 16 tokens), where the layer is bound
// by reading the weights from HBM once.  It consumes the weights in their storage format --
// packed int4 (two codes per byte, QUIK include/int4.h:78-98) or int8 -- straight from global
// memory into mma.sync fragments, so no unpacked copy of the weights is ever read or written:
//   int4 and int8: mma.sync.m16n8k32.s8   outliers: mma.sync.m16n8k16.f16/bf16
// (the 4-bit form of mma.sync is emulated on this architecture and ran at a tenth of the HBM rate;
// instead each packed word is split with three logic operations into two words of signed bytes
// that carry 16 x the code, and the factor 256 is shifted out of the exact int32 sum at the end)
// and applies the dequantize epilogue of QUIK src/asymmetric/asymmetric.cu:134-146 in the same
// launch (out = T(acc*(s_m*sw_n) + ((z_m + shift*s_m)*wred_n + (acc_fp + bias_n)))).
//
// Mapping: the tokens are the 16-row operand, 8 weight rows are the 8-column operand.  A dot
// product does not depend on the order of its terms, so each lane takes 32 contiguous bytes of a
// weight row (two 128-bit loads) and of the matching token rows per 128-byte k-block and feeds
// word j / word j+4 to MMA j: every 128-byte line of the weights is read exactly once, fully
// coalesced, with identical k-permutation on both operands.  A CTA owns 8 weight rows; its 8
// warps split the k-blocks (split-K inside the CTA, reduced through shared memory).
#include "common.cuh"

namespace quik {
namespace {

constexpr int SM_THREADS = 256, SM_WARPS = 8;

__device__ __forceinline__ uint4 ld_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight packed int4 codes -> two words of four signed bytes, each byte = 16 * code: the even
// codes (low nibbles) are shifted into the high half of their byte, the odd codes already sit
// there.  A product of two such bytes is 256 * (code_a * code_b), removed exactly at the end.
__device__ __forceinline__ void split_nibbles(uint32_t w, uint32_t &even16, uint32_t &odd16) {
  even16 = (w << 4) & 0xF0F0F0F0u;
  odd16 = w & 0xF0F0F0F0u;
}

template <typename T>
__device__ __forceinline__ void mma_fp(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_fp<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_fp<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                      uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two 16-byte pieces (bytes [off, off+16) and [off+16, off+32)) of a row; pieces beyond the row
// end or of an absent row read as zero.
__device__ __forceinline__ void load_pair(const uint8_t *row, bool row_ok, int off, int row_bytes, bool stream,
                                          uint4 &lo, uint4 &hi) {
  const uint4 z = make_uint4(0, 0, 0, 0);
  lo = z;
  hi = z;
  if (!row_ok) return;
  if (off + 16 <= row_bytes) lo = stream ? ld_stream(row + off) : __ldg(reinterpret_cast<const uint4 *>(row + off));
  if (off + 32 <= row_bytes) hi = stream ? ld_stream(row + off + 16) : __ldg(reinterpret_cast<const uint4 *>(row + off + 16));
}

template <typename T, int BITS, int NT>
__global__ void __launch_bounds__(SM_THREADS)
small_m_kernel(const uint8_t *__restrict__ q, const uint8_t *__restrict__ w, int M, int N, int row_bytes,
               const T *__restrict__ fp_x, const T *__restrict__ fp_w, int F, const T *__restrict__ meta,
               const T *__restrict__ scale_col, const T *__restrict__ wred, const T *__restrict__ bias,
               T *__restrict__ out, long long ldo) {
  __shared__ int s_int[SM_WARPS][NT][32][4];
  __shared__ float s_fp[SM_WARPS][NT][32][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * (8 * NT);
  const bool m_lo = g < M, m_hi = g + 8 < M;

  const int int_blocks = (row_bytes + 127) >> 7;
  const int fp_bytes = F * (int)sizeof(T);
  const int fp_blocks = (fp_bytes + 127) >> 7;
  const int nblocks = int_blocks + fp_blocks;

  const uint8_t *w_row[NT];
  const uint8_t *fw_row[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int wr = min(n0 + nt * 8 + g, N - 1);        // clamped weight row (stores are masked)
    w_row[nt] = w + (size_t)wr * row_bytes;
    fw_row[nt] = reinterpret_cast<const uint8_t *>(fp_w) + (size_t)wr * fp_bytes;
  }
  // Ask L2 for this CTA's share of the weights (all of it: 8*NT rows), then wait for the kernel that produces
  // the token codes: the weight stream from HBM overlaps that kernel and its launch.
  pdl_launch_dependents();
  {
    const int lines_per_row = (row_bytes + 127) >> 7, fp_lines = (fp_bytes + 127) >> 7;
    const int rows_here = min(8 * NT, N - n0);
    for (int i = threadIdx.x; i < rows_here * lines_per_row; i += SM_THREADS) {
      const int rr = i / lines_per_row, ln = i - rr * lines_per_row;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(w + (size_t)(n0 + rr) * row_bytes + (size_t)ln * 128));
    }
    for (int i = threadIdx.x; i < rows_here * fp_lines; i += SM_THREADS) {
      const int rr = i / fp_lines, ln = i - rr * fp_lines;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(fp_w) + (size_t)(n0 + rr) * fp_bytes + (size_t)ln * 128));
    }
  }
  pdl_wait();
  const uint8_t *q_lo = q + (size_t)g * row_bytes;
  const uint8_t *q_hi = q + (size_t)(g + 8) * row_bytes;
  const uint8_t *fx_lo = reinterpret_cast<const uint8_t *>(fp_x) + (size_t)g * fp_bytes;
  const uint8_t *fx_hi = reinterpret_cast<const uint8_t *>(fp_x) + (size_t)(g + 8) * fp_bytes;

  int ci[NT][4];
  float cf[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      ci[nt][r] = 0;
      cf[nt][r] = 0.f;
    }

  // The outlier blocks come first in the block numbering so that they spread over the warps
  // that would otherwise start one integer block later.
#pragma unroll 2
  for (int b = warp; b < nblocks; b += SM_WARPS) {
    const bool is_fp = b < fp_blocks;
    const int off = (is_fp ? b : b - fp_blocks) * 128 + t * 32;
    uint4 wl[NT], wh[NT], al, ah, bl, bh;
    if (is_fp) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) load_pair(fw_row[nt], true, off, fp_bytes, true, wl[nt], wh[nt]);
      load_pair(fx_lo, m_lo, off, fp_bytes, false, al, ah);
      load_pair(fx_hi, m_hi, off, fp_bytes, false, bl, bh);
      const uint32_t A0[4] = {al.x, al.y, al.z, al.w}, A1[4] = {ah.x, ah.y, ah.z, ah.w};
      const uint32_t B0[4] = {bl.x, bl.y, bl.z, bl.w}, B1[4] = {bh.x, bh.y, bh.z, bh.w};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint32_t W0[4] = {wl[nt].x, wl[nt].y, wl[nt].z, wl[nt].w}, W1[4] = {wh[nt].x, wh[nt].y, wh[nt].z, wh[nt].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_fp<T>(cf[nt], A0[j], B0[j], A1[j], B1[j], W0[j], W1[j]);
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) load_pair(w_row[nt], true, off, row_bytes, true, wl[nt], wh[nt]);
      load_pair(q_lo, m_lo, off, row_bytes, false, al, ah);
      load_pair(q_hi, m_hi, off, row_bytes, false, bl, bh);
      const uint32_t A0[4] = {al.x, al.y, al.z, al.w}, A1[4] = {ah.x, ah.y, ah.z, ah.w};
      const uint32_t B0[4] = {bl.x, bl.y, bl.z, bl.w}, B1[4] = {bh.x, bh.y, bh.z, bh.w};
      if (BITS == 8) {
        // word j holds k 4j..4j+3 of the lane's first 16 bytes, word j of the second piece the next 16
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t W0[4] = {wl[nt].x, wl[nt].y, wl[nt].z, wl[nt].w}, W1[4] = {wh[nt].x, wh[nt].y, wh[nt].z, wh[nt].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_s8(ci[nt], A0[j], B0[j], A1[j], B1[j], W0[j], W1[j]);
        }
      } else {
        // every packed word (8 codes) feeds one MMA: even codes form the low k-half, odd codes the high
        const uint32_t AW[8] = {A0[0], A0[1], A0[2], A0[3], A1[0], A1[1], A1[2], A1[3]};
        const uint32_t BW[8] = {B0[0], B0[1], B0[2], B0[3], B1[0], B1[1], B1[2], B1[3]};
        uint32_t ae[8], ao[8], be[8], bo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          split_nibbles(AW[j], ae[j], ao[j]);
          split_nibbles(BW[j], be[j], bo[j]);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t WW[8] = {wl[nt].x, wl[nt].y, wl[nt].z, wl[nt].w, wh[nt].x, wh[nt].y, wh[nt].z, wh[nt].w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t we, wo;
            split_nibbles(WW[j], we, wo);
            mma_s8(ci[nt], ae[j], be[j], ao[j], bo[j], we, wo);
          }
        }
      }
    }
  }

#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      s_int[warp][nt][lane][r] = ci[nt][r];
      s_fp[warp][nt][lane][r] = cf[nt][r];
    }
  __syncthreads();

  for (int o = threadIdx.x; o < NT * 128; o += SM_THREADS) {
    const int nt = o >> 7, l = (o >> 2) & 31, r = o & 3;
    int acc = 0;
    float facc = 0.f;
#pragma unroll
    for (int wv = 0; wv < SM_WARPS; ++wv) {
      acc += s_int[wv][nt][l][r];
      facc += s_fp[wv][nt][l][r];
    }
    if (BITS == 4) acc >>= 8;      // both operands carried a factor 16; the quotient is exact
    // accumulator register r of lane l: row (l/4) + 8*(r/2) of the token tile, column 2*(l%4) + (r%2)
    const int m = (l >> 2) + ((r >> 1) << 3);
    const int n = n0 + nt * 8 + ((l & 3) << 1) + (r & 1);
    if (m < M && n < N) {
      const float srow = Traits<T>::to_float(meta[2 * m]);
      const float zrow = Traits<T>::to_float(meta[2 * m + 1]);
      const float shift = BITS == 4 ? 8.0f : 128.0f;
      float add = facc;
      if (bias) add += Traits<T>::to_float(bias[n]);
      add = fmaf(fmaf(shift, srow, zrow), Traits<T>::to_float(wred[n]), add);
      out[(size_t)m * ldo + n] = Traits<T>::from_float(fmaf((float)acc, srow * Traits<T>::to_float(scale_col[n]), add));
    }
  }
}

}  // namespace

int launch_small_m(const void *q, const void *w, int bits, int M, int N, int K_int, const Epilogue &ep,
                   cudaStream_t st) {
  if (M == 0 || N == 0) return QUIK_OK;
  if (M > QUIK_SMALL_M_MAX) return QUIK_ERR_UNSUPPORTED;
  const int row_bytes = bits == 4 ? K_int / 2 : K_int;
  if (row_bytes % 16 != 0) return QUIK_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(w)) return QUIK_ERR_ALIGN;
  if (ep.F > 0 && (ep.F % 8 != 0 || !aligned16(ep.fp_a) || !aligned16(ep.fp_b))) return QUIK_ERR_ALIGN;
  if (ep.meta == nullptr || ep.w_reduced == nullptr || ep.y != nullptr) return QUIK_ERR_UNSUPPORTED;
  // weight rows per CTA: as many as still leave at least two CTAs per SM
  const int sms = num_sms();
  const int nt = (N >= 64 * sms) ? 4 : (N >= 32 * sms ? 2 : 1);
  const int grid = (N + 8 * nt - 1) / (8 * nt);
  LaunchCfg lc(dim3(grid), dim3(SM_THREADS), 0, st);
#define QUIK_SM(T, B, NT)                                                                                 \
  QUIK_CUDA_TRY(cudaLaunchKernelEx(                                                                       \
      &lc.cfg, small_m_kernel<T, B, NT>, static_cast<const uint8_t *>(q), static_cast<const uint8_t *>(w), M, N, \
      row_bytes, static_cast<const T *>(ep.fp_a), static_cast<const T *>(ep.fp_b), ep.F,                  \
      static_cast<const T *>(ep.meta), static_cast<const T *>(ep.scale_col),                              \
      static_cast<const T *>(ep.w_reduced), static_cast<const T *>(ep.bias), static_cast<T *>(ep.out),    \
      ep.ldo > 0 ? ep.ldo : (long long)N))
#define QUIK_SM_NT(T, B)                                                                                  \
  do {                                                                                                    \
    if (nt == 4) QUIK_SM(T, B, 4);                                                                        \
    else if (nt == 2) QUIK_SM(T, B, 2);                                                                   \
    else QUIK_SM(T, B, 1);                                                                                \
  } while (0)
  if (ep.dtype == QUIK_BF16) { if (bits == 4) QUIK_SM_NT(__nv_bfloat16, 4); else QUIK_SM_NT(__nv_bfloat16, 8); }
  else { if (bits == 4) QUIK_SM_NT(__half, 4); else QUIK_SM_NT(__half, 8); }
#undef QUIK_SM_NT
#undef QUIK_SM
  return check_launch("small_m_kernel");
}

}  // namespace quik
