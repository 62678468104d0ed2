// Epilogue of the tiled tcgen05 GEMMs (gemm_tcgen05.cu, gemm_tcgen05_ts.cu): launch parameters and the work of
// the eight epilogue warps of a CTA -- parking the outlier product, the dequantize arithmetic of
// QUIK src/asymmetric/asymmetric.cu:134-146 and the stores of the finished tile.
#pragma once
#include "common.cuh"
#include "tcgen05_ptx.cuh"

namespace quik {

namespace {

constexpr int BLOCK_M = 128;
constexpr int STAGE_K_BYTES = 128;           // one 128B-swizzle row of K per stage
constexpr int NUM_EPI_THREADS = 256;         // eight epilogue warps
constexpr int EPI_BUF_BYTES = 32 * 64;       // output staging of one epilogue warp: 32 rows x 64 bytes
constexpr int SMEM_LIMIT = 227 * 1024;

struct GemmParams {
  int M, N;
  int block_n;                    // tile width: multiple of 16
  int split_n;                    // columns of a tile that the first four epilogue warps take (multiple of 32 or block_n)
  int num_m_tiles, num_tiles;
  int int_kb, fp_kb;              // k-blocks per tile: integer (128 codes each) and outlier (64 elems)
  uint32_t idesc_int, idesc_fp;   // tcgen05 instruction descriptors
  int mode;                       // 0: int32 C, 1: dequantize
  int acc_shift;                  // the integer accumulator holds the product times 2^acc_shift (operands widened on chip)
  int a_slots;                    // operand slots in tensor memory (engine with the token operand in tensor memory)
  int l2_hint;                    // token-operand loads carry an L2 evict-last hint
  int issuers;                    // threads that issue the integer products (engine with both operands in shared memory)
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
  unsigned int *status;            // device status word that a wait which ran out sets
};

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
// One epilogue warp.  Warp (sub, half) owns rows [32*sub, 32*sub+32) of the CTA's 128 rows of the tile and the
// columns [cb, cb + cn): the first split_n columns for half 0, the rest for half 1.  It walks them 32 at a time; the
// last step of a range whose length is not a multiple of 32 holds 16 valid columns (`valid` below), the rest is
// ignored.  Tile j of the CTA uses accumulator region j & 1 (region_stride tensor-memory columns apart) for both of
// its products:
//   drain(j)   the outlier product (f32) + bias, rounded to T, is parked in the tile's place in `out` (it stays in
//              L2), which frees the region for the integer product;
//   finish(j)  the integer product (s32) is combined with the parked value by the dequantize arithmetic and the
//              result overwrites the parked value.
// Where the outlier product of (this warp, tile) is parked: every full 32 x 32 chunk inside its own 32-row x 64-byte
// block of `out` (so the final store of one chunk never touches the parked data of another), but permuted: the jj-th
// 16-byte piece of lane L goes to row 8*jj + L/4, piece L%4 of the block, so one warp instruction writes 8 rows x 64
// contiguous bytes (whole sectors) instead of 32 rows x 16 bytes.  The same lane reads its pieces back from the same
// addresses; nobody else looks at them.  Chunks that touch the matrix edge or hold fewer than 32 valid columns keep
// the plain row-per-lane layout with guards.
template <typename T, bool HAS_FP, int CTAS>
struct EpilogueWarp {
  const GemmParams &p;
  uint32_t tmem_base;
  int region_stride;                 // tensor-memory columns between the two accumulator regions
  int unit, num_units, rank;         // this CTA's unit (CTA or pair), number of units, rank inside the pair
  int lane, sub, half;
  int cb, cn, cn32;
  float *s_scol, *s_wred, *s_bias;   // [half_cap] each, private to this warp
  unsigned char *s_stage;            // 32 x 64 bytes, private to this warp
  uint64_t *acc_full, *acc_empty, *fp_full, *fp_drained;
  volatile int *abort_flag;
  bool ok = true;
  long long e_wait_fp = 0, e_wait_acc = 0, e_drain = 0, e_finish = 0;

  __device__ __forceinline__ EpilogueWarp(const GemmParams &p_, uint32_t tmem_base_, int region_stride_, int unit_,
                                          int num_units_, int rank_, int e, int sub_, int lane_, float *s_vec,
                                          int half_cap, unsigned char *s_out, uint64_t *acc_full_,
                                          uint64_t *acc_empty_, uint64_t *fp_full_, uint64_t *fp_drained_,
                                          volatile int *abort_flag_)
      : p(p_), tmem_base(tmem_base_), region_stride(region_stride_), unit(unit_), num_units(num_units_), rank(rank_),
        lane(lane_), sub(sub_), half(e >> 2), acc_full(acc_full_), acc_empty(acc_empty_), fp_full(fp_full_),
        fp_drained(fp_drained_), abort_flag(abort_flag_) {
    cb = half ? p.split_n : 0;
    cn = half ? p.block_n - p.split_n : p.split_n;
    cn32 = (cn + 31) & ~31;
    s_scol = s_vec + e * 3 * half_cap;
    s_wred = s_scol + half_cap;
    s_bias = s_wred + half_cap;
    s_stage = s_out + e * EPI_BUF_BYTES;
  }

  __device__ __forceinline__ uint4 *parked_piece(T *sub_base, int c0, int jj) const {   // sub_base = &out[first row of warp][n0]
    return reinterpret_cast<uint4 *>(sub_base + (size_t)(8 * jj + (lane >> 2)) * p.ldo + c0) + (lane & 3);
  }

  // park T(outlier product + bias) of tile j in `out`
  __device__ __forceinline__ void drain(int j) {
    constexpr int TILE_M = BLOCK_M * CTAS;
    const int tile = unit + j * num_units;
    const int m0 = (tile % p.num_m_tiles) * TILE_M + rank * BLOCK_M + sub * 32;   // first row of this warp
    const int n0 = (tile / p.num_m_tiles) * p.block_n + cb;
    const int lim = min(p.N - n0, cn);       // valid columns from n0 on (<= 0: none)
    const int r = j & 1;
    __syncwarp();
    for (int c = lane; c < cn32; c += 32)
      s_bias[c] = (c < lim && p.bias) ? ldf<T>(p.bias, n0 + c) : 0.f;
    __syncwarp();
    const long long tw = clock64();
    const bool ready = mbar_wait(smem_u32(fp_full + r), (uint32_t)(j >> 1) & 1u, abort_flag, p.status);
    if (!__all_sync(0xffffffffu, ready)) { ok = false; return; }
    const long long tw1 = clock64();
    e_wait_fp += tw1 - tw;
    tc_fence_after();
    const int row = m0 + lane;
    const bool rows_in = m0 + 32 <= p.M;
    T *sub_base = static_cast<T *>(p.out) + (size_t)m0 * p.ldo + n0;
    const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + r * region_stride + cb;
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
  }

  __device__ __forceinline__ void prefetch_parked(uint4 (&pk_next)[4], T *sub_base, const T *my_row, bool rows_in,
                                                  bool row_ok, int lim, int c0) const {
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
  }

  __device__ __forceinline__ void finish(int j) {
    constexpr int TILE_M = BLOCK_M * CTAS;
    const int tile = unit + j * num_units;
    const int m0 = (tile % p.num_m_tiles) * TILE_M + rank * BLOCK_M + sub * 32;   // first row of this warp
    const int n0 = (tile / p.num_m_tiles) * p.block_n + cb;
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
    prefetch_parked(pk_next, sub_base, my_row, rows_in, row_ok, lim, 0);
    const long long tw = clock64();
    const bool ready = mbar_wait(smem_u32(acc_full + r), (uint32_t)(j >> 1) & 1u, abort_flag, p.status);
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
    const int shift = p.acc_shift;
    const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + r * region_stride + cb;
#pragma unroll 1
    for (int c0 = 0; c0 < cn; c0 += 32) {
      uint32_t v[32];
      uint4 pk[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pk[i] = pk_next[i];
      __syncwarp();                          // tcgen05.ld is warp-collective: reconverge first
      tmem_ld32(taddr + c0, v);
      if (c0 + 32 < cn) prefetch_parked(pk_next, sub_base, my_row, rows_in, row_ok, lim, c0 + 32);
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
            if (4 * i < valid)
              dst[i] = make_int4((int)v[4 * i] >> shift, (int)v[4 * i + 1] >> shift, (int)v[4 * i + 2] >> shift,
                                 (int)v[4 * i + 3] >> shift);
        } else {
          for (int i = 0; i < 32; ++i)
            if (i < valid) p.C[off + i] = (int)v[i] >> shift;
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
          o[i] = fmaf((float)((int)v[i] >> shift), srow * sc[q], fmaf(zs, wr[q], o[i]));
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
  }

  // all tiles of this CTA, in the order that lets drain(j + 1) and finish(j) hide behind the products of tile j / j + 1
  __device__ __forceinline__ void run(int n_local) {
    if (HAS_FP && n_local > 0) drain(0);
    for (int j = 0; j < n_local && ok; ++j) {
      if (HAS_FP && j + 1 < n_local) drain(j + 1);
      if (!ok) break;
      finish(j);
    }
  }

  __device__ __forceinline__ void write_counters(int cta) const {
    unsigned long long *d = p.dbg + (size_t)cta * 16;
    d[4] = (unsigned long long)e_wait_fp;     // epilogue warp: waiting for an outlier product
    d[5] = (unsigned long long)e_wait_acc;    // ... waiting for an integer product
    d[6] = (unsigned long long)e_drain;       // ... parking outlier products
    d[7] = (unsigned long long)e_finish;      // ... final epilogues
  }
};

// ---- host helpers shared by the launchers -----------------------------------------------------
struct TileGeometry {
  int ctas, block_n;
};
// fills the shape-independent fields of GemmParams from the epilogue description
inline void fill_epilogue_params(GemmParams &p, const Epilogue &ep, int M, int N) {
  p.M = M;
  p.N = N;
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
  p.dbg = get_debug_counters();
  p.status = device_status_word();
}
inline int split_columns(int block_n) {
  const int h = (block_n / 2 + 31) & ~31;
  return h < block_n ? h : block_n;
}

}  // namespace
}  // namespace quik
