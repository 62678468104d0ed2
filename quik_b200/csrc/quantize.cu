// Activation quantizers.
//
// asym_quantize_kernel: per-token asymmetric int4/int8 quantizer with outlier-column gather.
// Semantics follow the reference kernel (QUIK src/asymmetric/asymmetric.cu:340-490): per row,
// max/min over the gathered integer columns, scale = T(fmaxf((max-min)/(2^b-1), 1e-6f)), zero =
// min, code = clamp(rn(hdiv(hsub(x, zero), scale)), 0, 2^b-1) - 2^(b-1), outlier columns copied.
//
// Design for B200: the reference reads every row three times through 8-byte indices with 2-byte
// loads, one 1024-thread block per row and block-wide barriers.  Here a CTA keeps the column ids
// in shared memory as 16-bit values for its whole lifetime and every warp owns whole rows: it
// streams a row from HBM exactly once (16-byte cp.async into its private shared-memory buffer)
// and does min/max (warp shuffles only), quantize+pack and the outlier gather from that copy, so
// no block-wide barrier sits on the row loop.  HBM traffic per row: cols*2 bytes in, codes +
// outliers + meta out.
#include "common.cuh"

namespace quik {

namespace {

constexpr int kQuantThreads = 256;

template <typename T> __device__ __forceinline__ T t_sub(T a, T b) { return __hsub(a, b); }
template <typename T> __device__ __forceinline__ T t_div(T a, T b) { return __hdiv(a, b); }

template <typename T, int BITS>
__device__ __forceinline__ int quantize_code(T x, T zero, T scale) {
  constexpr int kMaxQ = (1 << BITS) - 1;
  constexpr int kShift = 1 << (BITS - 1);
  int v = Traits<T>::to_int_rn(t_div(t_sub(x, zero), scale));
  return min(max(v, 0), kMaxQ) - kShift;
}

// ---- packed fp16 arithmetic for the quantizer's inner loops ---------------------------------------
// Two gathered values travel in one 32-bit register.  Every step reproduces, per 16-bit half, exactly
// what the scalar chain hsub -> hdiv -> half2int_rn -> clamp of the reference kernel produces:
//   * __hsub2 rounds each half like __hsub;
//   * __hdiv(a, b) is half(rcp.approx.ftz(b) * float(a)) plus a refinement that only touches quotients
//     of magnitude below 2^-17, which become code 0 with or without it -- so the refinement is skipped;
//   * clamping the quotient to [0, 2^b - 1] before rounding equals clamping after (the bounds are
//     integers and rounding is monotone; NaN turns into 0 either way);
//   * adding 1024 in fp16 leaves round-to-nearest-even(q) in the low mantissa bits (ulp is 1 there).
__device__ __forceinline__ uint32_t pack_halves(uint32_t lo, uint32_t hi) { return __byte_perm(lo, hi, 0x5410); }

template <int BITS>
__device__ __forceinline__ uint32_t codes_of_pair(uint32_t pair, __half2 zero2, float rcp_scale) {
  const __half2 d = __hsub2(*reinterpret_cast<const __half2 *>(&pair), zero2);
  const float2 f = __half22float2(d);
  __half2 q = __floats2half2_rn(f.x * rcp_scale, f.y * rcp_scale);
  q = __hmin2(__hmax2(q, __float2half2_rn(0.f)), __float2half2_rn((float)((1 << BITS) - 1)));
  q = __hadd2(q, __float2half2_rn(1024.f));
  return *reinterpret_cast<const uint32_t *>(&q) & 0x00FF00FFu;      // code_lo | code_hi << 16, both unsigned
}

// Four pair words (8 unsigned codes) -> output bytes.  PACKED: 8 nibbles in one word (code - 8 == code ^ 8
// on a nibble).  Otherwise one signed byte per code in two words: code - 128 == code ^ 0x80 (8 bits), and
// code - 8 through a borrow-free byte-wise subtraction (4 bits, one code per byte).
template <int BITS, bool PACKED>
__device__ __forceinline__ void emit_codes(const uint32_t (&c)[4], uint32_t &w0, uint32_t &w1) {
  if (PACKED) {
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) w |= ((c[j] | (c[j] >> 12)) & 0xFFu) << (8 * j);
    w0 = w ^ 0x88888888u;
    w1 = 0;
  } else {
    const uint32_t a = __byte_perm(c[0], c[1], 0x6420), b = __byte_perm(c[2], c[3], 0x6420);
    if (BITS == 8) {
      w0 = a ^ 0x80808080u;
      w1 = b ^ 0x80808080u;
    } else {
      w0 = ((a | 0x80808080u) - 0x08080808u) ^ 0x80808080u;
      w1 = ((b | 0x80808080u) - 0x08080808u) ^ 0x80808080u;
    }
  }
}

// One warp per row.  IdxT: int64_t (reference ABI) or uint16_t (layer-cached ids).
// Shared memory: [column ids of the CTA, 16-bit][one private row buffer per warp].
// CACHE != 0 (fp16 only): packed two-at-a-time arithmetic; CACHE > 0 additionally keeps the gathered
// values of up to CACHE chunks per lane in registers between the max/min pass and the quantize pass,
// so each value is gathered once.  CACHE == 0: scalar intrinsics (bf16).
template <typename T, int BITS, bool WIDE, typename IdxT, int CACHE>
__global__ void __launch_bounds__(kQuantThreads, 2)
asym_quantize_kernel(const T *__restrict__ src, const IdxT *__restrict__ int_idx,
                     const IdxT *__restrict__ fp_idx, int rows, int cols, int num_int, int num_fp,
                     uint8_t *__restrict__ dst, T *__restrict__ meta, T *__restrict__ fp_x,
                     int vec_load, int vec_store, int warps_per_cta) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int num_chunks = (num_int + 7) >> 3;           // 8 codes per chunk
  const int int_pad = num_chunks << 3;
  const int fp_pad = (num_fp + 7) & ~7;
  const int cols_pad = (cols + 7) & ~7;
  uint16_t *s_int = reinterpret_cast<uint16_t *>(smem_raw);               // [int_pad]
  uint16_t *s_fp = s_int + int_pad;                                       // [fp_pad]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  T *s_row = reinterpret_cast<T *>(s_fp + fp_pad) + (size_t)warp * cols_pad;   // this warp's row

  // Column ids -> shared memory, once per CTA; the pad of the last chunk repeats the first id so
  // that it never changes the row's max/min.  16-bit ids are copied eight at a time; every warp
  // first puts the copy of its first row in flight so that both latencies overlap.
  const int first_row = blockIdx.x + gridDim.x * warp;
  const bool prefetched = vec_load && warp < warps_per_cta && first_row < rows;
  if (prefetched) {
    const unsigned sbase = (unsigned)__cvta_generic_to_shared(s_row);
    const uint4 *g = reinterpret_cast<const uint4 *>(src + (size_t)first_row * cols);
    for (int i = lane; i < (cols >> 3); i += 32)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sbase + i * 16), "l"(g + i));
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }
  if (sizeof(IdxT) == 2 && (num_int & 7) == 0 && (reinterpret_cast<uintptr_t>(int_idx) & 15) == 0) {
    const uint4 *g = reinterpret_cast<const uint4 *>(int_idx);
    uint4 *d = reinterpret_cast<uint4 *>(s_int);
    for (int i = tid; i < (num_int >> 3); i += blockDim.x) d[i] = __ldg(g + i);
  } else {
#pragma unroll 4
    for (int i = tid; i < int_pad; i += blockDim.x)
      s_int[i] = static_cast<uint16_t>(i < num_int ? int_idx[i] : int_idx[0]);
  }
  for (int i = tid; i < num_fp; i += blockDim.x) s_fp[i] = static_cast<uint16_t>(fp_idx[i]);
  __syncthreads();
  if (warp >= warps_per_cta) return;

  const size_t dst_pitch = (BITS == 4 && !WIDE) ? (size_t)(num_int >> 1) : (size_t)num_int;
  // rows are dealt round-robin over the CTAs first, then over the warps of a CTA, so that a
  // short matrix still spreads over all SMs
  const int row_stride = gridDim.x * warps_per_cta;

  for (int r = blockIdx.x + gridDim.x * warp; r < rows; r += row_stride) {
    const T *row = src + (size_t)r * cols;
    __syncwarp();   // previous row fully consumed by every lane
    if (prefetched && r == first_row) {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    } else if (vec_load) {
      // global -> shared without a register round trip
      const unsigned sbase = (unsigned)__cvta_generic_to_shared(s_row);
      for (int i = lane; i < (cols >> 3); i += 32)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sbase + i * 16),
                     "l"(reinterpret_cast<const uint4 *>(row) + i));
      asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
    } else {
      for (int i = lane; i < cols; i += 32) s_row[i] = row[i];
    }
    __syncwarp();

    uint8_t *drow = dst + (size_t)r * dst_pitch;
    if (CACHE != 0) {
      // ---------- fp16 fast path: packed arithmetic; CACHE > 0 also keeps the gathered pairs ----------
      const unsigned short *row16 = reinterpret_cast<const unsigned short *>(s_row);
      constexpr int NC = CACHE > 0 ? CACHE : 1;
      uint32_t cache[NC][4];
      __half2 mx2 = __float2half2_rn(-INFINITY), mn2 = __float2half2_rn(INFINITY);
      auto gather_chunk = [&](int c, uint32_t (&pr)[4]) {
        const uint4 idv = *reinterpret_cast<const uint4 *>(s_int + (c << 3));
        const uint32_t w[4] = {idv.x, idv.y, idv.z, idv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) pr[j] = pack_halves(row16[w[j] & 0xffffu], row16[w[j] >> 16]);
      };
      auto minmax_chunk = [&](const uint32_t (&pr)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mx2 = __hmax2(mx2, *reinterpret_cast<const __half2 *>(&pr[j]));
          mn2 = __hmin2(mn2, *reinterpret_cast<const __half2 *>(&pr[j]));
        }
      };
      if (CACHE > 0) {
#pragma unroll
        for (int it = 0; it < NC; ++it) {
          const int c = lane + 32 * it;
          if (c < num_chunks) {
            gather_chunk(c, cache[it]);
            minmax_chunk(cache[it]);
          }
        }
      } else {
#pragma unroll 2
        for (int c = lane; c < num_chunks; c += 32) {
          uint32_t pr[4];
          gather_chunk(c, pr);
          minmax_chunk(pr);
        }
      }
      float mx = warp_max(fmaxf(__low2float(mx2), __high2float(mx2)));
      float mn = warp_min(fminf(__low2float(mn2), __high2float(mn2)));
      const __half scale = __float2half(fmaxf((mx - mn) / (float)((1 << BITS) - 1), 1e-6f));
      const __half zero = __float2half(mn);
      if (lane == 0) {
        reinterpret_cast<__half *>(meta)[2 * (size_t)r] = scale;
        reinterpret_cast<__half *>(meta)[2 * (size_t)r + 1] = zero;
      }
      float rcp_scale;
      asm("{rcp.approx.ftz.f32 %0, %1;\n}" : "=f"(rcp_scale) : "f"(__half2float(scale)));
      const __half2 zero2 = __half2half2(zero);
      auto emit_chunk = [&](int c, const uint32_t (&pr)[4]) {
        uint32_t codes[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) codes[j] = codes_of_pair<BITS>(pr[j], zero2, rcp_scale);
        uint32_t w0, w1;
        emit_codes<BITS, (BITS == 4 && !WIDE)>(codes, w0, w1);
        if (BITS == 4 && !WIDE) {
          if (vec_store) {
            *reinterpret_cast<uint32_t *>(drow + (size_t)c * 4) = w0;
          } else {
            const int nbytes = min(4, (num_int >> 1) - c * 4);
            for (int j = 0; j < nbytes; ++j) drow[c * 4 + j] = (uint8_t)(w0 >> (8 * j));
          }
        } else {
          if (vec_store) {
            *reinterpret_cast<uint2 *>(drow + (size_t)c * 8) = make_uint2(w0, w1);
          } else {
            const int nbytes = min(8, num_int - c * 8);
            for (int j = 0; j < nbytes; ++j)
              drow[c * 8 + j] = (uint8_t)((j < 4 ? w0 >> (8 * j) : w1 >> (8 * (j - 4))) & 0xFF);
          }
        }
      };
      if (CACHE > 0) {
#pragma unroll
        for (int it = 0; it < NC; ++it) {
          const int c = lane + 32 * it;
          if (c < num_chunks) emit_chunk(c, cache[it]);
        }
      } else {
#pragma unroll 2
        for (int c = lane; c < num_chunks; c += 32) {
          uint32_t pr[4];
          gather_chunk(c, pr);
          emit_chunk(c, pr);
        }
      }
    } else {
    // ---- pass 1: max / min over the gathered integer columns
    float mx = -INFINITY, mn = INFINITY;
#pragma unroll 2
    for (int c = lane; c < num_chunks; c += 32) {
      const uint4 idv = *reinterpret_cast<const uint4 *>(s_int + (c << 3));
      const uint32_t w[4] = {idv.x, idv.y, idv.z, idv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = Traits<T>::to_float(s_row[w[j] & 0xffffu]);
        const float b = Traits<T>::to_float(s_row[w[j] >> 16]);
        mx = fmaxf(mx, fmaxf(a, b));
        mn = fminf(mn, fminf(a, b));
      }
    }
    mx = warp_max(mx);
    mn = warp_min(mn);
    const T scale = Traits<T>::from_float(fmaxf((mx - mn) / (float)((1 << BITS) - 1), 1e-6f));
    const T zero = Traits<T>::from_float(mn);           // exact: mn is a value of type T
    if (lane == 0) {
      meta[2 * (size_t)r] = scale;
      meta[2 * (size_t)r + 1] = zero;
    }

    // ---- pass 2: quantize + pack
#pragma unroll 2
    for (int c = lane; c < num_chunks; c += 32) {
      const uint4 idv = *reinterpret_cast<const uint4 *>(s_int + (c << 3));
      const uint32_t w[4] = {idv.x, idv.y, idv.z, idv.w};
      int v[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = quantize_code<T, BITS>(s_row[w[j] & 0xffffu], zero, scale);
        v[2 * j + 1] = quantize_code<T, BITS>(s_row[w[j] >> 16], zero, scale);
      }
      if (BITS == 4 && !WIDE) {
        uint32_t p = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) p |= (uint32_t)(v[j] & 0xF) << (4 * j);
        if (vec_store) {
          *reinterpret_cast<uint32_t *>(drow + (size_t)c * 4) = p;
        } else {
          const int nbytes = min(4, (num_int >> 1) - c * 4);
          for (int j = 0; j < nbytes; ++j) drow[c * 4 + j] = (uint8_t)(p >> (8 * j));
        }
      } else {
        uint2 p;
        p.x = (uint32_t)(v[0] & 0xFF) | ((uint32_t)(v[1] & 0xFF) << 8) |
              ((uint32_t)(v[2] & 0xFF) << 16) | ((uint32_t)(v[3] & 0xFF) << 24);
        p.y = (uint32_t)(v[4] & 0xFF) | ((uint32_t)(v[5] & 0xFF) << 8) |
              ((uint32_t)(v[6] & 0xFF) << 16) | ((uint32_t)(v[7] & 0xFF) << 24);
        if (vec_store) {
          *reinterpret_cast<uint2 *>(drow + (size_t)c * 8) = p;
        } else {
          const int nbytes = min(8, num_int - c * 8);
          for (int j = 0; j < nbytes; ++j)
            drow[c * 8 + j] = (uint8_t)((j < 4 ? p.x >> (8 * j) : p.y >> (8 * (j - 4))) & 0xFF);
        }
      }
    }

    }

    // ---- outlier columns, verbatim
    T *frow = fp_x + (size_t)r * num_fp;
    for (int j = lane; j < num_fp; j += 32) frow[j] = s_row[s_fp[j]];
  }
}

template <typename T, int BITS, bool WIDE, typename IdxT, int CACHE>
int launch_asym_cached(const void *src, int rows, int cols, const void *int_idx, int num_int,
                  const void *fp_idx, int num_fp, void *dst, void *meta, void *fp_x,
                  cudaStream_t st) {
  const int int_pad = ((num_int + 7) >> 3) << 3, fp_pad = (num_fp + 7) & ~7,
            cols_pad = (cols + 7) & ~7;
  const size_t idx_bytes = (size_t)(int_pad + fp_pad) * 2, row_bytes = (size_t)cols_pad * sizeof(T);
  // as many warps (rows in flight) per CTA as shared memory allows, at most 8
  const size_t budget = 200 * 1024;
  int warps = (int)((budget - idx_bytes) / row_bytes);
  if (warps < 1) return QUIK_ERR_UNSUPPORTED;
  if (warps > kQuantThreads / 32) warps = kQuantThreads / 32;
  // small rows: keep the CTA at 8 warps but do not let one CTA hog an SM's shared memory
  const size_t smem = idx_bytes + (size_t)warps * row_bytes;
  auto kern = asym_quantize_kernel<T, BITS, WIDE, IdxT, CACHE>;
  // attribute and occupancy are looked up once per (instantiation, shared-memory size)
  static size_t cached_smem = 0;
  static int cached_per_sm = 0;
  if (cached_smem != smem || cached_per_sm < 1) {
    if (smem > 48 * 1024)
      QUIK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int occ = 0;
    QUIK_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kQuantThreads, smem));
    if (occ < 1) return QUIK_ERR_UNSUPPORTED;
    cached_smem = smem;
    cached_per_sm = occ;
  }
  const int per_sm = cached_per_sm;
  const int grid = max(1, min(rows, num_sms() * per_sm));
  const int vec_load = (cols % 8 == 0) && aligned16(src);
  const bool packed = (BITS == 4 && !WIDE);
  const int vec_store = (num_int % 8 == 0) &&
                        ((reinterpret_cast<uintptr_t>(dst) & (packed ? 3u : 7u)) == 0);
  kern<<<grid, kQuantThreads, smem, st>>>(
      static_cast<const T *>(src), static_cast<const IdxT *>(int_idx),
      static_cast<const IdxT *>(fp_idx), rows, cols, num_int, num_fp, static_cast<uint8_t *>(dst),
      static_cast<T *>(meta), static_cast<T *>(fp_x), vec_load, vec_store, warps);
  return check_launch("asym_quantize_kernel");
}

// fp16 rows of up to 16 chunks per lane (4096 integer columns) take the register-cached packed path
template <typename T, int BITS, bool WIDE, typename IdxT>
int launch_asym_t(const void *src, int rows, int cols, const void *int_idx, int num_int,
                  const void *fp_idx, int num_fp, void *dst, void *meta, void *fp_x,
                  cudaStream_t st) {
  constexpr bool is_half = sizeof(T) == 2 && Traits<T>::kIsHalf;
  if (is_half && num_int <= 8 * 32 * 16)
    return launch_asym_cached<T, BITS, WIDE, IdxT, is_half ? 16 : 0>(src, rows, cols, int_idx, num_int, fp_idx, num_fp,
                                                                      dst, meta, fp_x, st);
  // longer fp16 rows: same packed arithmetic, values gathered in both passes; bf16: scalar intrinsics
  return launch_asym_cached<T, BITS, WIDE, IdxT, is_half ? -1 : 0>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst,
                                                                    meta, fp_x, st);
}

template <typename T, typename IdxT>
int dispatch_bits(int bits, int wide, const void *src, int rows, int cols, const void *int_idx,
                  int num_int, const void *fp_idx, int num_fp, void *dst, void *meta, void *fp_x,
                  cudaStream_t st) {
  if (bits == 8)
    return launch_asym_t<T, 8, true, IdxT>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst,
                                           meta, fp_x, st);
  if (wide)
    return launch_asym_t<T, 4, true, IdxT>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst,
                                           meta, fp_x, st);
  return launch_asym_t<T, 4, false, IdxT>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst,
                                          meta, fp_x, st);
}

// ---------------------------------------------------------------------------------------------
// find_meta: one warp per row, 128-bit loads (QUIK src/asymmetric/asymmetric.cu:263-338).
template <typename T>
__global__ void find_meta_kernel(const T *__restrict__ src, int rows, int cols, int bits,
                                 T *__restrict__ meta, int vec) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const T *row = src + (size_t)warp * cols;
  float mx = -INFINITY, mn = INFINITY;
  if (vec) {
    const uint4 *g = reinterpret_cast<const uint4 *>(row);
    for (int i = lane; i < (cols >> 3); i += 32) {
      uint4 q = __ldg(g + i);
      const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = Traits<T>::to_float(e[j]);
        mx = fmaxf(mx, f);
        mn = fminf(mn, f);
      }
    }
  } else {
    for (int i = lane; i < cols; i += 32) {
      const float f = Traits<T>::to_float(row[i]);
      mx = fmaxf(mx, f);
      mn = fminf(mn, f);
    }
  }
  mx = warp_max(mx);
  mn = warp_min(mn);
  if (lane == 0) {
    meta[2 * (size_t)warp] = Traits<T>::from_float(fmaxf((mx - mn) / (float)((1 << bits) - 1), 1e-6f));
    meta[2 * (size_t)warp + 1] = Traits<T>::from_float(mn);
  }
}

// quantizeOld: elementwise over a pre-gathered matrix (QUIK src/asymmetric/asymmetric.cu:13-66).
// One thread per output byte (bits=4: two codes, the odd tail nibble stays 0).
template <typename T, int BITS>
__global__ void quantize_old_kernel(const T *__restrict__ src, const T *__restrict__ meta, int rows,
                                    int cols, uint8_t *__restrict__ dst) {
  const int cols_dst = BITS == 4 ? (cols + 1) / 2 : cols;
  const size_t total = (size_t)rows * cols_dst;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols_dst), c = (int)(i % cols_dst);
    const T scale = meta[2 * (size_t)r], zero = meta[2 * (size_t)r + 1];
    if (BITS == 8) {
      dst[i] = (uint8_t)(quantize_code<T, 8>(src[(size_t)r * cols + c], zero, scale) & 0xFF);
    } else {
      int lo = quantize_code<T, 4>(src[(size_t)r * cols + 2 * c], zero, scale);
      int hi = (2 * c + 1 < cols) ? quantize_code<T, 4>(src[(size_t)r * cols + 2 * c + 1], zero, scale) : 0;
      dst[i] = (uint8_t)((lo & 0xF) | ((hi & 0xF) << 4));
    }
  }
}

// symmetric quantize, fp16 (QUIK src/symmetric/symmetric.cu:6-78): rn(hdiv(x, scale[row])), no clamp.
template <int BITS>
__global__ void sym_quantize_kernel(const __half *__restrict__ src, const __half *__restrict__ scale,
                                    int rows, int cols, uint8_t *__restrict__ dst) {
  const int cols_dst = BITS == 4 ? (cols + 1) / 2 : cols;
  const size_t total = (size_t)rows * cols_dst;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols_dst), c = (int)(i % cols_dst);
    const __half s = scale[r];
    if (BITS == 8) {
      dst[i] = (uint8_t)(__half2int_rn(__hdiv(src[(size_t)r * cols + c], s)) & 0xFF);
    } else {
      int lo = __half2int_rn(__hdiv(src[(size_t)r * cols + 2 * c], s));
      int hi = (2 * c + 1 < cols) ? __half2int_rn(__hdiv(src[(size_t)r * cols + 2 * c + 1], s)) : 0;
      dst[i] = (uint8_t)((lo & 0xF) | ((hi & 0xF) << 4));
    }
  }
}

inline int ew_grid(size_t total, int threads) {
  size_t blocks = (total + threads - 1) / threads;
  size_t cap = (size_t)num_sms() * 16;
  return (int)max((size_t)1, min(blocks, cap));
}

}  // namespace

int launch_asym_quantize(const void *src, int dtype, int rows, int cols, const void *int_idx,
                         int num_int, const void *fp_idx, int num_fp, int idx_bytes, int bits,
                         int wide, void *dst, void *meta, void *fp_x, cudaStream_t st) {
  if (rows == 0) return QUIK_OK;
  if (dtype == QUIK_F16) {
    return idx_bytes == 8
               ? dispatch_bits<__half, int64_t>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, st)
               : dispatch_bits<__half, uint16_t>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, st);
  }
  return idx_bytes == 8
             ? dispatch_bits<__nv_bfloat16, int64_t>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, st)
             : dispatch_bits<__nv_bfloat16, uint16_t>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, st);
}

int launch_find_meta(const void *src, int dtype, int rows, int cols, int bits, void *meta,
                     cudaStream_t st) {
  if (rows == 0) return QUIK_OK;
  const int threads = 256, grid = (rows * 32 + threads - 1) / threads;
  const int vec = (cols % 8 == 0) && aligned16(src);
  if (dtype == QUIK_F16)
    find_meta_kernel<__half><<<grid, threads, 0, st>>>(static_cast<const __half *>(src), rows, cols, bits, static_cast<__half *>(meta), vec);
  else
    find_meta_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(static_cast<const __nv_bfloat16 *>(src), rows, cols, bits, static_cast<__nv_bfloat16 *>(meta), vec);
  return check_launch("find_meta_kernel");
}

int launch_quantize_old(const void *src, int dtype, const void *meta, int rows, int cols, int bits,
                        void *dst, cudaStream_t st) {
  if (rows == 0 || cols == 0) return QUIK_OK;
  const size_t total = (size_t)rows * (bits == 4 ? (cols + 1) / 2 : cols);
  const int threads = 256, grid = ew_grid(total, threads);
  uint8_t *d = static_cast<uint8_t *>(dst);
  if (dtype == QUIK_F16) {
    auto s = static_cast<const __half *>(src), m = static_cast<const __half *>(meta);
    if (bits == 4) quantize_old_kernel<__half, 4><<<grid, threads, 0, st>>>(s, m, rows, cols, d);
    else quantize_old_kernel<__half, 8><<<grid, threads, 0, st>>>(s, m, rows, cols, d);
  } else {
    auto s = static_cast<const __nv_bfloat16 *>(src), m = static_cast<const __nv_bfloat16 *>(meta);
    if (bits == 4) quantize_old_kernel<__nv_bfloat16, 4><<<grid, threads, 0, st>>>(s, m, rows, cols, d);
    else quantize_old_kernel<__nv_bfloat16, 8><<<grid, threads, 0, st>>>(s, m, rows, cols, d);
  }
  return check_launch("quantize_old_kernel");
}

int launch_sym_quantize(const void *src, const void *scale, int rows, int cols, int bits, void *dst,
                        cudaStream_t st) {
  if (rows == 0 || cols == 0) return QUIK_OK;
  const size_t total = (size_t)rows * (bits == 4 ? (cols + 1) / 2 : cols);
  const int threads = 256, grid = ew_grid(total, threads);
  auto s = static_cast<const __half *>(src), sc = static_cast<const __half *>(scale);
  uint8_t *d = static_cast<uint8_t *>(dst);
  if (bits == 4) sym_quantize_kernel<4><<<grid, threads, 0, st>>>(s, sc, rows, cols, d);
  else sym_quantize_kernel<8><<<grid, threads, 0, st>>>(s, sc, rows, cols, d);
  return check_launch("sym_quantize_kernel");
}

}  // namespace quik
