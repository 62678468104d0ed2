// Activation quantizers.
//
// asym_quantize_row_kernel: per-token asymmetric int4/int8 quantizer with outlier-column gather.
// Semantics follow the reference kernel (QUIK src/asymmetric/asymmetric.cu:340-490): per row,
// max/min over the gathered integer columns, scale = T(fmaxf((max-min)/(2^b-1), 1e-6f)), zero =
// min, code = clamp(rn(hdiv(hsub(x, zero), scale)), 0, 2^b-1) - 2^(b-1), outlier columns copied.
//
// Design for B200: the reference reads every row three times through 8-byte indices with 2-byte
// loads, one 1024-thread block per row.  Here a row is read from HBM exactly once (16-byte cp.async
// into shared memory, the next row already in flight), the column ids are 16-bit and live in
// registers for the CTA's lifetime, each value is gathered once and kept in registers between the
// max/min pass and the quantize pass, and fp16 rows are processed two values per instruction.
// HBM traffic per row: cols*2 bytes in, codes + outliers + meta out.
#include "common.cuh"

namespace quik {

namespace {

constexpr int kQuantThreads = 256;     // threads per row; few rows use twice as many

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

// ---- one CTA per row at a time ------------------------------------------------------------------------
// 256 threads share a row: each thread gathers a few chunks of 8 values (kept in registers between the
// max/min pass and the quantize pass), the row's max/min go through one block-wide reduction.  A CTA walks
// over rows blockIdx.x, blockIdx.x + gridDim.x, ...; the column ids are read once per CTA (16-bit, in
// registers) and the next row is copied into the second shared-memory buffer (16-byte cp.async) while the
// current one is processed, so HBM latency is paid once per CTA, not once per row.
// IdxT: int64_t (reference ABI) or uint16_t (layer-cached ids).
// NC = register-cached chunks per thread (6 covers rows of up to 12288 integer columns; longer rows gather twice)

//
// PROD: what produces the row that is quantized (the producer of X fused into the quantizer, so that the intermediate
// never goes to HBM; the callers on the input side of the layer, QUIK experiments/llama.py:402-407):
//   0  the row of `src` as it is (quik.asymmetric.quantize);
//   1  RMSNorm of the row: T(float(x) * rsqrt(mean(x^2) + eps)) * aux[col]   (aux = the norm's weight vector;
//      the arithmetic of LlamaRMSNorm: normalise in fp32, round to T, multiply by the weight in T);
//   2  SiLU(src) * aux: T(silu(float(g))) * u with g = src[row, col], u = aux[row, col] (aux = a second matrix,
//      the MLP's `up` output beside its `gate` output), both roundings as torch's F.silu(gate) * up.
template <typename T, int BITS, bool WIDE, typename IdxT, int NC, int NTHR, int PROD>
// (up to four cached chunks fit 80 registers: three CTAs of 256 threads per SM, measured 33.2 against 35.5 us for
// [4096, 8192]; six chunks would spill and measured slower under that bound, they keep two CTAs per SM = 128 registers)
__global__ void __launch_bounds__(NTHR, NTHR == 256 ? (NC <= 4 ? 3 : 2) : 1)
asym_quantize_row_kernel(const T *__restrict__ src, const IdxT *__restrict__ int_idx,
                         const IdxT *__restrict__ fp_idx, int rows, int cols, int num_int, int num_fp,
                         uint8_t *__restrict__ dst, T *__restrict__ meta, T *__restrict__ fp_x,
                         int vec_load, int vec_store, int vec_ids, int nbuf, const T *__restrict__ aux, float eps) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float s_red[2][NTHR / 32];
  const int cols_pad = (cols + 7) & ~7;
  T *s_buf = reinterpret_cast<T *>(smem_raw);          // two row buffers: the next row loads while this one is used
  T *s_aux = s_buf + (size_t)nbuf * cols_pad;          // PROD == 2: the same for the rows of the second matrix
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int num_chunks = (num_int + 7) >> 3;
  constexpr bool kPacked = BITS == 4 && !WIDE;
  pdl_launch_dependents();

  auto prefetch_row = [&](int r, int buf) {
    const unsigned sbase = (unsigned)__cvta_generic_to_shared(s_buf + (size_t)buf * cols_pad);
    const uint4 *g = reinterpret_cast<const uint4 *>(src + (size_t)r * cols);
    for (int i = tid; i < (cols >> 3); i += NTHR)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sbase + i * 16), "l"(g + i));
    if (PROD == 2) {
      const unsigned abase = (unsigned)__cvta_generic_to_shared(s_aux + (size_t)buf * cols_pad);
      const uint4 *ga = reinterpret_cast<const uint4 *>(aux + (size_t)r * cols);
      for (int i = tid; i < (cols >> 3); i += NTHR)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(abase + i * 16), "l"(ga + i));
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  // ids of chunk c as four words of two 16-bit ids; the pad of the last chunk repeats the first id
  auto load_ids = [&](int c, uint32_t (&w)[4]) {
    if (vec_ids) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(int_idx) + c);
      w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i0 = c * 8 + 2 * j, i1 = i0 + 1;
        const uint32_t a = (uint32_t)int_idx[i0 < num_int ? i0 : 0], b = (uint32_t)int_idx[i1 < num_int ? i1 : 0];
        w[j] = (a & 0xffffu) | (b << 16);
      }
    }
  };
  pdl_wait();       // the producer of `src` has completed; nothing global was touched before this point
  if (vec_load && nbuf == 2 && (int)blockIdx.x < rows) prefetch_row(blockIdx.x, 0);
  uint32_t ids[NC][4];
#pragma unroll
  for (int it = 0; it < NC; ++it) {
    const int c = tid + NTHR * it;
    if (c < num_chunks) load_ids(c, ids[it]);
  }

  int buf = 0;
  for (int r = blockIdx.x; r < rows; r += gridDim.x, buf ^= (nbuf - 1)) {
  T *s_row = s_buf + (size_t)buf * cols_pad;
  const unsigned short *row16 = reinterpret_cast<const unsigned short *>(s_row);
  if (vec_load && nbuf == 2) {
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();            // this row has landed for every thread; the other buffer is no longer read
    if (r + (int)gridDim.x < rows) prefetch_row(r + gridDim.x, buf ^ 1);
  } else if (vec_load) {        // very long rows: one buffer, no overlap
    __syncthreads();
    prefetch_row(r, 0);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
  } else {
    __syncthreads();
    const T *row = src + (size_t)r * cols;
    for (int i = tid; i < cols; i += NTHR) s_row[i] = row[i];
    if (PROD == 2) {
      const T *arow = aux + (size_t)r * cols;
      T *s_arow = s_aux + (size_t)buf * cols_pad;
      for (int i = tid; i < cols; i += NTHR) s_arow[i] = arow[i];
    }
    __syncthreads();
  }

  // ---- the producer of X, applied to the row in shared memory
  if (PROD == 1) {
    float ss = 0.f;
    for (int i = tid; i < cols; i += NTHR) {
      const float f = Traits<T>::to_float(s_row[i]);
      ss = fmaf(f, f, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_red[0][warp] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < NTHR / 32; ++w) ss += s_red[0][w];
    const float rstd = rsqrtf(ss / (float)cols + eps);
    for (int i = tid; i < cols; i += NTHR)
      s_row[i] = __hmul(Traits<T>::from_float(Traits<T>::to_float(s_row[i]) * rstd), aux[i]);
    __syncthreads();            // the transformed row is complete; s_red may be written again
  } else if (PROD == 2) {
    const T *s_arow = s_aux + (size_t)buf * cols_pad;
    for (int i = tid; i < cols; i += NTHR) {
      const float g = Traits<T>::to_float(s_row[i]);
      s_row[i] = __hmul(Traits<T>::from_float(g / (1.f + expf(-g))), s_arow[i]);
    }
    __syncthreads();
  }

  // ---- pass 1: gather (kept in registers) and max / min
  uint32_t pr[NC][4];
  float mx = -INFINITY, mn = INFINITY;
  auto gather = [&](const uint32_t (&w)[4], uint32_t (&p)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) p[j] = pack_halves(row16[w[j] & 0xffffu], row16[w[j] >> 16]);
  };
  auto minmax = [&](const uint32_t (&p)[4]) {
    if (Traits<T>::kIsHalf) {
      __half2 mx2 = __float2half2_rn(-INFINITY), mn2 = __float2half2_rn(INFINITY);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mx2 = __hmax2(mx2, *reinterpret_cast<const __half2 *>(&p[j]));
        mn2 = __hmin2(mn2, *reinterpret_cast<const __half2 *>(&p[j]));
      }
      mx = fmaxf(mx, fmaxf(__low2float(mx2), __high2float(mx2)));
      mn = fminf(mn, fminf(__low2float(mn2), __high2float(mn2)));
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const T *e = reinterpret_cast<const T *>(&p[j]);
        const float a = Traits<T>::to_float(e[0]), b = Traits<T>::to_float(e[1]);
        mx = fmaxf(mx, fmaxf(a, b));
        mn = fminf(mn, fminf(a, b));
      }
    }
  };
#pragma unroll
  for (int it = 0; it < NC; ++it) {
    const int c = tid + NTHR * it;
    if (c < num_chunks) {
      gather(ids[it], pr[it]);
      minmax(pr[it]);
    }
  }
  for (int c = tid + NTHR * NC; c < num_chunks; c += NTHR) {   // very long rows
    uint32_t w[4], p[4];
    load_ids(c, w);
    gather(w, p);
    minmax(p);
  }
  mx = warp_max(mx);
  mn = warp_min(mn);
  if (lane == 0) {
    s_red[0][warp] = mx;
    s_red[1][warp] = mn;
  }
  __syncthreads();
#pragma unroll
  for (int w = 0; w < NTHR / 32; ++w) {
    mx = fmaxf(mx, s_red[0][w]);
    mn = fminf(mn, s_red[1][w]);
  }
  const T scale = Traits<T>::from_float(fmaxf((mx - mn) / (float)((1 << BITS) - 1), 1e-6f));
  const T zero = Traits<T>::from_float(mn);           // exact: mn is a value of type T
  if (tid == 0) {
    meta[2 * (size_t)r] = scale;
    meta[2 * (size_t)r + 1] = zero;
  }

  // ---- pass 2: quantize + pack
  uint8_t *drow = dst + (size_t)r * (kPacked ? (size_t)(num_int >> 1) : (size_t)num_int);
  float rcp_scale;
  asm("{rcp.approx.ftz.f32 %0, %1;\n}" : "=f"(rcp_scale) : "f"(Traits<T>::to_float(scale)));
  auto emit = [&](int c, const uint32_t (&p)[4]) {
    uint32_t w0, w1;
    if (Traits<T>::kIsHalf) {
      const __half2 zero2 = __half2half2(*reinterpret_cast<const __half *>(&zero));
      uint32_t codes[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) codes[j] = codes_of_pair<BITS>(p[j], zero2, rcp_scale);
      emit_codes<BITS, kPacked>(codes, w0, w1);
    } else {
      int v[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const T *e = reinterpret_cast<const T *>(&p[j]);
        v[2 * j] = quantize_code<T, BITS>(e[0], zero, scale);
        v[2 * j + 1] = quantize_code<T, BITS>(e[1], zero, scale);
      }
      if (kPacked) {
        w0 = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) w0 |= (uint32_t)(v[j] & 0xF) << (4 * j);
        w1 = 0;
      } else {
        w0 = (uint32_t)(v[0] & 0xFF) | ((uint32_t)(v[1] & 0xFF) << 8) | ((uint32_t)(v[2] & 0xFF) << 16) |
             ((uint32_t)(v[3] & 0xFF) << 24);
        w1 = (uint32_t)(v[4] & 0xFF) | ((uint32_t)(v[5] & 0xFF) << 8) | ((uint32_t)(v[6] & 0xFF) << 16) |
             ((uint32_t)(v[7] & 0xFF) << 24);
      }
    }
    if (kPacked) {
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
#pragma unroll
  for (int it = 0; it < NC; ++it) {
    const int c = tid + NTHR * it;
    if (c < num_chunks) emit(c, pr[it]);
  }
  for (int c = tid + NTHR * NC; c < num_chunks; c += NTHR) {
    uint32_t w[4], p[4];
    load_ids(c, w);
    gather(w, p);
    emit(c, p);
  }

  // ---- outlier columns, verbatim
  T *frow = fp_x + (size_t)r * num_fp;
  for (int j = tid; j < num_fp; j += NTHR) frow[j] = s_row[(int)fp_idx[j]];
  }
}

struct RowProducer {
  const void *aux;     // PROD 1: norm weight [cols]; PROD 2: second matrix [rows, cols]
  float eps;
};

template <typename T, int BITS, bool WIDE, typename IdxT, int NC, int NTHR, int PROD>
int launch_asym_rows_nc(const void *src, int rows, int cols, const void *int_idx, int num_int,
                     const void *fp_idx, int num_fp, void *dst, void *meta, void *fp_x, const RowProducer &pr,
                     cudaStream_t st) {
  const size_t row_bytes = (size_t)((cols + 7) & ~7) * sizeof(T);
  constexpr int kMats = PROD == 2 ? 2 : 1;              // matrices whose rows are staged in shared memory
  const int nbuf = 2 * kMats * row_bytes <= 200 * 1024 ? 2 : 1;
  const size_t smem = nbuf * kMats * row_bytes;
  if (smem > 200 * 1024) return QUIK_ERR_UNSUPPORTED;
  auto kern = asym_quantize_row_kernel<T, BITS, WIDE, IdxT, NC, NTHR, PROD>;
  // shared-memory opt-in and occupancy: once per (instantiation, device, shared-memory size)
  static PerDeviceSmem state;
  int cached_per_sm = 0;
  {
    const int rc = ensure_smem(state, kern, smem, NTHR, &cached_per_sm);
    if (rc != QUIK_OK) return rc;
  }
  const int grid = min(rows, num_sms() * cached_per_sm);
  const int vec_load = (cols % 8 == 0) && aligned16(src) && (PROD != 2 || aligned16(pr.aux));
  const bool packed = (BITS == 4 && !WIDE);
  const int vec_store = (num_int % 8 == 0) && ((reinterpret_cast<uintptr_t>(dst) & (packed ? 3u : 7u)) == 0);
  const int vec_ids = sizeof(IdxT) == 2 && (num_int % 8 == 0) && aligned16(int_idx);
  LaunchCfg lc(dim3(grid), dim3(NTHR), smem, st);
  QUIK_CUDA_TRY(cudaLaunchKernelEx(&lc.cfg, kern, static_cast<const T *>(src), static_cast<const IdxT *>(int_idx),
                                   static_cast<const IdxT *>(fp_idx), rows, cols, num_int, num_fp,
                                   static_cast<uint8_t *>(dst), static_cast<T *>(meta), static_cast<T *>(fp_x),
                                   vec_load, vec_store, vec_ids, nbuf, static_cast<const T *>(pr.aux), pr.eps));
  return check_launch("asym_quantize_row_kernel");
}

template <typename T, int BITS, bool WIDE, typename IdxT, int NTHR, int PROD>
int launch_asym_rows_thr(const void *src, int rows, int cols, const void *int_idx, int num_int,
                         const void *fp_idx, int num_fp, void *dst, void *meta, void *fp_x, const RowProducer &pr,
                         cudaStream_t st) {
  const int per_thread = (((num_int + 7) >> 3) + NTHR - 1) / NTHR;
  if (per_thread <= 2)
    return launch_asym_rows_nc<T, BITS, WIDE, IdxT, 2, NTHR, PROD>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
  if (per_thread <= 4)
    return launch_asym_rows_nc<T, BITS, WIDE, IdxT, 4, NTHR, PROD>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
  return launch_asym_rows_nc<T, BITS, WIDE, IdxT, 6, NTHR, PROD>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
}

// With fewer rows than SMs the row's latency is all there is: 512 threads per row (measured 2.6 / 3.4 us against
// 2.9 / 4.1 us for 16 rows of 4096 / 11008 columns); with many rows 256 threads give more rows in flight per SM
// (10.9 / 21 us against 13.9 / 25.8 us for 2048 rows).  Sharing a long row among 512 or 1024 threads so that every
// thread keeps only two chunks in registers (63 registers instead of 120-128, twice the warps per SM) was measured
// slower: 39 instead of 25 us for 2048 rows of 11008 columns, no gain at 8192 columns.
template <typename T, int BITS, bool WIDE, typename IdxT, int PROD>
int launch_asym_rows(const void *src, int rows, int cols, const void *int_idx, int num_int,
                     const void *fp_idx, int num_fp, void *dst, void *meta, void *fp_x, const RowProducer &pr,
                     cudaStream_t st) {
  // rows so long that two buffers of 256-thread CTAs leave one CTA per SM (more than 100 KB for the pair) also take
  // 512 threads: 115 against 144 us for [4096, 28672]
  if (rows <= num_sms() || (size_t)cols * sizeof(T) * 2 > 100 * 1024)
    return launch_asym_rows_thr<T, BITS, WIDE, IdxT, 2 * kQuantThreads, PROD>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
  return launch_asym_rows_thr<T, BITS, WIDE, IdxT, kQuantThreads, PROD>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
}

template <typename T, typename IdxT, int PROD>
int dispatch_bits(int bits, int wide, const void *src, int rows, int cols, const void *int_idx,
                  int num_int, const void *fp_idx, int num_fp, void *dst, void *meta, void *fp_x,
                  const RowProducer &pr, cudaStream_t st) {
  if (bits == 8)
    return launch_asym_rows<T, 8, true, IdxT, PROD>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst,
                                                    meta, fp_x, pr, st);
  if (wide)
    return launch_asym_rows<T, 4, true, IdxT, PROD>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst,
                                                    meta, fp_x, pr, st);
  return launch_asym_rows<T, 4, false, IdxT, PROD>(src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst,
                                                   meta, fp_x, pr, st);
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
  const RowProducer none{nullptr, 0.f};
  if (dtype == QUIK_F16) {
    return idx_bytes == 8
               ? dispatch_bits<__half, int64_t, 0>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, none, st)
               : dispatch_bits<__half, uint16_t, 0>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, none, st);
  }
  return idx_bytes == 8
             ? dispatch_bits<__nv_bfloat16, int64_t, 0>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, none, st)
             : dispatch_bits<__nv_bfloat16, uint16_t, 0>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, none, st);
}

// The quantizer with the producer of X fused in (16-bit column ids only): prod 1 = RMSNorm with weight vector `aux` and
// `eps`, prod 2 = SiLU(src) * aux with a second matrix `aux`.
int launch_asym_quantize_fused(int prod, const void *src, const void *aux, float eps, int dtype, int rows, int cols,
                               const void *int_idx, int num_int, const void *fp_idx, int num_fp, int bits, int wide,
                               void *dst, void *meta, void *fp_x, cudaStream_t st) {
  if (rows == 0) return QUIK_OK;
  const RowProducer pr{aux, eps};
  if (prod == 1) {
    if (dtype == QUIK_F16)
      return dispatch_bits<__half, uint16_t, 1>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
    return dispatch_bits<__nv_bfloat16, uint16_t, 1>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
  }
  if (prod == 2) {
    if (dtype == QUIK_F16)
      return dispatch_bits<__half, uint16_t, 2>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
    return dispatch_bits<__nv_bfloat16, uint16_t, 2>(bits, wide, src, rows, cols, int_idx, num_int, fp_idx, num_fp, dst, meta, fp_x, pr, st);
  }
  return QUIK_ERR_UNSUPPORTED;
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
