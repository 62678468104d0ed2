// Elementwise dequantize / unpack kernels (HBM-bound, 128-bit accesses).
#include "common.cuh"

namespace quik {
namespace {

// QUIK src/asymmetric/asymmetric.cu:119-173.  The arithmetic is kept in the reference's order
// with explicit round-to-nearest multiplies and adds so that the compiler cannot contract them
// into fused multiply-adds: out = T( x*(s_r*s_c) + (((z_r + shift*s_r) * wred_c) + y) ).
__device__ __forceinline__ float dequant_value(int acc, float srow, float zrow, float shift,
                                               float scol, float wred, float y) {
  const float sh = __fmul_rn(__fadd_rn(zrow, __fmul_rn(shift, srow)), wred);
  const float xe = __fmul_rn((float)acc, __fmul_rn(srow, scol));
  return __fadd_rn(xe, __fadd_rn(sh, y));
}

template <typename T, int VEC>
__global__ void asym_dequantize_kernel(const int32_t *__restrict__ x, const T *__restrict__ meta,
                                       const T *__restrict__ scale_col, const T *__restrict__ wred,
                                       const T *__restrict__ y, T *__restrict__ out, int rows,
                                       int cols, float shift) {
  const int cvec = cols / VEC;
  const size_t total = (size_t)rows * cvec;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cvec), c0 = (int)(i % cvec) * VEC;
    const float srow = Traits<T>::to_float(meta[2 * (size_t)r]);
    const float zrow = Traits<T>::to_float(meta[2 * (size_t)r + 1]);
    const size_t off = (size_t)r * cols + c0;
    if (VEC == 8) {
      const int4 a0 = __ldg(reinterpret_cast<const int4 *>(x + off));
      const int4 a1 = __ldg(reinterpret_cast<const int4 *>(x + off) + 1);
      const uint4 yv = __ldg(reinterpret_cast<const uint4 *>(y + off));
      const uint4 sv = __ldg(reinterpret_cast<const uint4 *>(scale_col + c0));
      const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(wred + c0));
      const int acc[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const T *ye = reinterpret_cast<const T *>(&yv);
      const T *se = reinterpret_cast<const T *>(&sv);
      const T *we = reinterpret_cast<const T *>(&wv);
      uint4 o;
      T *oe = reinterpret_cast<T *>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        oe[j] = Traits<T>::from_float(dequant_value(acc[j], srow, zrow, shift, Traits<T>::to_float(se[j]),
                                                    Traits<T>::to_float(we[j]), Traits<T>::to_float(ye[j])));
      *reinterpret_cast<uint4 *>(out + off) = o;
    } else {
      out[off] = Traits<T>::from_float(dequant_value(x[off], srow, zrow, shift,
                                                     Traits<T>::to_float(scale_col[c0]),
                                                     Traits<T>::to_float(wred[c0]),
                                                     Traits<T>::to_float(y[off])));
    }
  }
}

// QUIK src/symmetric/symmetric.cu:80-113: fp16 per-operation arithmetic.
template <typename X>
__device__ __forceinline__ __half to_half_rn(X v) { return __int2half_rn((int)v); }
template <> __device__ __forceinline__ __half to_half_rn<__half>(__half v) { return v; }

template <typename X>
__global__ void sym_dequantize_kernel(const X *__restrict__ x, const __half *__restrict__ srow,
                                      const __half *__restrict__ scol, const __half *__restrict__ y,
                                      __half *__restrict__ out, int rows, int cols) {
  const size_t total = (size_t)rows * cols;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols), c = (int)(i % cols);
    // _rn forms: never contracted into a fused multiply-add, so each operation rounds like the torch
    // expression the reference asserts against (test/python/test_cuaprseLt.py:44-47)
    out[i] = __hadd_rn(__hmul_rn(__hmul_rn(to_half_rn<X>(x[i]), srow[r]), scol[c]), y[i]);
  }
}

// packed int4 -> int8, 16 bytes in / 32 bytes out per thread step (include/int4.h:78-98 order:
// low nibble first).
__global__ void unpack_int4_kernel(const uint8_t *__restrict__ src, int8_t *__restrict__ dst,
                                   size_t nbytes, int vec) {
  if (vec) {
    const size_t nvec = nbytes >> 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (size_t)gridDim.x * blockDim.x) {
      const uint4 p = __ldg(reinterpret_cast<const uint4 *>(src) + i);
      const uint32_t w[4] = {p.x, p.y, p.z, p.w};
      uint32_t o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // sign-extend 8 nibbles: (n ^ 8) - 8 per byte lane
        const uint32_t lo = w[j] & 0x0F0F0F0Fu, hi = (w[j] >> 4) & 0x0F0F0F0Fu;
        const uint32_t slo = __vsub4(lo ^ 0x08080808u, 0x08080808u);
        const uint32_t shi = __vsub4(hi ^ 0x08080808u, 0x08080808u);
        // interleave bytes: lo0 hi0 lo1 hi1 | lo2 hi2 lo3 hi3
        o[2 * j] = __byte_perm(slo, shi, 0x5140);
        o[2 * j + 1] = __byte_perm(slo, shi, 0x7362);
      }
      uint4 *d = reinterpret_cast<uint4 *>(dst) + 2 * i;
      d[0] = make_uint4(o[0], o[1], o[2], o[3]);
      d[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes;
         i += (size_t)gridDim.x * blockDim.x) {
      const int b = src[i];
      dst[2 * i] = (int8_t)(((b & 0xF) ^ 8) - 8);
      dst[2 * i + 1] = (int8_t)((((b >> 4) & 0xF) ^ 8) - 8);
    }
  }
}

inline int ew_grid(size_t total, int threads) {
  size_t blocks = (total + threads - 1) / threads;
  size_t cap = (size_t)num_sms() * 16;
  return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace

int launch_asym_dequantize(const int32_t *x, const void *meta, const void *scale_col,
                           const void *w_reduced, const void *y, void *out, int dtype, int rows,
                           int cols, int bits, cudaStream_t st) {
  if (rows == 0 || cols == 0) return QUIK_OK;
  const float shift = bits == 4 ? 8.0f : 128.0f;
  const bool vec = (cols % 8 == 0) && aligned16(x) && aligned16(y) && aligned16(out) &&
                   aligned16(scale_col) && aligned16(w_reduced);
  const int threads = 256;
  const int grid = ew_grid((size_t)rows * (vec ? cols / 8 : cols), threads);
#define QUIK_DQ(T, V)                                                                              \
  asym_dequantize_kernel<T, V><<<grid, threads, 0, st>>>(                                          \
      x, static_cast<const T *>(meta), static_cast<const T *>(scale_col),                          \
      static_cast<const T *>(w_reduced), static_cast<const T *>(y), static_cast<T *>(out), rows,   \
      cols, shift)
  if (dtype == QUIK_F16) { if (vec) QUIK_DQ(__half, 8); else QUIK_DQ(__half, 1); }
  else { if (vec) QUIK_DQ(__nv_bfloat16, 8); else QUIK_DQ(__nv_bfloat16, 1); }
#undef QUIK_DQ
  return check_launch("asym_dequantize_kernel");
}

int launch_sym_dequantize(const void *x, int x_bits, const void *scale_row, const void *scale_col,
                          const void *y, void *out, int rows, int cols, cudaStream_t st) {
  if (rows == 0 || cols == 0) return QUIK_OK;
  const int threads = 256, grid = ew_grid((size_t)rows * cols, threads);
  auto sr = static_cast<const __half *>(scale_row), sc = static_cast<const __half *>(scale_col),
       yy = static_cast<const __half *>(y);
  __half *o = static_cast<__half *>(out);
  if (x_bits == 8) sym_dequantize_kernel<int8_t><<<grid, threads, 0, st>>>(static_cast<const int8_t *>(x), sr, sc, yy, o, rows, cols);
  else if (x_bits == 16) sym_dequantize_kernel<__half><<<grid, threads, 0, st>>>(static_cast<const __half *>(x), sr, sc, yy, o, rows, cols);
  else sym_dequantize_kernel<int32_t><<<grid, threads, 0, st>>>(static_cast<const int32_t *>(x), sr, sc, yy, o, rows, cols);
  return check_launch("sym_dequantize_kernel");
}

int launch_unpack_int4(const uint8_t *src, int8_t *dst, int rows, int cols, cudaStream_t st) {
  const size_t nbytes = (size_t)rows * (cols / 2);
  if (nbytes == 0) return QUIK_OK;
  const int vec = (nbytes % 16 == 0) && aligned16(src) && aligned16(dst);
  const int threads = 256, grid = ew_grid(vec ? nbytes / 16 : nbytes, threads);
  unpack_int4_kernel<<<grid, threads, 0, st>>>(src, dst, nbytes, vec);
  return check_launch("unpack_int4_kernel");
}

}  // namespace quik
