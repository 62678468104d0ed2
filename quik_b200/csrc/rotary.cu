// Rotary position embedding applied in place to the q and k projections of a decoder block: the step between
// the q/k/v layers and attention (the caller after the quantized layers; QUIK experiments/llama.py leaves it to
// transformers' LlamaAttention).  One pass over q and k: 16-byte loads of the two halves of a head, the
// angle tables read once per token, each product and sum rounded to the storage type like the elementwise torch
// expression  x * cos + rotate_half(x) * sin  rounds them (so results are bit-identical to it).
#include "common.cuh"

namespace quik {
namespace {

template <typename T>
__global__ void rotary_kernel(T *__restrict__ q, T *__restrict__ k, const T *__restrict__ cos_t,
                              const T *__restrict__ sin_t, int tokens, int q_heads, int k_heads, int head_dim) {
  const int half = head_dim / 2, vec_per_head = half / 8, heads = q_heads + k_heads;
  const size_t total = (size_t)tokens * heads * vec_per_head;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const int h = (int)((i / vec_per_head) % heads);
    const int t = (int)(i / ((size_t)vec_per_head * heads));
    T *base = h < q_heads ? q + ((size_t)t * q_heads + h) * head_dim
                          : k + ((size_t)t * k_heads + (h - q_heads)) * head_dim;
    uint4 lo = *reinterpret_cast<const uint4 *>(base + v * 8);
    uint4 hi = *reinterpret_cast<const uint4 *>(base + half + v * 8);
    const uint4 cv = __ldg(reinterpret_cast<const uint4 *>(cos_t + (size_t)t * half + v * 8));
    const uint4 sv = __ldg(reinterpret_cast<const uint4 *>(sin_t + (size_t)t * half + v * 8));
    T *l = reinterpret_cast<T *>(&lo), *u = reinterpret_cast<T *>(&hi);
    const T *c = reinterpret_cast<const T *>(&cv), *s = reinterpret_cast<const T *>(&sv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = Traits<T>::to_float(l[j]), b = Traits<T>::to_float(u[j]);
      const float cc = Traits<T>::to_float(c[j]), ss = Traits<T>::to_float(s[j]);
      // every product of two 11-bit (8-bit) significands is exact in fp32: rounding it to T equals the
      // storage-type multiply; the sums likewise
      const float ac = Traits<T>::to_float(Traits<T>::from_float(__fmul_rn(a, cc)));
      const float nbs = Traits<T>::to_float(Traits<T>::from_float(__fmul_rn(-b, ss)));
      const float bc = Traits<T>::to_float(Traits<T>::from_float(__fmul_rn(b, cc)));
      const float as = Traits<T>::to_float(Traits<T>::from_float(__fmul_rn(a, ss)));
      l[j] = Traits<T>::from_float(__fadd_rn(ac, nbs));
      u[j] = Traits<T>::from_float(__fadd_rn(bc, as));
    }
    *reinterpret_cast<uint4 *>(base + v * 8) = lo;
    *reinterpret_cast<uint4 *>(base + half + v * 8) = hi;
  }
}

}  // namespace

int launch_rotary(void *q, void *k, const void *cos_t, const void *sin_t, int dtype, int tokens, int q_heads,
                  int k_heads, int head_dim, cudaStream_t st) {
  const size_t total = (size_t)tokens * (q_heads + k_heads) * (head_dim / 16);
  if (total == 0) return QUIK_OK;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads, cap = (size_t)num_sms() * 8;
  const int grid = (int)(blocks < cap ? blocks : cap);
  if (dtype == QUIK_F16)
    rotary_kernel<__half><<<grid, threads, 0, st>>>(static_cast<__half *>(q), static_cast<__half *>(k),
                                                     static_cast<const __half *>(cos_t),
                                                     static_cast<const __half *>(sin_t), tokens, q_heads, k_heads,
                                                     head_dim);
  else
    rotary_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(
        static_cast<__nv_bfloat16 *>(q), static_cast<__nv_bfloat16 *>(k), static_cast<const __nv_bfloat16 *>(cos_t),
        static_cast<const __nv_bfloat16 *>(sin_t), tokens, q_heads, k_heads, head_dim);
  return check_launch("rotary_kernel");
}

}  // namespace quik
