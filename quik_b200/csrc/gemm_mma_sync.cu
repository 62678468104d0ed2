// int8 x int8 -> int32 GEMM on the legacy warp-level tensor path (mma.sync.m16n8k32.s8).
//
// This is the comparison engine for the tcgen05 kernel (same operands, same epilogue) and the
// engine for shapes or devices where the tcgen05 path is switched off.  C[m,n] = sum_k A[m,k] *
// B[n,k]; A [M,K] and B [N,K] are both K-contiguous (QUIK src/matmul/matmul.cu:98-136).
// CTA tile 128x128x64, 8 warps of 64x32, cp.async double buffering, padded shared rows.
#include "common.cuh"

namespace quik {
namespace {

constexpr int BM = 128, BN = 128, BK = 64, PITCH = BK + 16, THREADS = 256;

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;   // src-size 0 -> the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename T>
__device__ __forceinline__ float ld_f(const void *p, size_t i) {
  return Traits<T>::to_float(static_cast<const T *>(p)[i]);
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
gemm_mma_sync_kernel(const int8_t *__restrict__ A, const int8_t *__restrict__ B, int M, int N, int K,
                     Epilogue ep) {
  __shared__ __align__(16) int8_t sA[2][BM][PITCH];
  __shared__ __align__(16) int8_t sB[2][BN][PITCH];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;                // 2 x 4 warps
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int nk = (K + BK - 1) / BK;

  auto load_stage = [&](int stage, int kb) {
    const int k0 = kb * BK;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * THREADS;                   // 512 chunks of 16 bytes per operand
      const int row = c >> 2, kc = (c & 3) * 16;
      const bool kin = (k0 + kc) < K;
      const bool va = kin && (m0 + row) < M, vb = kin && (n0 + row) < N;
      cp_async16(&sA[stage][row][kc], A + (size_t)(va ? m0 + row : 0) * K + (va ? k0 + kc : 0), va);
      cp_async16(&sB[stage][row][kc], B + (size_t)(vb ? n0 + row : 0) * K + (vb ? k0 + kc : 0), vb);
    }
    cp_async_commit();
  };

  int acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[i][j][r] = 0;

  load_stage(0, 0);
  for (int kb = 0; kb < nk; ++kb) {
    const int cur = kb & 1;
    if (kb + 1 < nk) {
      load_stage(cur ^ 1, kb + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < BK; ks += 32) {
      uint32_t af[4][4], bf[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = wm * 64 + i * 16 + g;
        af[i][0] = *reinterpret_cast<const uint32_t *>(&sA[cur][r][ks + 4 * t]);
        af[i][1] = *reinterpret_cast<const uint32_t *>(&sA[cur][r + 8][ks + 4 * t]);
        af[i][2] = *reinterpret_cast<const uint32_t *>(&sA[cur][r][ks + 16 + 4 * t]);
        af[i][3] = *reinterpret_cast<const uint32_t *>(&sA[cur][r + 8][ks + 16 + 4 * t]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = wn * 32 + j * 8 + g;
        bf[j][0] = *reinterpret_cast<const uint32_t *>(&sB[cur][c][ks + 4 * t]);
        bf[j][1] = *reinterpret_cast<const uint32_t *>(&sB[cur][c][ks + 16 + 4 * t]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_s8(acc[i][j], af[i], bf[j]);
    }
    __syncthreads();
  }

  // ---- epilogue: c0,c1 -> (row g, cols 2t, 2t+1); c2,c3 -> (row g+8, same cols)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = m0 + wm * 64 + i * 16 + g + h * 8;
      if (row >= M) continue;
      float srow = 0.f, zrow = 0.f;
      if (ep.mode == 1) {
        if (ep.meta) {
          srow = ld_f<T>(ep.meta, 2 * (size_t)row);
          zrow = ld_f<T>(ep.meta, 2 * (size_t)row + 1);
        } else {
          srow = ld_f<T>(ep.scale_row, row);
          zrow = ep.zero_row ? ld_f<T>(ep.zero_row, row) : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = n0 + wn * 32 + j * 8 + 2 * t + e;
          if (col >= N) continue;
          const int v = acc[i][j][2 * h + e];
          const size_t off = (size_t)row * N + col;
          if (ep.mode == 0) {
            ep.C[off] = v;
          } else {
            // same fused multiply-add formula as the tcgen05 engine's epilogue
            const float scol = ld_f<T>(ep.scale_col, col);
            float add = ep.y ? ld_f<T>(ep.y, off) : 0.f;
            if (ep.bias) add += ld_f<T>(ep.bias, col);
            if (ep.w_reduced) add = fmaf(fmaf(ep.shift_value, srow, zrow), ld_f<T>(ep.w_reduced, col), add);
            const float r = fmaf((float)v, srow * scol, add);
            static_cast<T *>(ep.out)[(size_t)row * (ep.ldo > 0 ? ep.ldo : N) + col] = Traits<T>::from_float(r);
          }
        }
      }
    }
  }
}

}  // namespace

int launch_gemm_mma_sync(const int8_t *A, const int8_t *B, int M, int N, int K, const Epilogue &ep,
                         cudaStream_t st) {
  if (M == 0 || N == 0) return QUIK_OK;
  if (ep.fp_a != nullptr && ep.F > 0) return QUIK_ERR_UNSUPPORTED;   // outlier GEMM: tcgen05 engine only
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return QUIK_ERR_UNSUPPORTED;
  if (ep.dtype == QUIK_BF16)
    gemm_mma_sync_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(A, B, M, N, K, ep);
  else
    gemm_mma_sync_kernel<__half><<<grid, THREADS, 0, st>>>(A, B, M, N, K, ep);
  return check_launch("gemm_mma_sync_kernel");
}

}  // namespace quik
