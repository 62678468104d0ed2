// Strided device-to-device copy on the SMs: rows x width_bytes with independent pitches, 16 bytes per access,
// several loads in flight per thread.  Source or destination may be a peer GPU's memory mapped into this process
// (plain loads and stores over NVLink).  The copy-engine form of the same copy is cudaMemcpy2DAsync; this kernel
// exists because the copy engines slow down on short rows (8 GPUs, rows of 2 KB: under 200 GB/s per rank).
// Peer memory is read with cache-volatile loads: the same addresses are read again in later launches after the peer
// has rewritten them.
#include "common.cuh"

namespace quik {
namespace {

// Small CTAs with few registers: they fit beside a resident CTA of the layer kernels (which leave about 6000 registers
// of an SM free), so the copies run while those kernels do.
constexpr int PC_THREADS = 128, PC_UNROLL = 4;

__device__ __forceinline__ uint4 ld_cv(const void *p) {
  uint4 v;
  asm volatile("ld.global.cv.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__global__ void __launch_bounds__(PC_THREADS, 12)
peer_copy_2d_kernel(uint8_t *__restrict__ dst, size_t dst_pitch, const uint8_t *__restrict__ src, size_t src_pitch,
                    unsigned vec_per_row, size_t total_vec) {
  const size_t stride = (size_t)gridDim.x * PC_THREADS;
  size_t i = (size_t)blockIdx.x * PC_THREADS + threadIdx.x;
  for (; i + (PC_UNROLL - 1) * stride < total_vec; i += PC_UNROLL * stride) {
    uint4 v[PC_UNROLL];
    size_t off_d[PC_UNROLL];
#pragma unroll
    for (int u = 0; u < PC_UNROLL; ++u) {
      const size_t j = i + u * stride;
      const size_t r = j / vec_per_row, c = j - r * vec_per_row;
      v[u] = ld_cv(src + r * src_pitch + c * 16);
      off_d[u] = r * dst_pitch + c * 16;
    }
#pragma unroll
    for (int u = 0; u < PC_UNROLL; ++u) *reinterpret_cast<uint4 *>(dst + off_d[u]) = v[u];
  }
  for (; i < total_vec; i += stride) {
    const size_t r = i / vec_per_row, c = i - r * vec_per_row;
    *reinterpret_cast<uint4 *>(dst + r * dst_pitch + c * 16) = ld_cv(src + r * src_pitch + c * 16);
  }
}

}  // namespace

int launch_peer_copy_2d(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes,
                        size_t rows, int ctas, cudaStream_t st) {
  const size_t vec_per_row = width_bytes / 16, total = vec_per_row * rows;
  if (total == 0) return QUIK_OK;
  size_t need = (total + PC_THREADS - 1) / PC_THREADS;
  int grid = ctas > 0 ? ctas : 64;
  if ((size_t)grid > need) grid = (int)need;
  peer_copy_2d_kernel<<<grid, PC_THREADS, 0, st>>>(static_cast<uint8_t *>(dst), dst_pitch,
                                                   static_cast<const uint8_t *>(src), src_pitch,
                                                   (unsigned)vec_per_row, total);
  return check_launch("peer_copy_2d_kernel");
}

}  // namespace quik
