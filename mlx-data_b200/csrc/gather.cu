// Staging of host sources by a kernel: when the samples of a batch sit in
// page-locked host memory that the GPU can address, a small persistent kernel
// reads exactly the rectangle each chain needs over PCIe and packs it into
// the lane's device arena.  A copy engine moves such a rectangle either as one
// contiguous block of full-width rows (more bytes) or as a strided 2-D copy
// (measured slower per byte than the bus allows); the kernel issues 512-byte
// aligned reads per warp and keeps about a megabyte in flight.
#include "context.h"

namespace mlxd {
namespace {

constexpr int kGatherThreads = 256;
constexpr int kGatherWarps = kGatherThreads / 32;

__global__ void __launch_bounds__(kGatherThreads) gather_host_rows_kernel(const GatherPiece* table, int n, uint32_t total_rows) {
  __shared__ __align__(16) uint8_t buf[kGatherWarps][512];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t n_warps = gridDim.x * kGatherWarps;
  uint8_t* wb = buf[warp];
  int i = 0;
  GatherPiece g = table[0];
  // rows of all pieces form one sequence; this warp takes every n_warps-th
  for (uint32_t t = blockIdx.x * kGatherWarps + warp; t < total_rows; t += n_warps) {
    while (t >= g.first_row + g.rows && i + 1 < n) {
      i++;
      g = table[i];
    }
    const uint32_t r = t - g.first_row;
    const uintptr_t s = reinterpret_cast<uintptr_t>(g.src) + (size_t)r * g.src_pitch;
    uint8_t* d = g.dst + (size_t)r * g.row_bytes;
    // 16-byte units that cover the row: they stay inside the pages the row touches
    const uintptr_t a0 = s & ~(uintptr_t)15;
    const uintptr_t a1 = (s + g.row_bytes + 15) & ~(uintptr_t)15;
    for (uintptr_t a = a0; a < a1; a += 512) {
      const uintptr_t mine = a + 16u * lane;
      if (mine < a1) {
        *reinterpret_cast<uint4*>(wb + 16 * lane) = *reinterpret_cast<const uint4*>(mine);
      }
      __syncwarp();
      const uintptr_t lo = a > s ? a : s;
      const uintptr_t end = s + g.row_bytes;
      const uintptr_t hi = a + 512 < end ? a + 512 : end;
      const uint8_t* from = wb + (lo - a);
      uint8_t* to = d + (lo - s);
      const int count = (int)(hi - lo);
      // head up to a 4-byte boundary of the destination, aligned words, tail
      const int head = min(count, (int)((4 - (reinterpret_cast<uintptr_t>(to) & 3)) & 3));
      if (lane < head) {
        to[lane] = from[lane];
      }
      const int words = (count - head) >> 2;
      const uint8_t* fw = from + head;
      const unsigned sh = (unsigned)(reinterpret_cast<uintptr_t>(fw) & 3) * 8;
      const uint32_t* fa = reinterpret_cast<const uint32_t*>(reinterpret_cast<uintptr_t>(fw) & ~(uintptr_t)3);
      uint32_t* tw = reinterpret_cast<uint32_t*>(to + head);
      for (int w = lane; w < words; w += 32) {
        const uint32_t x0 = fa[w];
        // the word after the last one of the buffer is never needed when sh == 0
        const uint32_t x1 = sh ? fa[w + 1] : 0u;
        tw[w] = __funnelshift_r(x0, x1, sh);
      }
      const int done = head + 4 * words;
      if (lane < count - done) {
        to[done + lane] = from[done + lane];
      }
      __syncwarp();
    }
  }
}

} // namespace

cudaError_t launch_gather_rows(const GatherPiece* table_dev, int n, uint32_t total_rows, cudaStream_t stream) {
  if (n <= 0 || total_rows == 0) {
    return cudaSuccess;
  }
  static thread_local int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
      return e;
    }
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      return e;
    }
  }
  // two CTAs per SM: 16 warps x 512 bytes in flight each, and room left for
  // the batch kernels of the other lanes
  unsigned blocks = (unsigned)sm_count * 2;
  const unsigned need = (total_rows + kGatherWarps - 1) / kGatherWarps;
  blocks = blocks < need ? blocks : need;
  gather_host_rows_kernel<<<blocks, kGatherThreads, 0, stream>>>(table_dev, n, total_rows);
  return cudaGetLastError();
}

} // namespace mlxd
