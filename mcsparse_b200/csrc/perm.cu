// Row permutation of (batch*head, L, D) tensors: the data movement around Fast PDDP when it is not
// fused into the attention kernel.
//
//   apply : out[bh, i, :] = x[bh, perm[bh, i], :]          (pca_group.py:40-42, apply_perm)
//   invert: out[bh, perm[bh, i], :] = x[bh, i, :]          (pca_group.py:45-49, invert_perm)
//
// The reference inverts with perm.argsort() followed by a gather; scattering through perm gives
// the same result without the sort.  Pure bandwidth kernels: 16-byte accesses, one row per group
// of (row_bytes / 16) lanes, grid sized to cover the rows once.
#include "kernels.cuh"

namespace mcs {
namespace {

template <bool kInvert>
__global__ void __launch_bounds__(256) perm_rows_kernel(const uint8_t* x, uint8_t* out, const long long* perm, long long rows_total,
                                                        int L, int chunks, long long x_bh, long long x_row, long long o_bh,
                                                        long long o_row) {
  // one thread per 16-byte chunk
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long r = t / chunks;
  const int c = (int)(t % chunks);
  if (r >= rows_total) return;
  const long long bh = r / L;
  const int i = (int)(r % L);
  const long long j = perm[r];
  const long long src_row = kInvert ? i : j, dst_row = kInvert ? j : i;
  const uint4 v = *reinterpret_cast<const uint4*>(x + bh * x_bh + src_row * x_row + (size_t)c * 16);
  *reinterpret_cast<uint4*>(out + bh * o_bh + dst_row * o_row + (size_t)c * 16) = v;
}

}  // namespace

int launch_perm_rows(const void* x, void* out, const long long* perm, int BH, int L, int row_bytes, long long x_bh, long long x_row,
                     long long o_bh, long long o_row, bool invert, cudaStream_t stream) {
  const int chunks = row_bytes / 16;
  const long long rows = (long long)BH * L;
  const long long threads = rows * chunks;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  if (invert)
    perm_rows_kernel<true><<<grid, 256, 0, stream>>>((const uint8_t*)x, (uint8_t*)out, perm, rows, L, chunks, x_bh, x_row, o_bh, o_row);
  else
    perm_rows_kernel<false><<<grid, 256, 0, stream>>>((const uint8_t*)x, (uint8_t*)out, perm, rows, L, chunks, x_bh, x_row, o_bh, o_row);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

namespace {
// 17-bit token indices (sequences of up to 131,072 keys) as 16 bits + one bit: 272 instead of 512 bytes per tile of 128.
__global__ void __launch_bounds__(256) index_pack17_kernel(const int32_t* __restrict__ gi, long long n, uint16_t* __restrict__ lo,
                                                           uint32_t* __restrict__ hi) {
  const long long i0 = ((long long)blockIdx.x * 256 + threadIdx.x);
  const long long step = (long long)gridDim.x * 256;
  for (long long i = i0; i < n + 31; i += step) {                  // whole warps: n is a multiple of 32
    const int v = i < n ? gi[i] : 0;
    const unsigned b = __ballot_sync(0xffffffffu, (v >> 16) & 1);
    if (i < n) {
      lo[i] = (uint16_t)(v & 0xFFFF);
      if ((threadIdx.x & 31) == 0) hi[i >> 5] = b;
    }
  }
}
__global__ void __launch_bounds__(256) index_unpack17_kernel(const uint16_t* __restrict__ lo, const uint32_t* __restrict__ hi, long long n,
                                                             int32_t* __restrict__ gi) {
  const long long step = (long long)gridDim.x * 256;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += step)
    gi[i] = (int)lo[i] | (int)(((hi[i >> 5] >> (i & 31)) & 1u) << 16);
}
}  // namespace

int launch_index_pack17(const int32_t* gi, long long n, uint16_t* lo, uint32_t* hi, cudaStream_t stream) {
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  index_pack17_kernel<<<(unsigned)blocks, 256, 0, stream>>>(gi, n, lo, hi);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}
int launch_index_unpack17(const uint16_t* lo, const uint32_t* hi, long long n, int32_t* gi, cudaStream_t stream) {
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  index_unpack17_kernel<<<(unsigned)blocks, 256, 0, stream>>>(lo, hi, n, gi);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mcs
