// Sequence-to-head reshard of Ulysses context parallelism by peer stores.
//
// Every rank holds a sequence shard x[rows, all heads] (rows = L / N tokens) and needs, for its own
// heads, all tokens: y[N * rows, seg] (seg = the bytes of the wanted heads of one token: all H / N
// local heads, or a chunk of them).  Rank `rank` therefore writes, for every peer r and every local row s,
//     dst_peers[r][(rank * rows + s) * seg  ...  + seg)  =  x[s * src_row_bytes + r * seg_stride ... + seg)
// straight into the peers' buffers (NVLink stores to mapped peer memory; the own block is a local
// copy).  One pass over the shard, no pack copy, no library collective; the launches of all ranks
// are ordered against their consumers by whatever the caller uses between kernels (a stream-ordered
// collective of the communication library), so nothing here waits for another GPU.
//
// Replaces the all-to-all that diffusers' _templated_context_parallel_attention issues in front of the
// reference's forward_op (mcsparse/h3/context_parallel.py:220-229).
#include "kernels.cuh"

namespace mcs {
namespace {

constexpr int kMaxPeers = 16;

struct PeerTable {
  uint8_t* dst[kMaxPeers];
};

// One thread moves kUnroll 16-byte chunks per iteration (loads first, then the stores: kUnroll requests in
// flight per thread); consecutive threads walk a source row, so reads are coalesced and the writes of a segment
// are contiguous per peer.  Two CTAs of 128 threads per SM keep enough stores in flight for the link rate (the
// exchange is bound by NVLink, not by the SMs).  The kernel cannot share an SM with the attention kernel, whose
// CTA leaves no sub-partition enough registers for another warp: chunks exchanged under a running attention
// kernel go through launch_ulysses_scatter_dma instead.
constexpr int kScatterThreads = 128;
constexpr int kUnroll = 4;

template <typename Index>
__global__ void __launch_bounds__(kScatterThreads, 4) ulysses_scatter_kernel(const uint8_t* __restrict__ src, const __grid_constant__ PeerTable peers,
                                                                             int rank, long long rows, int seg_chunks,
                                                                             int row_chunks, long long src_row_bytes,
                                                                             long long seg_stride_bytes) {
  const Index total = (Index)rows * (Index)row_chunks;
  const Index step = (Index)gridDim.x * kScatterThreads;
  const long long dst_row_bytes = (long long)seg_chunks * 16;
  for (Index t0 = (Index)blockIdx.x * kScatterThreads + threadIdx.x; t0 < total; t0 += step * kUnroll) {
    uint4 v[kUnroll];
    uint8_t* dst[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const Index t = t0 + (Index)u * step;
      dst[u] = nullptr;
      if (t < total) {
        const Index s = t / (Index)row_chunks;
        const int c = (int)(t - s * (Index)row_chunks);
        const int r = c / seg_chunks;                     // destination peer
        const int cc = c - r * seg_chunks;                // chunk inside the segment
        v[u] = *reinterpret_cast<const uint4*>(src + (long long)s * src_row_bytes + r * seg_stride_bytes + (size_t)cc * 16);
        dst[u] = peers.dst[r] + ((long long)rank * rows + (long long)s) * dst_row_bytes + (size_t)cc * 16;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (dst[u] != nullptr) *reinterpret_cast<uint4*>(dst[u]) = v[u];
  }
}

}  // namespace

int launch_ulysses_scatter(const void* src, void* const* dst_peers, int n_peers, int rank, long long rows,
                           long long seg_bytes, long long seg_stride_bytes, long long src_row_bytes, cudaStream_t stream) {
  if (n_peers < 1 || n_peers > kMaxPeers) return -2;
  PeerTable tab{};
  for (int i = 0; i < n_peers; ++i) tab.dst[i] = static_cast<uint8_t*>(dst_peers[i]);
  const int seg_chunks = (int)(seg_bytes / 16);
  const int row_chunks = seg_chunks * n_peers;
  const long long total = rows * row_chunks;
  if (total == 0) return 0;
  // two CTAs per SM (see the kernel), grid-stride for the rest
  const long long per_block = (long long)kScatterThreads * kUnroll;
  long long blocks = (total + per_block - 1) / per_block;
  if (blocks > 148 * 2) blocks = 148 * 2;
  const uint8_t* s8 = static_cast<const uint8_t*>(src);
  if (total + (long long)blocks * per_block < (1ll << 32))
    ulysses_scatter_kernel<uint32_t><<<(unsigned)blocks, kScatterThreads, 0, stream>>>(s8, tab, rank, rows, seg_chunks, row_chunks,
                                                                                      src_row_bytes, seg_stride_bytes);
  else
    ulysses_scatter_kernel<unsigned long long><<<(unsigned)blocks, kScatterThreads, 0, stream>>>(
        s8, tab, rank, rows, seg_chunks, row_chunks, src_row_bytes, seg_stride_bytes);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// The same reshard on the copy engines: one strided 2-D device copy per peer (rows x seg_bytes, source pitch =
// the token stride, destination packed).  The attention kernel keeps one CTA per SM with nearly all registers,
// so a scatter kernel launched beside it cannot become resident; DMA copies can run under it.
int launch_ulysses_scatter_dma(const void* src, void* const* dst_peers, int n_peers, int rank, long long rows,
                               long long seg_bytes, long long seg_stride_bytes, long long src_row_bytes, cudaStream_t stream) {
  if (n_peers < 1 || n_peers > kMaxPeers) return -2;
  if (rows == 0) return 0;
  const uint8_t* s8 = static_cast<const uint8_t*>(src);
  for (int i = 0; i < n_peers; ++i) {
    // start with the next rank, so that the ranks do not all write to the same peer first
    const int r = (rank + 1 + i) % n_peers;
    uint8_t* dst = static_cast<uint8_t*>(dst_peers[r]) + (long long)rank * rows * seg_bytes;
    if (cudaMemcpy2DAsync(dst, (size_t)seg_bytes, s8 + (long long)r * seg_stride_bytes, (size_t)src_row_bytes,
                          (size_t)seg_bytes, (size_t)rows, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
      return -8;
  }
  return 0;
}

}  // namespace mcs
