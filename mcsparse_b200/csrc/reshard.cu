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

// one thread per 16-byte chunk, consecutive threads walk a source row (coalesced reads; writes of a
// segment are contiguous per peer)
__global__ void __launch_bounds__(256) ulysses_scatter_kernel(const uint8_t* __restrict__ src, PeerTable peers, int rank,
                                                              long long rows, int seg_chunks, int row_chunks,
                                                              long long src_row_bytes, long long seg_stride_bytes) {
  const long long total = rows * row_chunks;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long s = t / row_chunks;
    const int c = (int)(t - s * row_chunks);
    const int r = c / seg_chunks;                     // destination peer
    const int cc = c - r * seg_chunks;                // chunk inside the segment
    const uint4 v = *reinterpret_cast<const uint4*>(src + s * src_row_bytes + r * seg_stride_bytes + (size_t)cc * 16);
    *reinterpret_cast<uint4*>(peers.dst[r] + ((long long)rank * rows + s) * ((long long)seg_chunks * 16) + (size_t)cc * 16) = v;
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
  // enough CTAs to fill the GPU several times over, grid-stride for the rest
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ulysses_scatter_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(src), tab, rank, rows, seg_chunks,
                                                               row_chunks, src_row_bytes, seg_stride_bytes);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mcs
