// Epilogue of the QKV projection of a context-parallel DiT attention layer, fused with the
// sequence-to-head exchange of Ulysses.
//
// Input: the projection output of `rows` local tokens, `n_seg` head slices of 128 (or 64) elements per
// token (any mix of query, key and value slices; slice s of token i starts at src + i * src_row_stride +
// s * D).  Per slice the kernel
//   * query / key slices: RMS-normalises the slice over its D elements (fp32: x * rsqrt(mean(x^2) + eps) * g[d]),
//     then applies the 3-D rotary embedding of the token's (frame, row, column) position: element pairs
//     (2p, 2p+1) are rotated by the angle of pair p, whose axis and frequency come from a table;
//   * value slices: copies;
// rounds once to the 16-bit type and stores the slice where the attention kernel of the OWNING rank reads
// it: dst[s] + (row0 + i) * dst_row_stride[s] elements, an address in this GPU's memory or in a peer's
// (plain stores over NVLink, 16 bytes per lane, a slice = one 256-byte run).  So the activations go from
// the GEMM output straight into the peers' (L, heads, D) buffers: no separate normalisation pass, no
// rotary pass, no pack copy and no library all-to-all.  Nothing here waits for another GPU; the caller
// orders the launch against the consumers.
//
// The reference runs RMSNorm and RoPE inside the host model and leaves the exchange to diffusers'
// _templated_context_parallel_attention in front of its forward_op (mcsparse/h3/context_parallel.py:
// 165-176, 220-229); this kernel stands for that stretch of the layer.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.cuh"
#include "ptx.cuh"

namespace mcs {
namespace {

constexpr int kThreads = 256;
constexpr int kLanesPerSlice = 16;                         // 16 lanes x 16 bytes = one 128-element 16-bit slice

struct SegTable {
  uint8_t* dst[kQkvMaxSegments];
  long long dst_row_stride[kQkvMaxSegments];               // elements
  int kind[kQkvMaxSegments];                               // 0 query, 1 key, 2 value
};

template <bool kFp16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (kFp16) {
    const __half2 h = *reinterpret_cast<const __half2*>(&u);
    return __half22float2(h);
  } else {
    return make_float2(bf16_lo(u), bf16_hi(u));
  }
}
template <bool kFp16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kFp16) return pack_f16x2(lo, hi);
  else return pack_bf16x2(lo, hi);
}

// D = 128: sixteen lanes per (token, slice), eight elements (four rotation pairs) per lane.  D = 64: the same
// sixteen lanes with four elements each (8-byte accesses).
template <int D, bool kFp16>
__global__ void __launch_bounds__(kThreads) qkv_norm_rope_scatter_kernel(const QkvEpilogueParams p, const __grid_constant__ SegTable seg) {
  constexpr int kEl = D / kLanesPerSlice;                  // elements per lane: 8 or 4
  constexpr int kPairs = kEl / 2;
  constexpr int kUnroll = 4;                               // slices in flight per half-warp: the kernel is bound by memory latency
  const int lane16 = threadIdx.x & 15;
  const long long slices = (long long)p.rows * p.n_seg;
  const long long step = (long long)gridDim.x * (kThreads / kLanesPerSlice);
  const int hw = p.grid_h * p.grid_w;
  const uint32_t half_mask = 0xFFFFu << (threadIdx.x & 16);
  for (long long sl0 = (long long)blockIdx.x * (kThreads / kLanesPerSlice) + (threadIdx.x >> 4); sl0 < slices; sl0 += step * kUnroll) {
    uint32_t w[kUnroll][kEl / 2];
    long long row[kUnroll];
    int seg_i[kUnroll];
    // all loads first
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long sl = sl0 + (long long)u * step;
      seg_i[u] = -1;
      if (sl < slices) {
        row[u] = sl / p.n_seg;
        seg_i[u] = (int)(sl - row[u] * p.n_seg);
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.src) + 2 * (row[u] * p.src_row_stride + (long long)seg_i[u] * D + lane16 * kEl);
        if constexpr (kEl == 8) {
          const uint4 v = *reinterpret_cast<const uint4*>(src);
          w[u][0] = v.x; w[u][1] = v.y; w[u][2] = v.z; w[u][3] = v.w;
        } else {
          const uint2 v = *reinterpret_cast<const uint2*>(src);
          w[u][0] = v.x; w[u][1] = v.y;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (seg_i[u] < 0) continue;                          // (uniform over the half-warp)
      const int s = seg_i[u];
      const int kind = seg.kind[s];
      if (kind != 2) {
        float x[kEl];
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          const float2 f = unpack2<kFp16>(w[u][j]);
          x[2 * j] = f.x;
          x[2 * j + 1] = f.y;
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < kEl; ++j) ss = fmaf(x[j], x[j], ss);
        // the sixteen lanes of a slice are a half-warp: xor offsets below 16 stay inside it, and the mask names
        // only that half (the other half may hold a value slice, or nothing at the end of the grid)
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) ss += __shfl_xor_sync(half_mask, ss, off);
        const float rinv = rsqrtf(ss * (1.0f / D) + p.eps);
        const float* g = (kind == 0 ? p.gamma_q : p.gamma_k) + lane16 * kEl;
        // position of the token on the (frames, rows, columns) grid
        const long long tok = p.token0 + row[u];
        const int f = (int)(tok / hw);
        const int rem = (int)(tok - (long long)f * hw);
        const int y = rem / p.grid_w;
        const int xw = rem - y * p.grid_w;
#pragma unroll
        for (int j = 0; j < kPairs; ++j) {
          const int pr = lane16 * kPairs + j;              // rotation pair inside the slice
          // pairs [0, n_t) turn with the frame index, [n_t, n_t + n_h) with the row, the rest with the column
          const int pos = pr < p.pairs_t ? f : (pr < p.pairs_t + p.pairs_h ? p.grid_f + y : p.grid_f + p.grid_h + xw);
          const float2 cs = __ldg(p.rope_cs + (long long)pos * (D / 2) + pr);
          const float a = x[2 * j] * rinv * g[2 * j];
          const float b = x[2 * j + 1] * rinv * g[2 * j + 1];
          w[u][j] = pack2<kFp16>(a * cs.x - b * cs.y, a * cs.y + b * cs.x);
        }
      }
      uint8_t* dst = seg.dst[s] + 2 * ((p.row0 + row[u]) * seg.dst_row_stride[s] + lane16 * kEl);
      if constexpr (kEl == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(w[u][0], w[u][1], w[u][2], w[u][3]);
      else *reinterpret_cast<uint2*>(dst) = make_uint2(w[u][0], w[u][1]);
    }
  }
}

}  // namespace

int launch_qkv_epilogue(const QkvEpilogueParams& p, void* const* dst, const long long* dst_row_stride, const int* kind,
                        bool fp16, cudaStream_t stream) {
  if (p.n_seg < 1 || p.n_seg > kQkvMaxSegments) return -2;
  if (p.rows == 0) return 0;
  SegTable seg{};
  for (int i = 0; i < p.n_seg; ++i) {
    seg.dst[i] = static_cast<uint8_t*>(dst[i]);
    seg.dst_row_stride[i] = dst_row_stride[i];
    seg.kind[i] = kind[i];
  }
  const long long slices = (long long)p.rows * p.n_seg;
  const long long per_block = kThreads / kLanesPerSlice;
  long long blocks = (slices + per_block * 4 - 1) / (per_block * 4);          // four slices per half-warp and iteration
  // memory- and link-bound: four CTAs of 256 threads per SM are plenty; grid-stride for the rest
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (p.D == 128) {
    if (fp16) qkv_norm_rope_scatter_kernel<128, true><<<(unsigned)blocks, kThreads, 0, stream>>>(p, seg);
    else qkv_norm_rope_scatter_kernel<128, false><<<(unsigned)blocks, kThreads, 0, stream>>>(p, seg);
  } else if (p.D == 64) {
    if (fp16) qkv_norm_rope_scatter_kernel<64, true><<<(unsigned)blocks, kThreads, 0, stream>>>(p, seg);
    else qkv_norm_rope_scatter_kernel<64, false><<<(unsigned)blocks, kThreads, 0, stream>>>(p, seg);
  } else {
    return -3;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mcs
