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

// Sixteen lanes (a half-warp) per token: the half-warp computes the token's grid position and fetches its rotation
// factors and the RMSNorm weights once, then walks the token's head slices two at a time (both 16-byte loads issued
// before either slice is touched).  D = 128: eight elements (four rotation pairs) per lane; D = 64: four elements.
template <int D, bool kFp16>
__global__ void __launch_bounds__(kThreads) qkv_norm_rope_scatter_kernel(const QkvEpilogueParams p, const __grid_constant__ SegTable seg) {
  constexpr int kEl = D / kLanesPerSlice;                  // elements per lane: 8 or 4
  constexpr int kPairs = kEl / 2;
  constexpr int kUnroll = 2;
  const int lane16 = threadIdx.x & 15;
  const uint32_t half_mask = 0xFFFFu << (threadIdx.x & 16);
  const int hw = p.grid_h * p.grid_w;
  const int n_seg = p.n_seg;
  // weights of this lane's elements
  float gq[kEl], gk[kEl];
#pragma unroll
  for (int j = 0; j < kEl; ++j) {
    gq[j] = __ldg(p.gamma_q + lane16 * kEl + j);
    gk[j] = __ldg(p.gamma_k + lane16 * kEl + j);
  }
  const long long step = (long long)gridDim.x * (kThreads / kLanesPerSlice);
  for (long long row = (long long)blockIdx.x * (kThreads / kLanesPerSlice) + (threadIdx.x >> 4); row < p.rows; row += step) {
    // position of the token on the (frames, rows, columns) grid and the (cos, sin) of this lane's rotation pairs:
    // pairs [0, n_t) turn with the frame index, [n_t, n_t + n_h) with the grid row, the rest with the grid column
    const unsigned tok = (unsigned)(p.token0 + row);       // (the C ABI checks that the grid has fewer than 2^31 tokens)
    const int f = (int)(tok / (unsigned)hw);
    const int rem = (int)(tok - (unsigned)f * (unsigned)hw);
    const int y = rem / p.grid_w;
    const int xw = rem - y * p.grid_w;
    float2 cs[kPairs];
#pragma unroll
    for (int j = 0; j < kPairs; ++j) {
      const int pr = lane16 * kPairs + j;
      const int pos = pr < p.pairs_t ? f : (pr < p.pairs_t + p.pairs_h ? p.grid_f + y : p.grid_f + p.grid_h + xw);
      cs[j] = __ldg(p.rope_cs + (size_t)pos * (D / 2) + pr);
    }
    const uint8_t* src_row = reinterpret_cast<const uint8_t*>(p.src) + 2 * (row * p.src_row_stride + lane16 * kEl);
    const long long drow = p.row0 + row;
#pragma unroll 1
    for (int s0 = 0; s0 < n_seg; s0 += kUnroll) {
      uint32_t w[kUnroll][kEl / 2];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (s0 + u < n_seg) {
          const uint8_t* src = src_row + 2 * (size_t)(s0 + u) * D;
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
        const int s = s0 + u;
        if (s >= n_seg) break;                               // (uniform over the half-warp)
        const int kind = seg.kind[s];
        if (kind != 2) {
          float x[kEl];
#pragma unroll
          for (int j = 0; j < kPairs; ++j) {
            const float2 fv = unpack2<kFp16>(w[u][j]);
            x[2 * j] = fv.x;
            x[2 * j + 1] = fv.y;
          }
          float ss = 0.f;
#pragma unroll
          for (int j = 0; j < kEl; ++j) ss = fmaf(x[j], x[j], ss);
          // the sixteen lanes of a slice are a half-warp: xor offsets below 16 stay inside it, and the mask names
          // only that half (the other half works on another token, or on nothing at the end of the grid)
#pragma unroll
          for (int off = 8; off >= 1; off >>= 1) ss += __shfl_xor_sync(half_mask, ss, off);
          const float rinv = rsqrtf(ss * (1.0f / D) + p.eps);
#pragma unroll
          for (int j = 0; j < kPairs; ++j) {
            const float a = x[2 * j] * rinv * (kind == 0 ? gq[2 * j] : gk[2 * j]);
            const float b = x[2 * j + 1] * rinv * (kind == 0 ? gq[2 * j + 1] : gk[2 * j + 1]);
            w[u][j] = pack2<kFp16>(a * cs[j].x - b * cs[j].y, a * cs[j].y + b * cs[j].x);
          }
        }
        uint8_t* dst = seg.dst[s] + 2 * (drow * seg.dst_row_stride[s] + lane16 * kEl);
        if constexpr (kEl == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(w[u][0], w[u][1], w[u][2], w[u][3]);
        else *reinterpret_cast<uint2*>(dst) = make_uint2(w[u][0], w[u][1]);
      }
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
  const long long per_block = kThreads / kLanesPerSlice;
  // one half-warp per token; memory- and link-bound: eight CTAs of 256 threads per SM, grid-stride for the rest
  long long blocks = (p.rows + per_block - 1) / per_block;
  if (blocks > 148 * 8) blocks = 148 * 8;
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
