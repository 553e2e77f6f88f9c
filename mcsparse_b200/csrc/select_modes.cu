// Variable-length token selection: how many tokens a query group needs to cover a probability mass.
//
// For every row of fp32 scores (the normalised mass of one query group over all key tokens, sink tokens
// excluded) the kernel returns
//     count = #{ i : sum of all scores ranked strictly before i  <  topp },   ranking by descending score,
// i.e. the length of the shortest prefix of the descending order whose mass reaches topp (everything if the
// whole row stays below it, at least one).  That is the reference's top-p rule
// (mcsparse/kernels/flash_mcsa/token_sparse.py:842-876: sort, cumulative sum, mask cumsum_before < topp, count),
// without sorting: the sum S(x) of all scores above a threshold x falls as x rises, so the boundary value b =
// min{x : S(x) < topp} is found by a search over the order-preserving 32-bit image of the scores (four
// thresholds in every pass over the row, sixteen passes), and one more pass counts the scores above b and those
// equal to it (ties enter one by one until the mass is reached).  A row is read from L2 seventeen times and
// never written; sums are accumulated in fp32 per thread and in fp64 across the CTA in a fixed order, so the
// result is reproducible.  The selection itself (which tokens) is done by the top-k kernel with this count as
// the row's budget.
#include "kernels.cuh"
#include "ptx.cuh"

namespace mcs {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxSinks = 64;

__device__ __forceinline__ uint32_t prob_key(float s) {
  uint32_t u = __float_as_uint(s);
  if (s != s) return 0u;                                   // NaN carries no mass and ranks last
  if (s == 0.f) u = 0u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);       // order-preserving
}
__device__ __forceinline__ float key_value(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(u);
}

struct Shared {
  double sum[3][kWarps];
  unsigned int cnt[3][kWarps];
  int sinks[kMaxSinks];
  double r_sum[3];
  unsigned int r_cnt[3];
};

// block-wide sums of three (count, mass) pairs; the result is in sh.r_* for every thread after the call
__device__ __forceinline__ void reduce3(Shared& sh, const unsigned int (&c)[3], const float (&s)[3]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    unsigned int ci = c[i];
    double si = (double)s[i];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      ci += __shfl_xor_sync(0xffffffffu, ci, off);
      si += __shfl_xor_sync(0xffffffffu, si, off);
    }
    if (lane == 0) { sh.cnt[i][warp] = ci; sh.sum[i][warp] = si; }
  }
  __syncthreads();
  if (threadIdx.x < 3) {
    unsigned int ci = 0;
    double si = 0.0;
    for (int w = 0; w < kWarps; ++w) { ci += sh.cnt[threadIdx.x][w]; si += sh.sum[threadIdx.x][w]; }
    sh.r_cnt[threadIdx.x] = ci;
    sh.r_sum[threadIdx.x] = si;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kThreads) topp_count_kernel(const float* __restrict__ scores, const int32_t* __restrict__ sinks,
                                                             int n_sink, long long rows, int L, float topp, int32_t* __restrict__ counts) {
  __shared__ Shared sh;
  if (threadIdx.x < n_sink) sh.sinks[threadIdx.x] = sinks[threadIdx.x];
  __syncthreads();
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* sc = scores + row * (long long)L;
    // one pass: counts and masses of the scores whose key lies above each of three thresholds
    auto pass = [&](uint32_t t0, uint32_t t1, uint32_t t2, bool eq_mode) {
      unsigned int c[3] = {0, 0, 0};
      float s[3] = {0.f, 0.f, 0.f};
      for (int j = threadIdx.x; j < L; j += kThreads) {
        bool sink = false;
        for (int i = 0; i < n_sink; ++i) sink |= (sh.sinks[i] == j);
        if (sink) continue;
        const float v = __ldg(sc + j);
        const uint32_t k = prob_key(v);
        const float m = (v == v) ? v : 0.f;
        if (!eq_mode) {
          if (k > t0) { ++c[0]; s[0] += m; }
          if (k > t1) { ++c[1]; s[1] += m; }
          if (k > t2) { ++c[2]; s[2] += m; }
        } else {
          if (k > t0) { ++c[0]; s[0] += m; }               // strictly above the boundary
          if (k == t0) ++c[1];                             // equal to it
        }
      }
      reduce3(sh, c, s);
    };
    // b = smallest x with S(x) < topp, S(x) = mass of the scores whose key is above x; S(0xFFFFFFFF) = 0 < topp
    uint32_t lo = 0u, hi = 0xFFFFFFFFu;                     // the answer lies in [lo, hi]
#pragma unroll 1
    while (lo < hi) {
      const uint64_t span = (uint64_t)hi - lo;             // >= 1
      const uint32_t t0 = lo + (uint32_t)(span / 4), t1 = lo + (uint32_t)(span / 2), t2 = lo + (uint32_t)(span / 4 * 3);
      pass(t0, t1, t2, false);
      const bool f0 = sh.r_sum[0] < (double)topp, f1 = sh.r_sum[1] < (double)topp, f2 = sh.r_sum[2] < (double)topp;
      __syncthreads();                                     // everyone has read the results before the next pass overwrites them
      // f is monotone (false ... false true ... true) over x
      if (f0) hi = t0;
      else if (f1) { lo = t0 + 1; hi = t1; }
      else if (f2) { lo = t1 + 1; hi = t2; }
      else lo = t2 + 1;
    }
    const uint32_t b = lo;
    pass(b, 0u, 0u, true);
    if (threadIdx.x == 0) {
      const unsigned int above = sh.r_cnt[0], equal = sh.r_cnt[1];
      const double s_above = sh.r_sum[0];
      const double v = (double)key_value(b);
      unsigned int take = equal;                           // ties enter one by one while the mass before them is below topp
      if (v > 0.0) {
        const double need = ((double)topp - s_above) / v;
        const double cn = ceil(need);
        take = cn < 1.0 ? 1u : (cn > (double)equal ? equal : (unsigned int)cn);
      }
      unsigned int n = above + take;
      if (n < 1u) n = 1u;
      const unsigned int cap = (unsigned int)(L - n_sink);
      counts[row] = (int32_t)(n > cap ? cap : n);
    }
    __syncthreads();
  }
}

}  // namespace

int launch_topp_count(const float* scores, const int32_t* sinks, int n_sink, long long rows, int L, float topp, int32_t* counts,
                      cudaStream_t stream) {
  if (rows == 0) return 0;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long grid = rows < (long long)sms * 4 ? rows : (long long)sms * 4;
  topp_count_kernel<<<(unsigned)grid, kThreads, 0, stream>>>(scores, sinks, n_sink, rows, L, topp, counts);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mcs
