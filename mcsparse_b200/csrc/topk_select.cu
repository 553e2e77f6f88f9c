// Exact top-k token selection with forced sink tokens, one score row per CTA.
//
// For every row of fp32 scores (one query group of one head) the kernel returns, in ascending
// index order, the sink tokens plus the (k_total - n_sink) non-sink tokens with the highest score;
// among equal scores the lowest indices win.  The result depends only on the fp32 scores, so it is
// bit-reproducible and can be compared exactly with a stable sort on the host.
//
// Tightens the reference's selection (mcsparse/kernels/flash_mcsa/token_sparse.py:755-945, topk
// mode with sink ranges): that code calls torch.topk(sorted=False) and then truncates the
// concatenation [sinks, topk] to a multiple of 128, which drops an implementation-defined subset;
// here the dropped entries are the lowest-ranked ones and the output is sorted.
//
// Algorithm per row (1024 threads):
//   1. map scores to order-preserving 32-bit keys (NaN highest; sinks get key 0, below every real
//      key) and stage the row in shared memory when it fits (<= ~200 KB), else re-read it from L2;
//   2. MSB-first radix select, four 8-bit passes with warp-aggregated shared-memory histograms,
//      finds the key T of the k-th largest element and how many elements equal to T are needed;
//   3. one counting sweep and one writing sweep compact the selected indices in index order with
//      warp ballots: element j is taken if it is a sink, or key > T, or key == T and fewer than
//      `need` equal keys precede it.
// The kernel is bandwidth-bound: each score is read once from HBM.
#include "kernels.cuh"
#include "ptx.cuh"

namespace mcs {

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kHistCopies = 8;
constexpr int kMaxSinks = 64;

__device__ __forceinline__ uint32_t score_key(float s) {
  uint32_t u = __float_as_uint(s);
  if (s != s) return 0xFFFFFFFFu;                         // NaN: above every number, as torch.topk ranks it
  if (s == 0.f) u = 0u;                                   // -0 and +0 rank equal
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);          // order-preserving
  return u < 2u ? 2u : u;                                  // keep 0 (sink) and 1 (padding) reserved
}

struct Shared {
  uint32_t hist[kHistCopies][256];
  uint32_t suffix[256];
  int sinks[kMaxSinks];
  int warp_sel[kWarps], warp_eq[kWarps];
  uint32_t prefix;
  int k_rem;
};

template <bool kStage>
__global__ void __launch_bounds__(kThreads, 1) topk_select_kernel(const TopkParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  Shared& sh = *reinterpret_cast<Shared*>(smem_raw);
  uint32_t* skeys = reinterpret_cast<uint32_t*>(smem_raw + sizeof(Shared));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int L = p.L, n_sink = p.n_sink;
  const int k = p.k_total - n_sink;                       // non-sink tokens to pick (>= 0, <= L - n_sink)

  if (tid < n_sink) sh.sinks[tid] = p.sinks[tid];
  __syncthreads();

#pragma unroll 1
  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const float* sc = p.scores + row * (long long)L;
    int32_t* out = p.out + row * (long long)p.k_total;

    auto is_sink = [&](int j) {
      bool s = false;
      for (int i = 0; i < n_sink; ++i) s |= (sh.sinks[i] == j);
      return s;
    };
    auto key_at = [&](int j) -> uint32_t {
      if (kStage) return skeys[j];
      return is_sink(j) ? 0u : score_key(__ldg(sc + j));
    };

    if (kStage) {
      for (int j = tid; j < L; j += kThreads) skeys[j] = score_key(__ldcs(sc + j));
      __syncthreads();
      if (tid < n_sink) skeys[sh.sinks[tid]] = 0u;
    }
    if (tid == 0) { sh.prefix = 0u; sh.k_rem = k; }
    __syncthreads();

    // ---- radix select: key T of the k-th largest non-sink element
    if (k > 0) {
#pragma unroll 1
      for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < kHistCopies * 256; i += kThreads) (&sh.hist[0][0])[i] = 0u;
        __syncthreads();
        const uint32_t prefix = sh.prefix;
        const uint32_t hi_mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
        uint32_t* hist = sh.hist[warp % kHistCopies];
        for (int j0 = warp * 32; j0 < L; j0 += kThreads) {
          const int j = j0 + lane;
          uint32_t key = 0u;
          if (j < L) key = key_at(j);
          const bool live = (j < L) && key != 0u && ((key & hi_mask) == prefix);
          const uint32_t digit = (key >> shift) & 0xFFu;
          // warp-aggregated histogram update: one atomic per distinct digit in the warp
          const uint32_t livemask = __ballot_sync(0xffffffffu, live);
          if (live) {
            const uint32_t peers = __match_any_sync(livemask, digit);
            if ((peers & ((1u << lane) - 1u)) == 0u) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
          }
        }
        __syncthreads();
        // suffix counts over digits: suffix[d] = number of live keys with digit >= d
        if (tid < 256) {
          uint32_t c = 0;
          for (int i = 0; i < kHistCopies; ++i) c += sh.hist[i][tid];
          sh.suffix[tid] = c;
        }
        __syncthreads();
        for (int off = 1; off < 256; off <<= 1) {
          uint32_t v = 0;
          if (tid < 256 && tid + off < 256) v = sh.suffix[tid + off];
          __syncthreads();
          if (tid < 256) sh.suffix[tid] += v;
          __syncthreads();
        }
        if (tid < 256) {
          const uint32_t ge = sh.suffix[tid];
          const uint32_t gt = tid < 255 ? sh.suffix[tid + 1] : 0u;
          const uint32_t kr = (uint32_t)sh.k_rem;
          if (gt < kr && kr <= ge) {                      // exactly one digit satisfies this
            sh.prefix = prefix | ((uint32_t)tid << shift);
            sh.k_rem = (int)(kr - gt);
          }
        }
        __syncthreads();
      }
    }
    const uint32_t T = sh.prefix;
    const int need = k > 0 ? sh.k_rem : 0;                // how many keys == T to take (lowest indices first)

    // ---- counting sweep: per warp span, how many are certainly selected (sink or > T) and how many equal T
    const int span = ((L + kWarps - 1) / kWarps + 31) & ~31;     // contiguous elements per warp, multiple of 32
    const int lo = warp * span, hi = min(lo + span, L);
    int c_sel = 0, c_eq = 0;
    for (int j0 = lo; j0 < hi; j0 += 32) {
      const int j = j0 + lane;
      uint32_t key = 1u;
      if (j < hi) key = key_at(j);
      const bool in = j < hi;
      c_sel += __popc(__ballot_sync(0xffffffffu, in && (key == 0u || (k > 0 && key > T))));
      c_eq += __popc(__ballot_sync(0xffffffffu, in && k > 0 && key == T && key != 0u));
    }
    if (lane == 0) { sh.warp_sel[warp] = c_sel; sh.warp_eq[warp] = c_eq; }
    __syncthreads();
    int eq_before = 0, out_before = 0;
    for (int w = 0; w < warp; ++w) {                       // 32 entries: a serial prefix is cheapest
      const int e = sh.warp_eq[w];
      out_before += sh.warp_sel[w] + min(max(need - eq_before, 0), e);
      eq_before += e;
    }
    // ---- writing sweep
    for (int j0 = lo; j0 < hi; j0 += 32) {
      const int j = j0 + lane;
      uint32_t key = 1u;
      if (j < hi) key = key_at(j);
      const bool in = j < hi;
      const bool eq = in && k > 0 && key == T && key != 0u;
      const uint32_t eq_b = __ballot_sync(0xffffffffu, eq);
      const int eq_rank = eq_before + __popc(eq_b & ((1u << lane) - 1u));
      const bool sel = in && (key == 0u || (k > 0 && key > T) || (eq && eq_rank < need));
      const uint32_t sel_b = __ballot_sync(0xffffffffu, sel);
      if (sel) {
        const int pos = out_before + __popc(sel_b & ((1u << lane) - 1u));
        if (pos < p.k_total) out[pos] = j;
      }
      eq_before += __popc(eq_b);
      out_before += __popc(sel_b);
    }
    __syncthreads();                                       // shared state is reused by the next row
  }
}

}  // namespace

size_t topk_stage_limit_bytes() { return 200 * 1024; }

int launch_topk_select(const TopkParams& p, cudaStream_t stream) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t row_bytes = (size_t)p.L * 4;
  const bool stage = row_bytes <= topk_stage_limit_bytes();
  const size_t smem = sizeof(Shared) + (stage ? row_bytes : 0);
  const int grid = (int)(p.rows < (long long)sms ? p.rows : sms);
  if (stage) {
    if (cudaFuncSetAttribute(topk_select_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -8;
    topk_select_kernel<true><<<grid, kThreads, smem, stream>>>(p);
  } else {
    topk_select_kernel<false><<<grid, kThreads, smem, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mcs
