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

  if (tid < n_sink) sh.sinks[tid] = p.sinks[tid];
  __syncthreads();

#pragma unroll 1
  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const float* sc = p.scores + row * (long long)L;
    int32_t* out = p.out + row * (long long)p.k_total;
    // this row's budget (sinks included): the common k_total, or its own entry of k_rows
    const int k_row = p.k_rows != nullptr ? min(max(p.k_rows[row], n_sink), p.k_total) : p.k_total;
    const int k = k_row - n_sink;                         // non-sink tokens to pick (>= 0, <= L - n_sink)

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
        if (pos < k_row) out[pos] = j;
      }
      eq_before += __popc(eq_b);
      out_before += __popc(sel_b);
    }
    for (int i = k_row + tid; i < p.k_total; i += kThreads) out[i] = 0;      // beyond the row's own budget: padding
    __syncthreads();                                       // shared state is reused by the next row
  }
}


constexpr int kKpt = 64;                 // keys per thread
constexpr int kRT = 512;                 // threads of the register-resident kernel (128 registers each: 64 keys + state)
constexpr int kRW = kRT / 32;
constexpr int kCandCap = 8192;           // candidate keys held in shared memory

struct SharedReg {
  uint32_t hist[kHistCopies][256];
  uint32_t suffix[256];
  uint32_t warp_tot[2][32];
  uint32_t prefix;
  int k_rem;
  uint32_t block_tot[2];
};

// Radix select over the keys a thread enumerates with `key_of(it, valid)` for it in [0, iters):
// returns through sh.prefix / sh.k_rem the key of the k-th largest key != 0 and how many keys
// equal to it are needed.  All threads of the CTA call it with the same iters and k >= 1.
template <int kPasses = 4, typename KeyOf>
__device__ __forceinline__ void radix_select_kth(SharedReg& sh, int iters, int k, KeyOf key_of) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Three block-wide barriers per pass: a barrier of 32 warps costs a few hundred cycles, and a version
  // with a shared-memory suffix scan (twenty barriers per pass) spent most of its time in them.
  uint32_t prefix = 0u;
  int k_rem = k;
#pragma unroll 1
  for (int pass = 0; pass < kPasses; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < kHistCopies * 256; i += kRT) (&sh.hist[0][0])[i] = 0u;
    __syncthreads();
    const uint32_t hi_mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    uint32_t* hist = sh.hist[warp % kHistCopies];
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
      bool valid = false;
      const uint32_t key = key_of(it, valid);
      const bool live = valid && key != 0u && ((key & hi_mask) == prefix);
      const uint32_t digit = (key >> shift) & 0xFFu;
      const uint32_t livemask = __ballot_sync(0xffffffffu, live);
      if (live) {
        const uint32_t peers = __match_any_sync(livemask, digit);
        if ((peers & ((1u << lane) - 1u)) == 0u) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
      }
    }
    __syncthreads();
    if (warp == 0) {
      // lane l owns digits 8l .. 8l+7: counts, suffix sums inside the lane, then across lanes by shuffles
      uint32_t c[8];
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        uint32_t v = 0;
#pragma unroll
        for (int i = 0; i < kHistCopies; ++i) v += sh.hist[i][8 * lane + d];
        c[d] = v;
      }
      uint32_t lane_sum = 0;
#pragma unroll
      for (int d = 0; d < 8; ++d) lane_sum += c[d];
      uint32_t above = lane_sum;                              // inclusive suffix over lanes >= this one
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t n = __shfl_down_sync(0xffffffffu, above, off);
        if (lane + off < 32) above += n;
      }
      uint32_t gt = above - lane_sum;                         // keys with a digit in a higher lane
      const uint32_t kr = (uint32_t)k_rem;
#pragma unroll
      for (int d = 7; d >= 0; --d) {
        const uint32_t ge = gt + c[d];
        if (gt < kr && kr <= ge) {                            // exactly one digit of one lane satisfies this
          sh.prefix = prefix | ((uint32_t)(8 * lane + d) << shift);
          sh.k_rem = (int)(kr - gt);
        }
        gt = ge;
      }
    }
    __syncthreads();
    prefix = sh.prefix;
    k_rem = sh.k_rem;
  }
  __syncthreads();                                            // everyone has read the result: callers may reuse sh
}

// Exclusive block-wide scan of one 32-bit value per thread (two 16-bit counters packed, or one
// counter); returns this thread's exclusive prefix and the block total.  Two barriers; consecutive
// calls must alternate `parity` (the scratch is double-buffered instead of fenced by a third barrier).
__device__ __forceinline__ uint32_t block_scan_excl(SharedReg& sh, uint32_t v, uint32_t& total, int parity) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t incl = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  if (lane == 31) sh.warp_tot[parity][warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const uint32_t w = lane < kRW ? sh.warp_tot[parity][lane] : 0u;
    uint32_t wi = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, wi, off);
      if (lane >= off) wi += n;
    }
    if (lane < kRW) sh.warp_tot[parity][lane] = wi - w;  // exclusive prefix of the warp totals
    if (lane == 31) sh.block_tot[parity] = wi;
  }
  __syncthreads();
  total = sh.block_tot[parity];
  return sh.warp_tot[parity][warp] + incl - v;
}

// position of score j inside the staging row: 16-byte chunks XOR-swizzled so that the coalesced fill
// (consecutive threads, consecutive chunks) and the per-thread read of 16 consecutive chunks are both
// free of bank conflicts
__device__ __forceinline__ int stage_pos(int j) {
  const int c = j >> 2;
  return ((c ^ ((c >> 4) & 7)) << 2) | (j & 3);
}

template <bool kVec>
__global__ void __launch_bounds__(kRT, 1) topk_select_reg_kernel(const TopkParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  SharedReg& sh = *reinterpret_cast<SharedReg*>(smem_raw);
  uint32_t* ckeys = reinterpret_cast<uint32_t*>(smem_raw + sizeof(SharedReg));
  float* stage = reinterpret_cast<float*>(ckeys + kCandCap);             // one row of scores, swizzled
  const int tid = threadIdx.x;
  const int L = p.L, n_sink = p.n_sink;
  const int j0 = tid * kKpt;                                             // this thread owns scores [j0, j0 + 32)

  // The next row streams into shared memory (cp.async) while the current one is processed out of
  // registers, so the HBM latency of a row is not exposed between rows.
  auto fetch = [&](long long row) {
    const float* sc = p.scores + row * (long long)L;
    if (kVec) {
      const uint32_t sbase = smem_u32(stage);
      for (int c = tid; 4 * c < L; c += kRT)                       // L % 4 == 0 on this path
        cp_async16(sbase + 16u * (uint32_t)(c ^ ((c >> 4) & 7)), sc + 4 * c);
    } else {
      for (int j = tid; j < L; j += kRT) stage[stage_pos(j)] = __ldcs(sc + j);
    }
  };
  if (blockIdx.x < p.rows) fetch(blockIdx.x);
  // sinks owned by this thread, as a bit mask over its 64 slots (the sink list is the same for every row)
  unsigned long long sink_mask = 0ull;
  for (int s = 0; s < n_sink; ++s) {
    const int js = p.sinks[s];
    if ((js >> 6) == tid) sink_mask |= 1ull << (js & 63);
  }

#pragma unroll 1
  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    int32_t* out = p.out + row * (long long)p.k_total;
    const int k_row = p.k_rows != nullptr ? min(max(p.k_rows[row], n_sink), p.k_total) : p.k_total;
    const int k = k_row - n_sink;
    cp_async_wait_all();
    __syncthreads();
    // ---- keys into registers: slot q holds score j0 + q; padding beyond L gets the lowest key
    uint32_t key[kKpt];
#pragma unroll
    for (int i = 0; i < kKpt / 4; ++i) {
      // (the barrier keeps the compiler from hoisting all sixteen loads above the conversions, which
      // would need 64 more registers than there are)
      if ((i & 3) == 0) asm volatile("" ::: "memory");
      const int c = (j0 >> 2) + i;
      const float4 f = *reinterpret_cast<const float4*>(stage + 4 * (c ^ ((c >> 4) & 7)));
      const float fv[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t kq = (4 * c + e < L) ? score_key(fv[e]) : 1u;
        key[4 * i + e] = ((sink_mask >> (4 * i + e)) & 1ull) ? 0u : kq;      // sinks: key 0, always selected, never counted
      }
    }
    __syncthreads();                                                     // the staging row is free again
    if (row + gridDim.x < p.rows) fetch(row + gridDim.x);
    uint32_t T = 0u;
    int need = 0;
    if (k > 0) {
      // ---- 1. conservative lower bound from a 1024-key sample
      uint32_t t_lo = 1u;                 // 1 = every key that is not a sink (padding ranks lowest)
      // sample: slots 0 and 32 of every thread (every 32nd score, 1024 keys); the rank aimed at is the expected
      // rank of the k-th key plus 4.5 standard deviations of its sampling noise, and only the upper 16 bits of
      // the sample quantile are resolved (the bound only has to be below the answer, not exact)
      const long long exp_rank = ((long long)k * 2 * kRT + L - 1) / L;
      const long long r_s = exp_rank + (long long)(4.5f * sqrtf((float)exp_rank)) + 4;
      if (r_s < kRT) {
        const uint32_t s0 = key[0] > 1u ? key[0] : 0u, s1 = key[32] > 1u ? key[32] : 0u;
        radix_select_kth<2>(sh, 2, (int)r_s, [&](int it, bool& valid) { valid = true; return it == 0 ? s0 : s1; });
        t_lo = sh.prefix < 1u ? 1u : sh.prefix;
      }
      // ---- 2. count the keys >= t_lo and > t_lo.  If at least k are strictly greater, those are the
      // candidates; if not, but at least k are >= t_lo, the k-th largest IS t_lo (a tie group sits on the
      // bound - common for masses that underflow to zero) and nothing is left to select; otherwise the
      // sample misjudged the row and every key becomes a candidate.
      uint32_t total_gt = 0;
      int par = 0;
      bool selected = false;
      while (true) {
        uint32_t ge = 0, gt = 0;
#pragma unroll
        for (int q = 0; q < kKpt; ++q) {
          ge += (key[q] >= t_lo) ? 1u : 0u;                  // sinks (key 0) are never candidates
          gt += (key[q] > t_lo) ? 1u : 0u;
        }
        uint32_t tot;
        const uint32_t base = block_scan_excl(sh, ge | (gt << 16), tot, par);
        par ^= 1;
        const uint32_t total_ge = tot & 0xFFFFu;
        total_gt = tot >> 16;
        if ((int)total_gt >= k) {
          if (total_gt <= (uint32_t)kCandCap) {
            uint32_t w = base >> 16;
#pragma unroll
            for (int q = 0; q < kKpt; ++q)
              if (key[q] > t_lo) ckeys[w++] = key[q];
          }
          break;
        }
        if ((int)total_ge >= k) {
          T = t_lo;
          need = k - (int)total_gt;
          selected = true;
          break;
        }
        t_lo = 1u;                                           // the sample misjudged this row
      }
      __syncthreads();
      // ---- 3. exact k-th largest among the candidates
      if (!selected) {
        if (total_gt <= (uint32_t)kCandCap) {
          const int C = (int)total_gt;
          radix_select_kth(sh, (C + kRT - 1) / kRT, k, [&](int it, bool& valid) {
            const int j = it * kRT + tid;
            valid = j < C;
            return valid ? ckeys[j] : 0u;
          });
        } else {
          // too many candidates for shared memory (the sampled bound failed badly): select over the row as
          // it lies in global memory
          const float* sc = p.scores + row * (long long)L;
          radix_select_kth(sh, (L + kRT - 1) / kRT, k, [&](int it, bool& valid) {
            const int j = it * kRT + tid;
            valid = j < L;
            if (!valid) return 0u;
            bool sink = false;
            for (int s2 = 0; s2 < n_sink; ++s2) sink |= (p.sinks[s2] == j);
            return sink ? 0u : score_key(__ldg(sc + j));
          });
        }
        T = sh.prefix;
        need = sh.k_rem;
      }
    }

    // ---- 4. write-out in index order: one block-wide scan of (certainly selected, equal to T) counts.
    // The per-thread result is kept as two 64-bit masks over its slots, so the write loop below only
    // visits the few selected slots and needs no key any more.
    // (padding keys are 1 and T, a real key, is at least 2, so no range check is needed; sinks are in sink_mask)
    unsigned long long sel_mask = sink_mask, eq_mask = 0ull;
    if (k > 0) {
#pragma unroll
      for (int q = 0; q < kKpt; ++q) {
        const uint32_t kq = key[q];
        if (kq > T) sel_mask |= 1ull << q;
        if (kq == T) eq_mask |= 1ull << q;
      }
    }
    const uint32_t sel = (uint32_t)__popcll(sel_mask), eq = (uint32_t)__popcll(eq_mask);
    uint32_t tot;
    const uint32_t pre = block_scan_excl(sh, sel | (eq << 16), tot, 0);
    const uint32_t sel_pre = pre & 0xFFFFu, eq_pre = pre >> 16;
    // position of an element = certainly-selected before it + min(equal before it, need)
    unsigned long long m = sel_mask | eq_mask;
    while (m != 0ull) {
      const int q = __ffsll((long long)m) - 1;
      m &= m - 1ull;
      const unsigned long long below = (1ull << q) - 1ull;
      const uint32_t s_b = sel_pre + (uint32_t)__popcll(sel_mask & below);
      const uint32_t e_b = eq_pre + (uint32_t)__popcll(eq_mask & below);
      const bool is_eq = (eq_mask >> q) & 1ull;
      if (!is_eq || e_b < (uint32_t)need) {
        const uint32_t pos = s_b + min(e_b, (uint32_t)need);
        if (pos < (uint32_t)k_row) out[pos] = j0 + q;
      }
    }
    for (int i = k_row + tid; i < p.k_total; i += kRT) out[i] = 0;           // beyond the row's own budget: padding
  }
  cp_async_wait_all();
}

}  // namespace

size_t topk_stage_limit_bytes() { return 200 * 1024; }

int launch_topk_select(const TopkParams& p, cudaStream_t stream) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (p.L <= kKpt * kRT) {
    // register-resident path; cp.async needs every row start 16-byte aligned
    const size_t smem = sizeof(SharedReg) + (size_t)kCandCap * 4 + (size_t)kKpt * kRT * 4;
    const int grid = (int)(p.rows < (long long)sms ? p.rows : sms);
    const bool vec = (p.L % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.scores) & 15u) == 0);
    if (cudaFuncSetAttribute(topk_select_reg_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(topk_select_reg_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -8;
    if (vec) topk_select_reg_kernel<true><<<grid, kRT, smem, stream>>>(p);
    else topk_select_reg_kernel<false><<<grid, kRT, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -8;
  }
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
