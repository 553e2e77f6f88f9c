// Gather-KV sparse flash-attention forward for sm_100a (bf16 / fp16 / FP8-e4m3 inputs).
//
// Persistent kernel, one CTA per SM.  A work item is one query group: up to 128
// rows of the (optionally permuted) query sequence of one (batch, head) that
// share one list of selected KV token indices.  CTAs walk the items round-robin
// in (head-major, group-minor) order so that the groups in flight at any moment
// read the K/V of one or two heads, which then stay resident in L2.
//
// Roles inside the CTA (576 threads = 18 warps; the two SM sub-partitions that host five warps
// limit every thread to 96 registers):
//   warps 0-3   softmax stream A: columns 0-63 of every 128-token KV tile
//   warps 4-7   softmax stream B: columns 64-127
//               thread r of a stream owns query row r (= TMEM lane r).  The two
//               threads of a row (warps w and w+4, same SM sub-partition) share one
//               running row maximum, so both halves of P accumulate into ONE output
//               accumulator; they agree on it with one two-warp barrier-with-OR per
//               tile (the maximum itself is exchanged only when it has to be raised),
//               and keep separate partial row sums that the epilogue adds.
//   warps 8-11  producers: gather the tile's K rows and V rows with 16-byte
//               cp.async (16 lanes cover one 256-byte row) into a 5-slot ring of
//               128-byte-swizzled tiles in the canonical tcgen05 operand layout;
//               completion is signalled by cp.async.mbarrier.arrive.  The row
//               gather is the scarcest resource of the kernel (measured ceiling about
//               38 B/clk/SM with four warps issuing), hence the deep ring.
//   warp 12     issues S = Q K^T into a double-buffered score tile;
//   warp 13     issues O += P_x V_x for both streams (P read from tensor memory, V as an
//               MN-major shared-memory operand).  Both run converged; one elected lane
//               executes the tcgen05 instructions.
//   warps 14-17 epilogue: one warp per tensor-memory lane group copies the finished O out,
//               normalises, adds the residual and writes the rows, while the other roles are
//               already working on the next item.
//
// Tensor memory (512 columns): score buffers S[0], S[1] (128 columns each), probability
// buffers P[0], P[1] (64 columns each: 32 per stream), O (128 columns).  The dependency
// chains are kept short and independent:
//   * a softmax thread copies its 64 scores to registers and releases S[buf] at once, so
//     Q K^T of tile g+2 only waits for that copy, not for softmax or P V of tile g;
//   * P has its own buffers, so the softmax of tile g+2 only waits for P V of tile g
//     (two tiles back) before storing;
//   * Q is double-buffered in shared memory, so all of this continues across work items.
// With P aliased onto S (one chain Q K^T -> softmax -> P V -> next Q K^T per buffer) the
// round trip of about 2,500 cycles of wake-up, commit and MMA latencies per two tiles left
// the tensor pipe idle most of the time.
//
// The epilogue computes O / (l_A + l_B), adds the cached dense-minus-sparse residual in
// fp32, rounds once to the output type and scatters rows back to the original token
// order when a permutation is given.
//
// Math follows the reference's Hopper kernel
// (mcsparse/kernels/flash_mcsa/ops/flash_sparse_attn/cute/flash_fwd_sm90.py:1005-1340,
// softmax.py:126-227); gather addressing follows topk_gather_kv.py:351-445.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.cuh"
#include "ptx.cuh"

// share of the e4m3 path's exponentials evaluated by a polynomial on the FMA pipe: 0 none, 1 one in four, 2 one in eight
#ifndef MCS_FP8_POLY
#define MCS_FP8_POLY 2
#endif

namespace mcs {

namespace {

constexpr int kTileN = 128;            // KV tokens per tile
constexpr int kThreads = 576;          // 8 softmax + 4 producer + 2 MMA-issuing + 4 epilogue warps
constexpr int kSoftmaxWarps = 8;
constexpr int kProducerWarps = 4;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kRowsPerProducerWarp = 128 / kProducerWarps;
constexpr int kProducerWarp0 = 8;
constexpr int kMmaWarp = 12;
constexpr int kEpiWarp0 = 14;           // warps 14-17: lane groups 2, 3, 0, 1
constexpr int kEpiWarps = 4;
// All warps run with the same register budget (no setmaxnreg: with a partial last warpgroup its
// hand-over never completed on this part).
constexpr int kRing = 5;               // K/V tile slots
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;          // S[buf] at kColS + 128*buf
constexpr uint32_t kColP = 256;        // P[buf] at kColP + 64*buf; stream x at +32*x
constexpr uint32_t kColO = 384;        // O
constexpr int kMaxDynSmem = 232448;    // 227 KB

enum {
  BAR_FULL = 0,                        // [kRing] producers -> MMA
  BAR_EMPTY = BAR_FULL + kRing,        // [kRing] MMA -> producers
  BAR_Q_FULL = BAR_EMPTY + kRing,      // [2]
  BAR_Q_EMPTY = BAR_Q_FULL + 2,        // [2]
  BAR_S_FULL = BAR_Q_EMPTY + 2,        // [2] score tile ready
  BAR_S_FREE = BAR_S_FULL + 2,         // [2] every softmax thread has copied its scores out of S[buf]
  BAR_P_READY = BAR_S_FREE + 2,        // [2 streams][2 bufs]
  BAR_PV_DONE = BAR_P_READY + 4,       // [2] P V of the tile in P[buf] done: P[buf] reusable, O stable
  BAR_O_FULL = BAR_PV_DONE + 2,
  BAR_O_EMPTY,
  BAR_STATS,                           // both streams published their (max, sum) of the finished item
  BAR_STAGE_FREE,                      // [2] epilogue staging (= Q buffer of the finished item) released
  BAR_DRAIN = BAR_STAGE_FREE + 2,      // [2] error path of the two issuers
  BAR_DRAIN_END = BAR_DRAIN + 1,
  BAR_COUNT
};

// RB = bytes per Q/K/V row (head_dim * element size); STAGE = bytes of dedicated epilogue staging
template <int RB, int STAGE>
struct Smem {
  static constexpr int kBlocks = RB / 128;               // 128-byte column blocks
  static constexpr int kTileBytes = kBlocks * 16384;     // 128 rows x RB bytes
  static constexpr int kQ = 0;                           // 2 buffers
  static constexpr int kRingOff = 2 * kTileBytes;
  static constexpr int kBars = kRingOff + kRing * kTileBytes;
  static constexpr int kStats = kBars + BAR_COUNT * 8;   // float [3][128]: partial row sums of streams A, B; row max
  static constexpr int kXch = kStats + 3 * 128 * 4;      // float [2 streams][128]: tile maxima, exchanged on a raise
  // 8-bit inputs (the only case with dedicated staging): a second [2][128] block carries the "dominant maximum" flags
  static constexpr int kTmemSlot = kXch + (STAGE > 0 ? 4 : 2) * 128 * 4;
  // Epilogue staging: 256 rows x (head_dim) bytes of 16-bit output halves.  With 16-bit inputs it is
  // exactly one Q buffer, and the finished item's own Q buffer (idle by then) is used; with 8-bit
  // inputs the Q buffer is half that size and a dedicated area is carved out instead.
  static constexpr int kStage = (kTmemSlot + 16 + 127) & ~127;
  static constexpr int kTotal = kStage + STAGE;
  static constexpr int kDynamic = (kTotal + 1024 <= kMaxDynSmem) ? kTotal + 1024 : kMaxDynSmem;
};


// One producer warp copies kRowsPerProducerWarp rows of D 16-bit elements into a swizzled
// tile.  Lane (l % rows) holds the source row index of tile row (row0 + l); a negative
// index zero-fills the row.  `lane_src` = table base + 16 * (this lane's chunk).
template <int RB>
__device__ __forceinline__ void warp_gather_rows(uint32_t s_tile, int row0, int my_row_idx, const uint8_t* lane_src,
                                                 size_t row_bytes, int lane) {
  constexpr int kChunks = RB / 16;           // 16-byte chunks per row
  constexpr int kRowsPerInstr = 32 / kChunks;
  const int sub = lane / kChunks;
  const int c = lane % kChunks;
  // row0 is a multiple of 8, so (row & 7) == (rl & 7); the chunk XOR splits into a per-lane
  // part and a compile-time part
  const uint32_t dst0 = s_tile + (c >> 3) * 16384 + (row0 + sub) * 128;
  const uint32_t cs4 = static_cast<uint32_t>(((c & 7) ^ sub) << 4);
#pragma unroll
  for (int i = 0; i < kRowsPerProducerWarp / kRowsPerInstr; ++i) {
    const int rl = i * kRowsPerInstr + sub;
    const int id = __shfl_sync(0xffffffffu, my_row_idx, rl);
    const uint32_t dst = dst0 + i * kRowsPerInstr * 128 + (cs4 ^ (((i * kRowsPerInstr) & 7) << 4));
    if (id >= 0) {
      cp_async16(dst, lane_src + (size_t)id * row_bytes);
    } else {
      cp_async16_zfill(dst, lane_src, 0);
    }
  }
}

template <bool kFp16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (kFp16) return pack_f16x2(lo, hi);
  else return pack_bf16x2(lo, hi);
}
template <bool kFp16>
__device__ __forceinline__ float2 unpack16(uint32_t u) {
  if constexpr (kFp16) {
    const __half2 h = *reinterpret_cast<const __half2*>(&u);
    return __half22float2(h);
  } else {
    return make_float2(bf16_lo(u), bf16_hi(u));
  }
}

// Decoded work item.
struct Item {
  int b, h, bh, m, row_base, rows_valid, T;
  const int32_t* gi;
};

__device__ __forceinline__ Item decode_item(const GatherAttnParams& p, int item) {
  Item it;
  it.m = item % p.M;
  it.bh = item / p.M;
  it.h = it.bh % p.H;
  it.b = it.bh / p.H;
  it.row_base = it.m * p.group_rows;
  it.rows_valid = min(p.group_rows, p.Sq - it.row_base);
  const int max_tiles = p.gather_len / kTileN;
  it.T = max_tiles;
  if (p.gl != nullptr) it.T = min(max(p.gl[item], 1), max_tiles);
  it.gi = (p.dense || p.gi == nullptr) ? nullptr : p.gi + (size_t)item * p.gather_len;
  return it;
}

// kType: 0 = bf16, 1 = fp16, 2 = e4m3 (Q/K/V 8-bit, P quantised to e4m3, fp32 accumulation, bf16 out).
// FP8 follows the reference's contract (mcsparse/.../cute/interface.py:358-373, flash_fwd_sm90_fp8.py:
// 145-241): logits = (q8 . k8) * scale_qk_log2[b,h,m] in the log2 domain, O * scale_v[b,h]; V is used
// as it lies in memory (MN-major MMA operand), so neither the Hopper kernel's in-smem transpose nor
// its d-column pre-permutation exists here.
template <int D, int kType, bool kDense>
__global__ void __launch_bounds__(kThreads, 1) gather_attn_kernel(const GatherAttnParams p,
                                                                    const __grid_constant__ DenseTileMaps maps) {
  // dense mode with valid tensor maps: K/V tiles arrive by TMA (one elected thread, two 16 KB boxes per tile)
  const bool use_tma = kDense && maps.valid != 0;
  constexpr bool kFp16 = kType == 1;
  constexpr bool kFp8 = kType == 2;
  constexpr int kEs = kFp8 ? 1 : 2;              // bytes per Q/K/V element
  constexpr int RB = D * kEs;
  constexpr int kStageDedicated = kFp8 ? 256 * D : 0;   // 16-bit inputs stage in the finished item's Q buffer
  using L = Smem<RB, kStageDedicated>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bars = s_base + L::kBars;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  float* stats = reinterpret_cast<float*>(smem + L::kStats);
  float* xch = reinterpret_cast<float*>(smem + L::kXch);
  auto bar = [&](int i) { return bars + 8u * i; };
  auto sQ = [&](int qb) { return s_base + L::kQ + qb * L::kTileBytes; };
  auto sRing = [&](int slot) { return s_base + L::kRingOff + slot * L::kTileBytes; };

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);      // provably warp-uniform
  const int n_items = p.B * p.H * p.M;

  if (static_cast<int>(smem - smem_raw) + L::kTotal > L::kDynamic) {
    if (tid == 0) atomicCAS(p.status, 0, 90);  // shared-memory carve-up does not fit: refuse to run
    return;
  }

  // ---- setup
  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(bar(BAR_FULL + i), use_tma ? 1 : kProducerThreads);
      mbar_init(bar(BAR_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_Q_FULL + i), kProducerThreads);
      mbar_init(bar(BAR_Q_EMPTY + i), 1);
      mbar_init(bar(BAR_S_FULL + i), 1);
      mbar_init(bar(BAR_S_FREE + i), kSoftmaxWarps);
      mbar_init(bar(BAR_P_READY + i), kSoftmaxWarps / 2);
      mbar_init(bar(BAR_P_READY + 2 + i), kSoftmaxWarps / 2);
      mbar_init(bar(BAR_PV_DONE + i), 1);
      mbar_init(bar(BAR_STAGE_FREE + i), kEpiWarps);
    }
    mbar_init(bar(BAR_O_FULL), 1);
    mbar_init(bar(BAR_O_EMPTY), kEpiWarps);
    mbar_init(bar(BAR_STATS), kSoftmaxWarps);
    mbar_init(bar(BAR_DRAIN), 1);
    mbar_init(bar(BAR_DRAIN + 1), 1);
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 8) {
    // =====================================================================
    // softmax streams: thread == query row == TMEM lane
    // =====================================================================
    // One arrival per warp: an mbarrier arrive is a shared-memory atomic, the 32 lanes of a warp
    // arriving on the same barrier are serialised, and per-thread arrivals cost the CTA hundreds of
    // serialised atomics per tile.  Every lane has finished (and fenced) its part before __syncwarp.
    auto warp_arrive = [&](uint32_t b) {
      __syncwarp();
      if (lane == 0) mbar_arrive(b);
    };
    const int x = warp >> 2;                       // stream 0 (A) or 1 (B)
    const int r_in = (warp & 3) * 32 + lane;       // row inside the group
    const uint32_t lane_addr = (static_cast<uint32_t>(warp & 3) * 32u) << 16;
    float scale_log2 = p.scale_log2;
    // Lazy rescale: the running max is only raised (and O rescaled) when a tile's max exceeds
    // it by more than kRescale log2 units, so P stays <= 2^(kRescale + kBias): far inside the
    // bf16 / fp32 range (threshold 24); fp16 P needs <= 65504 (threshold 12); e4m3 P must stay
    // <= 448, and its 3-bit mantissa / 2^-9 floor want the row maximum well above 1: threshold 4
    // with P biased by 2^4, so the largest P of a row lies in [2^4, 2^8].  The bias multiplies P and
    // the row sum alike and cancels in O / l.
    constexpr float kRescale = kFp8 ? 4.0f : (kFp16 ? 12.0f : 24.0f);
    constexpr float kBias = kFp8 ? 4.0f : 0.0f;
    int g = 0;      // tiles processed by this CTA so far
    int ic = 0;     // items processed by this CTA so far
    bool ok = true;

    constexpr int kHalf = D / 2;                 // output columns whose accumulator this stream rescales
    bool s_ready = false;       // next tile's score barrier was already complete when probed
    const int pair_bar = 1 + (warp & 3);            // named barrier of this row block's two warps (w, w+4)
    // where a bounded wait expired (failure path only): item, tile, and whether that tile's pair barrier was passed
    int fail_item = 0, fail_t = 0;
    bool fail_bar_done = false;
    const uint32_t tOh = tmem + kColO + x * kHalf + lane_addr;   // this thread's half of its output row
#pragma unroll 1
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++ic) {
      const Item it = decode_item(p, item);
      if (kFp8) scale_log2 = p.scale_qk_log2[item];
      float m_run = -INFINITY;   // running (possibly stale) row max, log2 domain; identical in both streams
      float l_run = 0.f;         // this stream's partial row sum relative to m_run
#pragma unroll 1
      for (int t = 0; t < it.T; ++t, ++g) {
        const int buf = g & 1;
        if (!s_ready) ok = mbar_wait(bar(BAR_S_FULL + buf), (g >> 1) & 1, p.status, 10);
        if (!ok) { fail_item = item; fail_t = t; fail_bar_done = false; break; }
        tc_fence_after();
        // Copy this thread's 64 scores to registers and hand S[buf] back to the Q K^T issuer at once.
        const uint32_t tSx = tmem + kColS + buf * 128 + x * 64 + lane_addr;
        uint32_t sc[64];
        tmem_ld32(tSx, *reinterpret_cast<uint32_t(*)[32]>(&sc[0]));
        tmem_ld32(tSx + 32, *reinterpret_cast<uint32_t(*)[32]>(&sc[32]));
        tmem_wait_ld();
        tc_fence_before();
        warp_arrive(bar(BAR_S_FREE + buf));
        if (kDense && t == it.T - 1) {
          // dense mode: key positions beyond the sequence end (zero-filled rows of the last tile) get -inf
          const int rem = p.Sk - t * kTileN - x * 64;      // valid columns of this stream's half
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i >= rem) sc[i] = 0xff800000u;
        }
        // P[buf] was last read by P V of tile g-2: probe now, wait (if at all) just before the stores
        const bool p_free = g < 2 || mbar_test_wait(bar(BAR_PV_DONE + buf), ((g >> 1) - 1) & 1);
        // four independent chains of three-input maxima
        float mx0 = fmaxf(__uint_as_float(sc[0]), __uint_as_float(sc[1]));
        float mx1 = fmaxf(__uint_as_float(sc[2]), __uint_as_float(sc[3]));
        float mx2 = fmaxf(__uint_as_float(sc[4]), __uint_as_float(sc[5]));
        float mx3 = fmaxf(__uint_as_float(sc[6]), __uint_as_float(sc[7]));
#pragma unroll
        for (int i = 8; i < 64; i += 8) {
          mx0 = fmax3(mx0, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
          mx2 = fmax3(mx2, __uint_as_float(sc[i + 4]), __uint_as_float(sc[i + 5]));
          mx3 = fmax3(mx3, __uint_as_float(sc[i + 6]), __uint_as_float(sc[i + 7]));
        }
        const float m_loc = fmaxf(fmax3(mx0, mx1, mx2), mx3) * scale_log2;
        // Lazy raise of the shared running max.  One barrier-with-OR per tile between the two warps of
        // this row block tells both whether any of their 64 threads wants a raise (always at the first
        // tile of an item, rarely afterwards); only then are the tile maxima exchanged.
        bool want = (m_loc - m_run) > kRescale;
        bool dom = false;
        if constexpr (kFp8) {
          // e4m3 P has three mantissa bits: up to 3 % error per element, which only shows in the output of a row
          // whose mass sits on one or two keys.  A new row maximum that would hold more than an eighth of the mass
          // accumulated so far therefore becomes the reference point at once (not lazily): its P is then 2^kBias,
          // exactly representable, and the dominant term of the row carries no rounding error at all.
          dom = (m_loc > m_run) && (ex2_approx(m_loc - m_run + kBias) > 0.125f * l_run);
          want = want || dom;
        }
        if (named_bar_red_or(pair_bar, 64, want)) {
          xch[x * 128 + r_in] = m_loc;
          if constexpr (kFp8) xch[256 + x * 128 + r_in] = dom ? 1.f : 0.f;
          named_bar_sync(pair_bar, 64);
          const float m_new = fmaxf(m_loc, xch[(x ^ 1) * 128 + r_in]);
          bool raise = (m_new - m_run) > kRescale;            // the same decision in both threads of the row
          if constexpr (kFp8) raise = raise || ((dom || xch[256 + (x ^ 1) * 128 + r_in] != 0.f) && m_new > m_run);
          // everything accumulated relative to the old max is multiplied by alpha = 2^(old - new):
          // the partial row sum and, from the second tile on, this thread's half of the output row
          // (stable once the previous P V is done)
          const float alpha = raise ? ex2_approx(m_run - m_new) : 1.f;
          if (raise) m_run = m_new;
          l_run *= alpha;
          if (t > 0) {
            ok = mbar_wait(bar(BAR_PV_DONE + ((g - 1) & 1)), ((g - 1) >> 1) & 1, p.status, 12);
            if (!ok) { fail_item = item; fail_t = t; fail_bar_done = true; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < kHalf / 8; ++c) {
              uint32_t r[8];
              tmem_ld8(tOh + c * 8, r);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 8; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st8(tOh + c * 8, r);
            }
          }
        }
        const float neg_m = kBias - m_run;
        if (!p_free) ok = mbar_wait(bar(BAR_PV_DONE + buf), ((g >> 1) - 1) & 1, p.status, 15);
        if (!ok) { fail_item = item; fail_t = t; fail_bar_done = true; break; }
        // exp2, partial row sum, pack, store P: 16 values (8 or 4 columns) at a time
        const uint32_t tPx = tmem + kColP + buf * 64 + x * 32 + lane_addr;
        float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
        uint32_t pk8[8];       // e4m3 only: two groups of 16 values share one store
#pragma unroll
        for (int h4 = 0; h4 < 4; ++h4) {
          uint32_t pk[8];
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            const int e = h4 * 16 + 2 * i;
            const float p0 = ex2_approx(fmaf(__uint_as_float(sc[e]), scale_log2, neg_m));
            const float p1 = ex2_approx(fmaf(__uint_as_float(sc[e + 1]), scale_log2, neg_m));
            const float p2 = ex2_approx(fmaf(__uint_as_float(sc[e + 2]), scale_log2, neg_m));
            // e4m3: a share of the exponentials runs on the FMA pipe, at the precision an e4m3 probability needs
            // (measured at the long-video shape: 7.13 ms with none, 6.96 with one in four, 6.93 with one in eight)
            const float y3 = fmaf(__uint_as_float(sc[e + 3]), scale_log2, neg_m);
            // (for 16-bit inputs the same trade loses: 0.837 / 0.879 ms against 0.824 with one in sixteen / one in eight)
            const float p3 = (kFp8 && (MCS_FP8_POLY == 1 || (MCS_FP8_POLY == 2 && (i & 2)))) ? ex2_poly2(y3) : ex2_approx(y3);
            ls0 += p0;
            ls1 += p1;
            ls2 += p2;
            ls3 += p3;
            if constexpr (kFp8) {
              pk8[(h4 & 1) * 4 + i / 2] = pack_e4m3x4(p0, p1, p2, p3);
            } else {
              pk[i] = pack16<kFp16>(p0, p1);
              pk[i + 1] = pack16<kFp16>(p2, p3);
            }
          }
          if constexpr (kFp8) {
            if (h4 & 1) tmem_st8(tPx + (h4 >> 1) * 8, pk8);      // 32 e4m3 values = 8 columns
          } else {
            tmem_st8(tPx + h4 * 8, pk);                         // 16 16-bit values = 8 columns
          }
        }
        l_run += (ls0 + ls1) + (ls2 + ls3);
        // probe the next tile's score barrier now, so that a satisfied wait costs nothing at the loop top
        s_ready = mbar_test_wait(bar(BAR_S_FULL + ((g + 1) & 1)), ((g + 1) >> 1) & 1);
        tmem_wait_st();
        tc_fence_before();
        warp_arrive(bar(BAR_P_READY + 2 * x + buf));
        if (t == it.T - 1) {
          // Last tile done: publish this stream's partial row sum (and the shared max) for the epilogue
          // warps, once they have read the previous item's (normally long true).
          if (ic > 0) ok = mbar_wait(bar(BAR_O_EMPTY), (ic - 1) & 1, p.status, 13);
          if (!ok) { fail_item = item; fail_t = t; fail_bar_done = true; break; }
          stats[x * 128 + r_in] = l_run;
          if (x == 0) stats[256 + r_in] = m_run;
          warp_arrive(bar(BAR_STATS));
        }
      }
      if (!ok) break;
    }
    if (!ok) {
      // Failure path: a bounded wait expired (the status word says where).  The partner warp of this row
      // block may still be running; a named barrier has no bounded wait, so this warp keeps meeting the
      // partner at the pair barrier once per remaining tile (and at the exchange barrier whenever the
      // OR says so), until the partner runs into its own expired wait and ends the same way.
      int item = fail_item, t = fail_t;
      bool done = fail_bar_done;
      while (item < n_items) {
        const int T = decode_item(p, item).T;
        for (; t < T; ++t) {
          if (!done && named_bar_red_or(pair_bar, 64, false)) named_bar_sync(pair_bar, 64);
          done = false;
        }
        t = 0;
        item += gridDim.x;
      }
    }
    tc_fence_before();
  } else if (warp < kMmaWarp) {
    // =====================================================================
    // producers: K/V/Q row gathers.
    //
    // Producer warp pw gathers tile rows 32*pw..+31 of every K, V and Q tile with 16-byte cp.async (the
    // softmax warps never use the load/store unit, so they are never queued behind the hundreds of copies
    // in flight).  In the dense mode with tensor maps one elected thread of warp 0 issues the K/V tiles as
    // TMA boxes instead and the four warps only gather Q.
    // =====================================================================
    const int pw = warp - kProducerWarp0;
    const int row0 = pw * kRowsPerProducerWarp;
    const int my_row = row0 + lane;                              // tile row / query row of this thread
    const int chunk_off = (lane % (RB / 16)) * 16;               // this lane's 16-byte chunk inside a row
    const size_t q_row = kEs * (size_t)p.q_stride[1], k_row = kEs * (size_t)p.k_stride[1], v_row = kEs * (size_t)p.v_stride[1];
    int slot = 0, slot_phase = 0;   // ring position; the phase flips every wrap
    bool wrapped = false;
    bool ok = true;

    auto enter_item = [&](int item, int ic) {
      // called once per item when the K cursor reaches it: request Q, warm L2 for this item's residual
      // (read by the epilogue warps later) and for the next item's indices
      const Item it = decode_item(p, item);
      const int qbuf = ic & 1;
      int src_row = -1;
      if (my_row < it.rows_valid) {
        const int row = it.row_base + my_row;
        src_row = row;
        if (p.perm != nullptr) src_row = static_cast<int>(p.perm[(size_t)it.bh * p.Sq + row]);
        if (p.residual != nullptr) {
          const uint8_t* res_row = reinterpret_cast<const uint8_t*>(p.residual) +
                                   2 * ((size_t)it.b * p.r_stride[0] + (size_t)it.h * p.r_stride[1] + (size_t)row * p.r_stride[2]);
          prefetch_l2(res_row);
          if (D == 128) prefetch_l2(res_row + 128);
        }
      }
      if (!kDense && item + (int)gridDim.x < n_items) {
        // (packed indices: 2 bytes per entry; their bit planes are 1/16 of that and are left to the loads themselves)
        const size_t next = (size_t)(item + gridDim.x) * p.gather_len;
        const uint8_t* gin = p.gi16 != nullptr ? reinterpret_cast<const uint8_t*>(p.gi16 + next) : reinterpret_cast<const uint8_t*>(p.gi + next);
        const int bytes = p.gather_len * (p.gi16 != nullptr ? 2 : 4);
        for (int off = (pw * 32 + lane) * 128; off < bytes; off += kProducerThreads * 128) prefetch_l2(gin + off);
      }
      if (ic >= 2) ok = ok && mbar_wait(bar(BAR_Q_EMPTY + qbuf), ((ic >> 1) - 1) & 1, p.status, 22) &&
                      mbar_wait(bar(BAR_STAGE_FREE + qbuf), ((ic >> 1) - 1) & 1, p.status, 26);
      if (!ok) return;
      const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q) +
                          kEs * ((size_t)it.b * p.q_stride[0] + (size_t)it.h * p.q_stride[2]) + chunk_off;
      warp_gather_rows<RB>(sQ(qbuf), row0, src_row, qb, q_row, lane);
      cp_async_arrive_noinc(bar(BAR_Q_FULL + qbuf));
    };

    // per-item constants of a cursor
    struct Cur {
      int item, ic, t, T, b, h;
      const int32_t* gi;     // this thread's entry of tile 0
      size_t ioff;           // the same as an offset into the index tensor (packed form)
      const uint8_t* kv;     // K or V base of (b, h) + chunk offset of this lane
    };
    const bool tma_leader = elect_one();
    auto load_tile_tma = [&](const Cur& c, bool is_v) {
      // dense mode: the tile is 128 consecutive key rows of one (batch, head): kBlocks TMA boxes of 128 rows x
      // 128 bytes, issued by one thread of producer warp 0; rows beyond the sequence end arrive as zeros
      if (pw == 0) {
        if (wrapped) ok = ok && mbar_wait(bar(BAR_EMPTY + slot), slot_phase ^ 1, p.status, 20);
        if (!ok) return;
        if (tma_leader) {
          mbar_arrive_expect_tx(bar(BAR_FULL + slot), L::kTileBytes);
          const void* map = is_v ? static_cast<const void*>(maps.v) : static_cast<const void*>(maps.k);
          int co[4] = {0, 0, 0, 0};
          co[is_v ? maps.v_pos_h : maps.k_pos_h] = c.h;
          co[is_v ? maps.v_pos_row : maps.k_pos_row] = c.t * kTileN;
          co[is_v ? maps.v_pos_b : maps.k_pos_b] = c.b;
#pragma unroll
          for (int cb = 0; cb < L::kBlocks; ++cb)
            tma_load_4d(sRing(slot) + cb * 16384, map, cb * (128 / kEs), co[1], co[2], co[3], bar(BAR_FULL + slot));
        }
      }
      if (++slot == kRing) { slot = 0; slot_phase ^= 1; wrapped = true; }
    };
    auto load_tile = [&](const uint8_t* lane_src, size_t row_bytes, int idx, bool is_v) {
      if (wrapped) ok = ok && mbar_wait(bar(BAR_EMPTY + slot), slot_phase ^ 1, p.status, 20);
      if (!ok) return;
      // raw index, clamped only here: the global load issued one step earlier stays in flight until now
      warp_gather_rows<RB>(sRing(slot), row0, min(max(idx, 0), p.Sk - 1), lane_src, row_bytes, lane);
      cp_async_arrive_noinc(bar(BAR_FULL + slot));
      if (++slot == kRing) { slot = 0; slot_phase ^= 1; wrapped = true; }
    };

    auto set_item = [&](Cur& c, const void* tensor, const int64_t* stride) {
      const Item it = decode_item(p, c.item);
      c.T = it.T;
      c.b = it.b;
      c.h = it.h;
      c.gi = kDense ? nullptr : it.gi + my_row;
      c.ioff = (size_t)c.item * p.gather_len + my_row;
      c.kv = reinterpret_cast<const uint8_t*>(tensor) + kEs * ((size_t)it.b * stride[0] + (size_t)it.h * stride[2]) + chunk_off;
    };
    // dense mode: the "selected" tokens of tile t are simply t*128 .. t*128+127 (rows beyond the end are
    // clamped here and masked in the softmax)
    auto load_idx = [&](const Cur& c) -> int {
      if (kDense) return c.t * kTileN + my_row;
      if (p.gi16 != nullptr) {
        // 17-bit indices: the low 16 bits as an array of their own, bit 16 in a bit plane (one word per 32 entries)
        const size_t o = c.ioff + (size_t)c.t * kTileN;
        const uint32_t lo = __ldg(p.gi16 + o), hi = (__ldg(p.gi_hi + (o >> 5)) >> (o & 31)) & 1u;
        return static_cast<int>(lo | (hi << 16));
      }
      return __ldg(c.gi + c.t * kTileN);
    };

    // Fill order = consumption order of the MMA warp: K(0), then per tile g: K(g+1), V(g),
    // where g+1 may belong to the next work item (its Q is requested just before its K(0)).
    // The indices of the next K tile are fetched one step ahead of their use.
    if (blockIdx.x < n_items) {
      Cur kc{static_cast<int>(blockIdx.x), 0, 0, 0, 0, 0, nullptr, 0, nullptr}, vc = kc;
      set_item(kc, p.k, p.k_stride);
      set_item(vc, p.v, p.v_stride);
      enter_item(kc.item, kc.ic);
      int idx_k = load_idx(kc);
      if (use_tma) load_tile_tma(kc, false); else load_tile(kc.kv, k_row, idx_k, false);
      int idx_v = idx_k;
      auto advance_k = [&]() {
        if (++kc.t >= kc.T) {
          kc.t = 0;
          kc.item += gridDim.x;
          ++kc.ic;
          if (kc.item < n_items) set_item(kc, p.k, p.k_stride);
        }
      };
      advance_k();
      bool have_k = kc.item < n_items;
      if (have_k) idx_k = load_idx(kc);
#pragma unroll 1
      while (ok) {
        const int idx_cur = idx_k;
        const bool had_k = have_k;
        if (had_k) {
          if (kc.t == 0) enter_item(kc.item, kc.ic);
          if (!ok) break;
          if (use_tma) load_tile_tma(kc, false); else load_tile(kc.kv, k_row, idx_cur, false);
          if (!ok) break;
          advance_k();
          have_k = kc.item < n_items;
          if (have_k) idx_k = load_idx(kc);       // in flight while V(g) is issued
        }
        if (!had_k) {
          // no K entry in this (final) step: skip its ring number so that V(g) is always entry 2g+2
          if (++slot == kRing) { slot = 0; slot_phase ^= 1; wrapped = true; }
        }
        if (use_tma) load_tile_tma(vc, true); else load_tile(vc.kv, v_row, idx_v, true);
        if (!ok) break;
        idx_v = idx_cur;                           // V(g+1) uses the indices of K(g+1)
        if (++vc.t >= vc.T) {
          if (!had_k) break;                       // last tile of the last item
          vc.t = 0;
          vc.item += gridDim.x;
          ++vc.ic;
          set_item(vc, p.v, p.v_stride);
        }
      }
    }
    cp_async_wait_all();
    tc_fence_before();
  } else if (warp >= kEpiWarp0) {
    // =====================================================================
    // epilogue warps: one per tensor-memory lane group, thread == query row.
    //
    // out = O / (l_A + l_B) + residual, rounded once to the output type and written to the row's
    // original position.  The softmax warps are the busiest part of the CTA, so nothing of this
    // runs there: these four warps pick a finished item up as soon as its last P V has completed,
    // copy O out of tensor memory (after which the next item's first P V may overwrite it) and do
    // the global traffic at leisure while the next item is already being processed.
    //
    // Global traffic is staged through shared memory so that every global access is coalesced: a
    // thread owns a ROW in tensor memory, and 32 row-strided 16-byte accesses per instruction cost
    // the load/store unit 32 wavefronts each.  Each warp has a private 32-row area, XOR-swizzled
    // by row so that both access patterns are conflict-free.  With 16-bit inputs the area is the
    // finished item's own Q buffer (idle once the item's last Q K^T has completed).
    // =====================================================================
    const int lg = warp & 3;                              // lane group of this warp
    const int r_in = lg * 32 + lane;                      // row inside the group
    const uint32_t lane_addr = (static_cast<uint32_t>(lg) * 32u) << 16;
    constexpr float kBias = kFp8 ? 4.0f : 0.0f;           // P bias of the e4m3 path (see the softmax role)
    constexpr int kRowBytes = D * 2;                      // bytes of an output row
    constexpr int kCh = kRowBytes / 16;                   // 16-byte chunks per row
    constexpr int kRpi = 32 / kCh;                        // rows covered by one coalesced warp access
    auto warp_arrive = [&](uint32_t b) {
      __syncwarp();
      if (lane == 0) mbar_arrive(b);
    };
    bool ok = true;
    int ic = 0;
#pragma unroll 1
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++ic) {
      const Item it = decode_item(p, item);
      const int qbuf = ic & 1;
      const uint32_t st = (kFp8 ? (s_base + L::kStage) : sQ(qbuf)) + static_cast<uint32_t>(lg) * 32u * kRowBytes;
      const float vscale = kFp8 ? p.scale_v[it.bh] : 1.f;
      unsigned long long my_out = 0ull;                   // this row's output address, 0 for a padding row
      float* my_lse = nullptr;
      if (r_in < it.rows_valid) {
        const int row = it.row_base + r_in;               // position in (permuted) query order
        long long orow = row;
        if (p.perm != nullptr && !p.out_group_order) orow = p.perm[(size_t)it.bh * p.Sq + row];
        uint8_t* obase = reinterpret_cast<uint8_t*>(p.out);
        long long lrow = orow;
        if (p.n_out_peers > 0) {
          // sequence-sharded output: the row belongs to rank orow / rows_per_peer; the store below goes
          // straight into that rank's memory (the all-to-all back of Ulysses, fused into this epilogue)
          const int peer = static_cast<int>(orow / p.out_rows_per_peer);
          lrow = orow - (long long)peer * p.out_rows_per_peer;
          obase = reinterpret_cast<uint8_t*>(p.out_peer[peer]);
        }
        my_out = reinterpret_cast<unsigned long long>(
            obase + 2 * ((size_t)it.b * p.o_stride[0] + (size_t)lrow * p.o_stride[1] + (size_t)it.h * p.o_stride[2]));
        if (p.lse != nullptr) my_lse = p.lse + (size_t)it.bh * p.Sq + orow;
      }
      const bool has_res = p.residual != nullptr;
      const int ch = lane % kCh;
      // the staging area is free once the item's last Q K^T has read Q (16-bit inputs), or at once
      if (!kFp8) ok = mbar_wait(bar(BAR_Q_EMPTY + qbuf), (ic >> 1) & 1, p.status, 40);
      if (!ok) break;
      if (has_res) {
        // residual rows of this warp, coalesced, straight into the staging area
        const uint8_t* rb = reinterpret_cast<const uint8_t*>(p.residual) +
                            2 * ((size_t)it.b * p.r_stride[0] + (size_t)it.h * p.r_stride[1]);
        const size_t r_row = 2 * (size_t)p.r_stride[2];
#pragma unroll
        for (int i = 0; i < kCh; ++i) {
          const int rl = i * kRpi + lane / kCh;           // row inside the warp's 32 rows
          const uint32_t dst = st + rl * kRowBytes + ((ch ^ (rl % kCh)) << 4);
          if (lg * 32 + rl < it.rows_valid)
            cp_async16(dst, rb + (size_t)(it.row_base + lg * 32 + rl) * r_row + ch * 16);
          else
            cp_async16_zfill(dst, rb, 0);
        }
      }
      if (!mbar_wait(bar(BAR_O_FULL), ic & 1, p.status, 11)) { ok = false; break; }
      if (!mbar_wait(bar(BAR_STATS), ic & 1, p.status, 14)) { ok = false; break; }
      tc_fence_after();
      // both streams' partial sums are relative to the same (shared) row maximum
      const float m_all = stats[256 + r_in];
      const float l_all = stats[r_in] + stats[128 + r_in];
      const float w = p.out_sign * vscale / l_all;          // out_sign -1: out = residual - attention
      const uint32_t tO = tmem + kColO + lane_addr;
      const uint32_t my_row = st + lane * kRowBytes;
      cp_async_wait_all();
      __syncwarp();
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        uint32_t ra[16];
        tmem_ld16(tO + c * 16, ra);
        tmem_wait_ld();
        if (c == D / 16 - 1) {
          // all of this warp's reads of O and of the statistics are done
          tc_fence_before();
          warp_arrive(bar(BAR_O_EMPTY));
        }
#pragma unroll
        for (int q4 = 0; q4 < 2; ++q4) {
          const uint32_t addr = my_row + ((((c * 2 + q4) ^ (lane % kCh))) << 4);
          uint4 res = make_uint4(0, 0, 0, 0);
          if (has_res) res = lds_v4(addr);
          const uint32_t rw[4] = {res.x, res.y, res.z, res.w};
          uint32_t ow[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 rr = unpack16<kFp16>(rw[j]);
            const int k = q4 * 8 + 2 * j;
            const float o0 = fmaf(__uint_as_float(ra[k]), w, rr.x);
            const float o1 = fmaf(__uint_as_float(ra[k + 1]), w, rr.y);
            ow[j] = pack16<kFp16>(o0, o1);
          }
          sts_v4(addr, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
      }
      // natural-log LSE of the scaled logits
      if (my_lse != nullptr) *my_lse = (m_all + lg2_approx(l_all) - kBias) * 0.6931471805599453f;
      __syncwarp();
      // coalesced write-out: kCh lanes per output row
#pragma unroll
      for (int i = 0; i < kCh; ++i) {
        const int rl = i * kRpi + lane / kCh;
        const unsigned long long optr = __shfl_sync(0xffffffffu, my_out, rl);
        const uint4 v = lds_v4(st + rl * kRowBytes + ((ch ^ (rl % kCh)) << 4));
        if (optr != 0ull) *reinterpret_cast<uint4*>(optr + ch * 16) = v;
      }
      warp_arrive(bar(BAR_STAGE_FREE + qbuf));            // the staging area (a Q buffer) may be refilled
    }
    tc_fence_before();
  } else {
    // =====================================================================
    // MMA issuers: warp 12 issues every S = Q K^T, warp 13 every O += P V.  Both warps run their
    // loops converged on warp-uniform values; one elected lane executes the tcgen05 instructions.
    // The MMA queue holds about five 128x128x16 products, so whatever an issuer does between two
    // bursts (waits, commits, bookkeeping) has to fit into about 300 cycles or the tensor pipe drains;
    // two issuers keep each other's gaps covered.  The two products share no tensor-memory buffer (P has its own), so
    // the issuers never wait for each other: Q K^T of tile g+2 waits for the softmax threads'
    // register copy of S[buf] (BAR_S_FREE), P V of tile g for P (BAR_P_READY) and V.
    // Ring entries are numbered K(0)=0, K(g)=2g-1, V(g)=2g+2 (the producers skip one number before
    // the very last V), so each issuer steps through its own entries two at a time.
    // =====================================================================
    constexpr uint32_t kFmt = (kFp16 || kFp8) ? 0u : 1u;   // kind::f16: 0 f16, 1 bf16; kind::f8f6f4: 0 e4m3
    // descriptor high word: stride byte offset 1024, version 1, 128-byte swizzle
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
    auto desc = [&](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
    // A satisfied mbarrier wait still costs its full latency when the next instruction depends on it,
    // so barriers are probed early without blocking and only waited for if they were not complete.
    auto wait_if = [&](bool done, uint32_t b, uint32_t parity, int site) -> bool {
      return done || mbar_wait(b, parity, p.status, site);
    };
    const bool leader = elect_one();
    if (warp == kMmaWarp && blockIdx.x < n_items) {
      // ------------------------------------------------------------------ Q K^T issuer
      constexpr uint32_t idesc_qk = mma_idesc(kFmt, kFmt, 0, 0, 128, kTileN);
      constexpr uint32_t kLboK = (16u >> 4) << 16;       // K-major operands (Q, K): LBO unused
      bool ok = true;
      int slot = 0, phase = 0;                           // ring position of the next K entry
      int item = blockIdx.x, ic = 0, t = 0, T = decode_item(p, item).T, g = 0;
      // optional telemetry (mcs_set_clock_buffer): SM cycles and nanoseconds this CTA's tile loop ran, i.e.
      // the SM clock under the kernel's own load, which no host-side poll can resolve
      const bool telemetry = p.clock_out != nullptr && blockIdx.x == 0;
      long long clk_c0 = 0;
      unsigned long long clk_g0 = 0;
      if (telemetry) { clk_c0 = clock64(); clk_g0 = globaltimer_ns(); }
#pragma unroll 1
      while (item < n_items) {
        const int qbuf = ic & 1, buf = g & 1;
        const bool k_ready = mbar_test_wait(bar(BAR_FULL + slot), phase);
        const bool s_free = g < 2 || mbar_test_wait(bar(BAR_S_FREE + buf), ((g >> 1) - 1) & 1);
        if (t == 0 && !mbar_wait(bar(BAR_Q_FULL + qbuf), (ic >> 1) & 1, p.status, 31)) { ok = false; break; }
        if (!wait_if(k_ready, bar(BAR_FULL + slot), phase, 30)) { ok = false; break; }
        if (!wait_if(s_free, bar(BAR_S_FREE + buf), ((g >> 1) - 1) & 1, 35)) { ok = false; break; }
        fence_proxy_async_smem();
        tc_fence_after();
        const uint32_t tS = tmem + kColS + buf * 128;
        const uint32_t qlo = ((sQ(qbuf) & 0x3FFFFu) >> 4) | kLboK;
        const uint32_t klo = ((sRing(slot) & 0x3FFFFu) >> 4) | kLboK;
#pragma unroll
        for (int j = 0; j < RB / 32; ++j) {
          // one k-step = 32 bytes of every row (16 16-bit or 32 8-bit elements) inside the 128-byte swizzle span
          const uint32_t koff = (j >> 2) * (16384 >> 4) + (j & 3) * 2;
          if (leader) {
            if constexpr (kFp8) mma_f8_ss(tS, desc(qlo + koff), desc(klo + koff), idesc_qk, j > 0);
            else mma_f16_ss(tS, desc(qlo + koff), desc(klo + koff), idesc_qk, j > 0);
          }
        }
        if (leader) {
          tc_commit(bar(BAR_EMPTY + slot));
          tc_commit(bar(BAR_S_FULL + buf));
          if (t == T - 1) tc_commit(bar(BAR_Q_EMPTY + qbuf));
        }
        // next K entry: 0 -> 1, then +2
        const int step = g == 0 ? 1 : 2;
        slot += step;
        if (slot >= kRing) { slot -= kRing; phase ^= 1; }
        ++g;
        if (++t >= T) {
          t = 0;
          item += gridDim.x;
          ++ic;
          if (item < n_items) T = decode_item(p, item).T;
        }
      }
      if (telemetry && lane == 0) {
        p.clock_out[0] = clock64() - clk_c0;
        p.clock_out[1] = static_cast<long long>(globaltimer_ns() - clk_g0);
        p.clock_out[2] = g;
      }
      if (!ok) {
        // error path: let outstanding MMAs retire before tensor memory is released
        if (leader) tc_commit(bar(BAR_DRAIN));
        mbar_wait_quiet(bar(BAR_DRAIN), 0, 1 << 20);
      }
    } else if (warp == kMmaWarp + 1 && blockIdx.x < n_items) {
      // ------------------------------------------------------------------ P V issuer
      constexpr uint32_t idesc_pv = mma_idesc(kFmt, kFmt, 0, 1, 128, D);
      constexpr uint32_t kLboV = (16384u >> 4) << 16;    // MN-major V: 16 KB between 64-element column blocks
      bool ok = true;
      int slot = 2, phase = 0;                           // ring position of the next V entry (V(0) = entry 2)
      int item = blockIdx.x, ic = 0, t = 0, T = decode_item(p, item).T, g = 0;
#pragma unroll 1
      while (item < n_items) {
        const int buf = g & 1;
        const bool v_ready = mbar_test_wait(bar(BAR_FULL + slot), phase);
        const bool pa_ready = mbar_test_wait(bar(BAR_P_READY + buf), (g >> 1) & 1);
        const bool pb_ready = mbar_test_wait(bar(BAR_P_READY + 2 + buf), (g >> 1) & 1);
        if (!wait_if(v_ready, bar(BAR_FULL + slot), phase, 34)) { ok = false; break; }
        if (t == 0 && ic > 0 && !mbar_wait(bar(BAR_O_EMPTY), (ic - 1) & 1, p.status, 32)) { ok = false; break; }
        const uint32_t vlo = ((sRing(slot) & 0x3FFFFu) >> 4) | kLboV;
        fence_proxy_async_smem();
        // Both halves of P before the first product: each product adds to ALL columns of O, and when the running
        // maximum was raised each of the row's two threads rescales its own half of them first; a product issued on
        // one stream's arrival alone could land in columns the other thread is still rescaling.
        if (!wait_if(pa_ready, bar(BAR_P_READY + buf), (g >> 1) & 1, 33) ||
            !wait_if(pb_ready, bar(BAR_P_READY + 2 + buf), (g >> 1) & 1, 33)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const uint32_t tP = tmem + kColP + buf * 64 + x * 32;
          const uint32_t tO = tmem + kColO;
          if constexpr (kFp8) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              // A: 32 e4m3 values = 8 TMEM columns per k-step; B: 32 KV rows of 128 bytes = 4096 bytes
              if (leader) mma_f8_ts(tO, tP + j * 8, desc(vlo + (x * 2 + j) * (4096 >> 4)), idesc_pv, (t > 0) || (x > 0) || (j > 0));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // A: 16 packed 16-bit values = 8 TMEM columns per k-step; B: 16 KV rows = 2048 bytes
              if (leader) mma_f16_ts(tO, tP + j * 8, desc(vlo + (x * 4 + j) * (2048 >> 4)), idesc_pv, (t > 0) || (x > 0) || (j > 0));
            }
          }
        }
        if (!ok) break;
        if (leader) {
          tc_commit(bar(BAR_EMPTY + slot));
          tc_commit(bar(BAR_PV_DONE + buf));
          if (t == T - 1) tc_commit(bar(BAR_O_FULL));
        }
        slot += 2;
        if (slot >= kRing) { slot -= kRing; phase ^= 1; }
        ++g;
        if (++t >= T) {
          t = 0;
          item += gridDim.x;
          ++ic;
          if (item < n_items) T = decode_item(p, item).T;
        }
      }
      if (!ok) {
        if (leader) tc_commit(bar(BAR_DRAIN + 1));
        mbar_wait_quiet(bar(BAR_DRAIN + 1), 0, 1 << 20);
      }
    }
    __syncwarp();
    tc_fence_before();
  }

  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// Measurement aid: the K/V row gather of a sparse attention launch and nothing else.  Same grid, same item walk,
// same four producer warps and the same copy routine as the attention kernel; the tiles go into a six-slot ring
// that nobody reads, four tiles of copies in flight per thread.  Its duration is the time the launch's selected
// rows need to come out of L2 into shared memory when no other role competes: a floor for the attention kernel
// that no change to its softmax or tensor-core schedule can lower.
template <int RB>
__global__ void __launch_bounds__(kProducerThreads, 1) gather_rate_probe_kernel(const GatherAttnParams p) {
  constexpr int kTileBytes = (RB / 128) * 16384;
  constexpr int kSlots = 6;
  constexpr int kEs = 1;     // RB counts bytes
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t s_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int lane = threadIdx.x & 31, pw = threadIdx.x >> 5;
  const int row0 = pw * kRowsPerProducerWarp, my_row = row0 + lane;
  const int chunk_off = (lane % (RB / 16)) * 16;
  const int es = RB / p.D;                      // bytes per element
  const size_t k_row = (size_t)es * p.k_stride[1], v_row = (size_t)es * p.v_stride[1];
  const int n_items = p.B * p.H * p.M;
  int slot = 0;
  (void)kEs;
#pragma unroll 1
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const Item it = decode_item(p, item);
    const uint8_t* kb = reinterpret_cast<const uint8_t*>(p.k) + (size_t)es * ((size_t)it.b * p.k_stride[0] + (size_t)it.h * p.k_stride[2]) + chunk_off;
    const uint8_t* vb = reinterpret_cast<const uint8_t*>(p.v) + (size_t)es * ((size_t)it.b * p.v_stride[0] + (size_t)it.h * p.v_stride[2]) + chunk_off;
    int idx_next = __ldg(it.gi + my_row);
#pragma unroll 1
    for (int t = 0; t < it.T; ++t) {
      const int idx = min(max(idx_next, 0), p.Sk - 1);
      if (t + 1 < it.T) idx_next = __ldg(it.gi + (t + 1) * kTileN + my_row);
      warp_gather_rows<RB>(s_base + slot * kTileBytes, row0, idx, kb, k_row, lane);
      cp_async_commit_group();
      slot = slot + 1 == kSlots ? 0 : slot + 1;
      warp_gather_rows<RB>(s_base + slot * kTileBytes, row0, idx, vb, v_row, lane);
      cp_async_commit_group();
      slot = slot + 1 == kSlots ? 0 : slot + 1;
      cp_async_wait_group<4>();
    }
  }
  cp_async_wait_all();
}

int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

template <int D, int kType, bool kDense = false>
int launch(const GatherAttnParams& p, cudaStream_t stream) {
  using L = Smem<D * (kType == 2 ? 1 : 2), kType == 2 ? 256 * D : 0>;
  auto kern = gather_attn_kernel<D, kType, kDense>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
  if (e != cudaSuccess) return -8;
  const long long items = (long long)p.B * p.H * p.M;
  const int grid = (int)(items < num_sms() ? items : num_sms());
  DenseTileMaps maps{};
  if (kDense) {
    // K/V tiles of the dense mode are consecutive rows: load them with TMA when the layout allows it
    maps.valid = encode_tile_map(p.k, p.k_stride, p.B, p.Sk, p.H, D, maps.k, maps.k_pos_h, maps.k_pos_row, maps.k_pos_b) &&
                 encode_tile_map(p.v, p.v_stride, p.B, p.Sk, p.H, D, maps.v, maps.v_pos_h, maps.v_pos_row, maps.v_pos_b);
  }
  kern<<<grid, kThreads, L::kDynamic, stream>>>(p, maps);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace

int launch_gather_attn_16bit(const GatherAttnParams& p, bool fp16, cudaStream_t stream) {
  if (p.dense) {
    // dense mode is its own instantiation so that the sparse kernel's inner loops carry none of it
    if (p.D == 128) return fp16 ? launch<128, 1, true>(p, stream) : launch<128, 0, true>(p, stream);
    if (p.D == 64) return fp16 ? launch<64, 1, true>(p, stream) : launch<64, 0, true>(p, stream);
    return -3;
  }
  if (p.D == 128) return fp16 ? launch<128, 1>(p, stream) : launch<128, 0>(p, stream);
  if (p.D == 64) return fp16 ? launch<64, 1>(p, stream) : launch<64, 0>(p, stream);
  return -3;
}

int launch_gather_rate_probe(const GatherAttnParams& p, int elem_bytes, cudaStream_t stream) {
  if (p.gi == nullptr || p.dense || (p.D != 64 && p.D != 128) || (elem_bytes != 1 && elem_bytes != 2)) return -3;
  const int rb = p.D * elem_bytes;
  const long long items = (long long)p.B * p.H * p.M;
  const int grid = (int)(items < num_sms() ? items : num_sms());
  auto run = [&](auto kern, int tile_bytes) {
    const int smem = 6 * tile_bytes + 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -8;
    kern<<<grid, kProducerThreads, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -8;
  };
  if (rb == 256) return run(gather_rate_probe_kernel<256>, 32768);
  if (rb == 128) return run(gather_rate_probe_kernel<128>, 16384);
  return -3;          // 64-byte rows (8-bit, D = 64) are not a configuration of the attention kernel
}

int launch_gather_attn_e4m3(const GatherAttnParams& p, cudaStream_t stream) {
  if (p.D == 128) return launch<128, 2>(p, stream);
  return -3;
}

}  // namespace mcs
