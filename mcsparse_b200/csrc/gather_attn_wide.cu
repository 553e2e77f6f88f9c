// Gather-KV sparse flash-attention forward for the head dimensions the main kernel has no instantiation for:
// any multiple of 8 up to 256 other than 64 and 128 (96, 144, 160, 192, 256 ...) for bf16 / fp16, and any multiple
// of 16 up to 256 other than 128 for e4m3 (the reference's FP8 kernel lists 128 and 160).
//
// The reference pads 144 to 160 in its wrapper and keeps one compiled kernel per padded size
// (mcsparse/kernels/flash_mcsa/ops/flash_sparse_attn/cute/interface.py:45-74, :138-159).  Here the padding happens
// on the way into shared memory: a row is copied in 16-byte chunks into NB = ceil(row bytes / 128) swizzled column
// blocks and the chunks beyond the row are zero-filled, so no padded copy of Q, K or V exists in global memory.
//
// Same math and the same argument block as the main kernel (gather_attn.cu); a simpler schedule, because these
// sizes leave less room: with D = 256 a K or V tile is 64 KB and the output accumulator takes 256 of the 512
// tensor-memory columns.  One CTA per work item (one query group of one (batch, head)), 9 warps:
//   warps 0-3  softmax + epilogue, thread == query row == tensor-memory lane, all 128 columns of a tile
//   warps 4-7  producers: 16-byte cp.async row gathers of Q, then K(0), K(1), V(0), K(2), V(1), ... into a ring
//              of 2-4 tile slots
//   warp 8     issues S = Q K^T (SS) and O += P V (P from tensor memory, V as an MN-major operand) in the order
//              QK(0), QK(1), PV(0), QK(2), PV(1), ...: the product of tile g+1 runs under the softmax of tile g.
// Tensor memory: S 128 columns, P 64, O up to 256.  Every mbarrier wait is bounded and reports through the status
// word; a role whose wait expires leaves its loop, the others follow through their own bounded waits.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.cuh"
#include "ptx.cuh"

namespace mcs {

namespace {

constexpr int kTileN = 128;
constexpr int kThreadsW = 288;
constexpr int kProducerWarp0W = 4;
constexpr int kProducerThreadsW = 128;
constexpr int kMmaWarpW = 8;
constexpr uint32_t kColSW = 0, kColPW = 128, kColOW = 192;

enum {
  WB_FULL = 0,              // [4] producers -> issuer
  WB_EMPTY = 4,             // [4] issuer -> producers
  WB_Q_FULL = 8,
  WB_S_FULL,                // scores of a tile complete
  WB_S_FREE,                // every softmax thread has copied its scores out
  WB_P_READY,               // probabilities of a tile stored
  WB_PV_DONE,               // P V of a tile complete: P reusable, O stable
  WB_DRAIN,
  WB_COUNT
};

template <int NB>
struct SmemW {
  static constexpr int kTileBytes = NB * 16384;                // 128 rows x NB column blocks of 128 bytes
  static constexpr int kRing = NB <= 2 ? 4 : (NB == 3 ? 3 : 2);
  static constexpr int kQ = 0;
  static constexpr int kRingOff = kTileBytes;
  static constexpr int kBars = kRingOff + kRing * kTileBytes;
  static constexpr int kTmemSlot = kBars + WB_COUNT * 8;
  static constexpr int kTotal = kTmemSlot + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

// One warp copies tile rows row0..row0+31: lane r holds the source row of tile row row0 + r (negative: zero row).
// Eight lanes cover 128 contiguous bytes of a row, four rows per instruction; chunks at or beyond d_chunks
// (the padding up to the next multiple of 64 elements) are zero-filled.
template <int NB>
__device__ __forceinline__ void warp_gather_rows_w(uint32_t s_tile, int row0, int my_row_idx, const uint8_t* base,
                                                   size_t row_bytes, int d_chunks, int lane) {
  const int c8 = lane & 7, sub = lane >> 3;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rl = i * 4 + sub;
    const int id = __shfl_sync(0xffffffffu, my_row_idx, rl);
    const int row = row0 + rl;
    const uint32_t dst = s_tile + row * 128 + ((c8 ^ (row & 7)) << 4);
#pragma unroll
    for (int blk = 0; blk < NB; ++blk) {
      const int c = blk * 8 + c8;
      if (id >= 0 && c < d_chunks) cp_async16(dst + blk * 16384, base + (size_t)id * row_bytes + c * 16);
      else cp_async16_zfill(dst + blk * 16384, base, 0);
    }
  }
}

// kType: 0 = bf16, 1 = fp16, 2 = e4m3 (Q/K/V 8-bit, logits scaled by scale_qk_log2[b,h,m], P quantised to e4m3 with a
// bias of 2^4, O scaled by scale_v[b,h], bf16 out: the contract of the main kernel's e4m3 instantiation)
template <int NB, int kType>
__global__ void __launch_bounds__(kThreadsW, 1) gather_attn_wide_kernel(const GatherAttnParams p) {
  constexpr bool kFp16 = kType == 1;
  constexpr bool kFp8 = kType == 2;
  constexpr int kEs = kFp8 ? 1 : 2;                   // bytes per Q/K/V element
  using L = SmemW<NB>;
  constexpr int R = L::kRing;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bars = s_base + L::kBars;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  auto bar = [&](int i) { return bars + 8u * i; };
  auto sRing = [&](int slot) { return s_base + L::kRingOff + slot * L::kTileBytes; };
  const uint32_t sQ = s_base + L::kQ;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);

  // ---- the work item of this CTA
  const int item = blockIdx.x;
  const int m = item % p.M, bh = item / p.M, h = bh % p.H, b = bh / p.H;
  const int row_base = m * p.group_rows;
  const int rows_valid = min(p.group_rows, p.Sq - row_base);
  int T = p.gather_len / kTileN;
  if (p.gl != nullptr) T = min(max(p.gl[item], 1), T);
  const int d_chunks = p.D * kEs / 16;            // 16-byte chunks of a Q/K/V row
  const int ksteps = (p.D * kEs + 31) / 32;       // k-steps of Q K^T (32 bytes of every row each)
  const int n_pv = (p.D + 15) / 16 * 16;          // output columns the P V product computes
  const int o_chunks = p.D / 8;                   // 16-byte chunks of an output row (16-bit elements)

  if (tid == 0) {
    for (int i = 0; i < R; ++i) {
      mbar_init(bar(WB_FULL + i), kProducerThreadsW);
      mbar_init(bar(WB_EMPTY + i), 1);
    }
    mbar_init(bar(WB_Q_FULL), kProducerThreadsW);
    mbar_init(bar(WB_S_FULL), 1);
    mbar_init(bar(WB_S_FREE), 4);
    mbar_init(bar(WB_P_READY), 4);
    mbar_init(bar(WB_PV_DONE), 1);
    mbar_init(bar(WB_DRAIN), 1);
    mbar_fence_init();
  }
  // S 128 + P 64 + O: 16-bit heads of up to 64 leave room for two CTAs per SM, each with half of tensor memory
  constexpr uint32_t kTmemColsW = (NB == 1 && !kFp8) ? 256 : 512;
  if (warp == kMmaWarpW) {
    tmem_alloc(smem_u32(tmem_slot), kTmemColsW);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) {
    // ===================================================================== softmax and epilogue
    auto warp_arrive = [&](uint32_t bb) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bb);
    };
    const int r_in = warp * 32 + lane;
    const uint32_t lane_addr = (static_cast<uint32_t>(warp) * 32u) << 16;
    const float scale_log2 = kFp8 ? p.scale_qk_log2[item] : p.scale_log2;
    // lazy raise of the running maximum with the thresholds of the main kernel; e4m3 P is biased by 2^4 so that the
    // largest probability of a row lies in [2^4, 2^8]
    constexpr float kRescale = kFp8 ? 4.0f : (kFp16 ? 12.0f : 24.0f);
    constexpr float kBias = kFp8 ? 4.0f : 0.0f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int g = 0; g < T && ok; ++g) {
      ok = mbar_wait(bar(WB_S_FULL), g & 1, p.status, 60);
      if (!ok) break;
      tc_fence_after();
      uint32_t sc[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tmem + kColSW + c * 32 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&sc[c * 32]));
      tmem_wait_ld();
      tc_fence_before();
      warp_arrive(bar(WB_S_FREE));
      if (p.dense && g == T - 1) {
        const int rem = p.Sk - g * kTileN;                // valid key columns of the last tile
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i >= rem) sc[i] = 0xff800000u;
      }
      float mx0 = __uint_as_float(sc[0]), mx1 = __uint_as_float(sc[1]), mx2 = __uint_as_float(sc[2]), mx3 = __uint_as_float(sc[3]);
#pragma unroll
      for (int i = 4; i < 128; i += 8) {
        mx0 = fmax3(mx0, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
        if (i + 4 < 128) {
          mx2 = fmax3(mx2, __uint_as_float(sc[i + 4]), __uint_as_float(sc[i + 5]));
          mx3 = fmax3(mx3, __uint_as_float(sc[i + 6]), __uint_as_float(sc[i + 7]));
        }
      }
      const float m_loc = fmaxf(fmax3(mx0, mx1, mx2), mx3) * scale_log2;
      bool raise = (m_loc - m_run) > kRescale;
      if constexpr (kFp8) {
        // a new maximum that would hold more than an eighth of the mass so far becomes the reference point at once:
        // its e4m3 probability is then exact (see the main kernel)
        raise = raise || ((m_loc > m_run) && (ex2_approx(m_loc - m_run + kBias) > 0.125f * l_run));
      }
      const float alpha = raise ? ex2_approx(m_run - m_loc) : 1.f;
      if (raise) m_run = m_loc;
      const float neg_m = kBias - m_run;
      // exponentials and packing first (registers only), then the wait for the previous P V
      uint32_t pk[64];
      float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(sc[i]), scale_log2, neg_m));
        const float p1 = ex2_approx(fmaf(__uint_as_float(sc[i + 1]), scale_log2, neg_m));
        const float p2 = ex2_approx(fmaf(__uint_as_float(sc[i + 2]), scale_log2, neg_m));
        const float p3 = ex2_approx(fmaf(__uint_as_float(sc[i + 3]), scale_log2, neg_m));
        ls0 += p0; ls1 += p1; ls2 += p2; ls3 += p3;
        if constexpr (kFp8) {
          pk[i / 4] = pack_e4m3x4(p0, p1, p2, p3);
        } else {
          pk[i / 2] = kFp16 ? pack_f16x2(p0, p1) : pack_bf16x2(p0, p1);
          pk[i / 2 + 1] = kFp16 ? pack_f16x2(p2, p3) : pack_bf16x2(p2, p3);
        }
      }
      l_run = l_run * alpha + ((ls0 + ls1) + (ls2 + ls3));
      if (g > 0) {
        // P and O are free once P V of the previous tile has completed
        ok = mbar_wait(bar(WB_PV_DONE), (g - 1) & 1, p.status, 61);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, raise)) {
          const uint32_t tO = tmem + kColOW + lane_addr;
#pragma unroll 1
          for (int c = 0; c < n_pv / 8; ++c) {
            uint32_t r[8];
            tmem_ld8(tO + c * 8, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st8(tO + c * 8, r);
          }
        }
      }
      const uint32_t tP = tmem + kColPW + lane_addr;
#pragma unroll
      for (int c = 0; c < (kFp8 ? 4 : 8); ++c) tmem_st8(tP + c * 8, *reinterpret_cast<uint32_t(*)[8]>(&pk[c * 8]));
      tmem_wait_st();
      tc_fence_before();
      warp_arrive(bar(WB_P_READY));
    }
    if (ok) ok = mbar_wait(bar(WB_PV_DONE), (T - 1) & 1, p.status, 62);
    if (ok) {
      tc_fence_after();
      // ---- epilogue: out = sign * O / l + residual, one rounding; the row goes to its original position
      const bool valid = r_in < rows_valid;
      const int row = row_base + r_in;
      long long orow = row;
      if (valid && p.perm != nullptr && !p.out_group_order) orow = p.perm[(size_t)bh * p.Sq + row];
      uint8_t* obase = reinterpret_cast<uint8_t*>(p.out);
      long long lrow = orow;
      if (p.n_out_peers > 0) {
        const int peer = static_cast<int>(orow / p.out_rows_per_peer);
        lrow = orow - (long long)peer * p.out_rows_per_peer;
        obase = reinterpret_cast<uint8_t*>(p.out_peer[valid ? peer : 0]);
      }
      uint8_t* optr = obase + 2 * ((size_t)b * p.o_stride[0] + (size_t)lrow * p.o_stride[1] + (size_t)h * p.o_stride[2]);
      const uint8_t* rptr = p.residual == nullptr ? nullptr
          : reinterpret_cast<const uint8_t*>(p.residual) + 2 * ((size_t)b * p.r_stride[0] + (size_t)h * p.r_stride[1] + (size_t)row * p.r_stride[2]);
      const float w = p.out_sign * (kFp8 ? p.scale_v[bh] : 1.f) / l_run;
      const uint32_t tO = tmem + kColOW + lane_addr;
#pragma unroll 1
      for (int c = 0; c < o_chunks; ++c) {
        uint32_t ra[8];
        tmem_ld8(tO + c * 8, ra);
        tmem_wait_ld();
        if (valid) {
          uint4 res = make_uint4(0, 0, 0, 0);
          if (rptr != nullptr) res = *reinterpret_cast<const uint4*>(rptr + c * 16);
          const uint32_t rw[4] = {res.x, res.y, res.z, res.w};
          uint32_t ow[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float rx, ry;
            if constexpr (kFp16) {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&rw[j]));
              rx = f.x; ry = f.y;
            } else {
              rx = bf16_lo(rw[j]); ry = bf16_hi(rw[j]);
            }
            const float o0 = fmaf(__uint_as_float(ra[2 * j]), w, rx);
            const float o1 = fmaf(__uint_as_float(ra[2 * j + 1]), w, ry);
            ow[j] = kFp16 ? pack_f16x2(o0, o1) : pack_bf16x2(o0, o1);
          }
          *reinterpret_cast<uint4*>(optr + c * 16) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
      }
      if (valid && p.lse != nullptr) p.lse[(size_t)bh * p.Sq + orow] = (m_run + lg2_approx(l_run) - kBias) * 0.6931471805599453f;
    }
    tc_fence_before();
  } else if (warp < kMmaWarpW) {
    // ===================================================================== producers
    const int pw = warp - kProducerWarp0W;
    const int row0 = pw * 32;
    const int my_row = row0 + lane;
    const size_t q_row = kEs * (size_t)p.q_stride[1], k_row = kEs * (size_t)p.k_stride[1], v_row = kEs * (size_t)p.v_stride[1];
    const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q) + kEs * ((size_t)b * p.q_stride[0] + (size_t)h * p.q_stride[2]);
    const uint8_t* kb = reinterpret_cast<const uint8_t*>(p.k) + kEs * ((size_t)b * p.k_stride[0] + (size_t)h * p.k_stride[2]);
    const uint8_t* vb = reinterpret_cast<const uint8_t*>(p.v) + kEs * ((size_t)b * p.v_stride[0] + (size_t)h * p.v_stride[2]);
    {
      int src_row = -1;
      if (my_row < rows_valid) {
        src_row = row_base + my_row;
        if (p.perm != nullptr) src_row = static_cast<int>(p.perm[(size_t)bh * p.Sq + src_row]);
      }
      warp_gather_rows_w<NB>(sQ, row0, src_row, qb, q_row, d_chunks, lane);
      cp_async_arrive_noinc(bar(WB_Q_FULL));
    }
    const size_t ioff = (size_t)item * p.gather_len + my_row;
    auto load_idx = [&](int g) -> int {
      int idx;
      if (p.dense) {
        idx = g * kTileN + my_row;
      } else if (p.gi16 != nullptr) {
        const size_t o = ioff + (size_t)g * kTileN;
        const uint32_t lo = __ldg(p.gi16 + o), hi = (__ldg(p.gi_hi + (o >> 5)) >> (o & 31)) & 1u;
        idx = static_cast<int>(lo | (hi << 16));
      } else {
        idx = __ldg(p.gi + ioff + (size_t)g * kTileN);
      }
      return min(max(idx, 0), p.Sk - 1);
    };
    int held0 = 0, held1 = 0;        // indices of the two key tiles whose V tile is still to come
    int idx_next = load_idx(0);
    bool ok = true;
#pragma unroll 1
    for (int e = 0; e < 2 * T && ok; ++e) {
      // ring entries in the issuer's consumption order: K(0), K(1), V(0), K(2), V(1), ..., K(T-1), V(T-2), V(T-1)
      bool is_v;
      int g;
      if (e == 0) { is_v = false; g = 0; }
      else if (e == 2 * T - 1) { is_v = true; g = T - 1; }
      else if (e & 1) { is_v = false; g = (e + 1) >> 1; }
      else { is_v = true; g = (e >> 1) - 1; }
      const int slot = e % R, use = e / R;
      if (use > 0) ok = mbar_wait(bar(WB_EMPTY + slot), (use - 1) & 1, p.status, 63);
      if (!ok) break;
      int idx;
      if (is_v) {
        idx = (g & 1) ? held1 : held0;
      } else {
        idx = idx_next;
        if (g & 1) held1 = idx; else held0 = idx;
        if (g + 1 < T) idx_next = load_idx(g + 1);     // in flight while this tile's copies are issued
      }
      warp_gather_rows_w<NB>(sRing(slot), row0, idx, is_v ? vb : kb, is_v ? v_row : k_row, d_chunks, lane);
      cp_async_arrive_noinc(bar(WB_FULL + slot));
    }
    cp_async_wait_all();
    tc_fence_before();
  } else {
    // ===================================================================== issuer of both products
    constexpr uint32_t kFmt = (kFp16 || kFp8) ? 0u : 1u;   // kind::f16: 0 f16, 1 bf16; kind::f8f6f4: 0 e4m3
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, 128-byte swizzle
    auto desc = [&](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
    constexpr uint32_t kLboK = (16u >> 4) << 16;
    constexpr uint32_t kLboV = (16384u >> 4) << 16;        // MN-major V: 16 KB between 64-element column blocks
    const uint32_t idesc_qk = mma_idesc(kFmt, kFmt, 0, 0, 128, kTileN);
    const uint32_t idesc_pv = mma_idesc(kFmt, kFmt, 0, 1, 128, static_cast<uint32_t>(n_pv));
    const bool leader = elect_one();
    bool ok = true;
    auto issue_qk = [&](int g) {
      const int e = g == 0 ? 0 : 2 * g - 1;
      const int slot = e % R, use = e / R;
      if (g == 0) ok = mbar_wait(bar(WB_Q_FULL), 0, p.status, 64);
      ok = ok && mbar_wait(bar(WB_FULL + slot), use & 1, p.status, 65);
      if (g > 0) ok = ok && mbar_wait(bar(WB_S_FREE), (g - 1) & 1, p.status, 66);
      if (!ok) return;
      fence_proxy_async_smem();
      tc_fence_after();
      const uint32_t qlo = ((sQ & 0x3FFFFu) >> 4) | kLboK;
      const uint32_t klo = ((sRing(slot) & 0x3FFFFu) >> 4) | kLboK;
#pragma unroll 1
      for (int j = 0; j < ksteps; ++j) {
        const uint32_t koff = (j >> 2) * (16384 >> 4) + (j & 3) * 2;
        if (leader) {
          if constexpr (kFp8) mma_f8_ss(tmem + kColSW, desc(qlo + koff), desc(klo + koff), idesc_qk, j > 0);
          else mma_f16_ss(tmem + kColSW, desc(qlo + koff), desc(klo + koff), idesc_qk, j > 0);
        }
      }
      if (leader) {
        tc_commit(bar(WB_EMPTY + slot));
        tc_commit(bar(WB_S_FULL));
      }
    };
    auto issue_pv = [&](int g) {
      const int e = g < T - 1 ? 2 * g + 2 : 2 * T - 1;
      const int slot = e % R, use = e / R;
      ok = mbar_wait(bar(WB_FULL + slot), use & 1, p.status, 67) && mbar_wait(bar(WB_P_READY), g & 1, p.status, 68);
      if (!ok) return;
      fence_proxy_async_smem();
      tc_fence_after();
      const uint32_t vlo = ((sRing(slot) & 0x3FFFFu) >> 4) | kLboV;
      if constexpr (kFp8) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // A: 32 e4m3 probabilities = 8 tensor-memory columns per k-step; B: 32 key rows = 4096 bytes
          if (leader) mma_f8_ts(tmem + kColOW, tmem + kColPW + j * 8, desc(vlo + j * (4096 >> 4)), idesc_pv, (g > 0) || (j > 0));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // A: 16 packed probabilities = 8 tensor-memory columns per k-step; B: 16 key rows = 2048 bytes
          if (leader) mma_f16_ts(tmem + kColOW, tmem + kColPW + j * 8, desc(vlo + j * (2048 >> 4)), idesc_pv, (g > 0) || (j > 0));
        }
      }
      if (leader) {
        tc_commit(bar(WB_EMPTY + slot));
        tc_commit(bar(WB_PV_DONE));
      }
    };
    issue_qk(0);
#pragma unroll 1
    for (int g = 0; g < T && ok; ++g) {
      if (g + 1 < T) issue_qk(g + 1);
      if (!ok) break;
      issue_pv(g);
    }
    if (!ok) {
      // error path: let outstanding products retire before tensor memory is released
      if (leader) tc_commit(bar(WB_DRAIN));
      mbar_wait_quiet(bar(WB_DRAIN), 0, 1 << 20);
    }
    __syncwarp();
    tc_fence_before();
  }

  __syncthreads();
  if (warp == kMmaWarpW) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemColsW);
  }
}

template <int NB, int kType>
int launch_wide(const GatherAttnParams& p, cudaStream_t stream) {
  using L = SmemW<NB>;
  auto kern = gather_attn_wide_kernel<NB, kType>;
  // an 8-bit head of up to 128 fits one 128-byte block but needs all of tensor memory: ask for enough shared memory
  // that only one such CTA is resident per SM
  const int smem = (kType == 2 && NB == 1 && L::kDynamic < 120 * 1024) ? 120 * 1024 : L::kDynamic;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -8;
  const long long items = (long long)p.B * p.H * p.M;
  kern<<<static_cast<unsigned>(items), kThreadsW, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace

int launch_gather_attn_wide(const GatherAttnParams& p, bool fp16, cudaStream_t stream) {
  if (p.D < 8 || p.D > 256 || p.D % 8 != 0 || p.group_rows > 128) return -3;
  const int nb = (p.D + 63) / 64;
  switch (nb) {
    case 1: return fp16 ? launch_wide<1, 1>(p, stream) : launch_wide<1, 0>(p, stream);
    case 2: return fp16 ? launch_wide<2, 1>(p, stream) : launch_wide<2, 0>(p, stream);
    case 3: return fp16 ? launch_wide<3, 1>(p, stream) : launch_wide<3, 0>(p, stream);
    default: return fp16 ? launch_wide<4, 1>(p, stream) : launch_wide<4, 0>(p, stream);
  }
}

int launch_gather_attn_wide_e4m3(const GatherAttnParams& p, cudaStream_t stream) {
  if (p.D < 16 || p.D > 256 || p.D % 16 != 0 || p.group_rows > 128) return -3;
  return p.D <= 128 ? launch_wide<1, 2>(p, stream) : launch_wide<2, 2>(p, stream);
}

}  // namespace mcs
