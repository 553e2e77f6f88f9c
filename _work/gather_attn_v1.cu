// Gather-KV sparse flash-attention forward for sm_100a (bf16 / fp16).
//
// One CTA per (batch, head, query group).  A query group is up to 128 rows of
// the (optionally permuted) query sequence that share one list of selected KV
// token indices.  Per 128-token KV tile:
//
//   producer warps   gather the tile's K rows and V rows with 16-byte cp.async
//                    (16 lanes cover one 256-byte row, so every warp request is
//                    two fully used 256-byte segments) into 128-byte-swizzled
//                    shared memory in the canonical tcgen05 operand layout;
//   MMA warp         one thread issues S = Q K^T (tcgen05.mma, operands in shared
//                    memory, accumulator in tensor memory) and O += P V (P read
//                    from tensor memory, V as an MN-major shared-memory operand);
//   softmax warps    thread r owns query row r == TMEM lane r: reads its S row
//                    with tcgen05.ld, keeps the online-softmax state in
//                    registers (log2 domain, lazy rescale of O), writes P back
//                    into the S columns as packed 16-bit values.
//
// Two CTAs are resident per SM (96 KB shared memory and 256 TMEM columns each),
// so one CTA's softmax overlaps the other's tensor-core work.
//
// The epilogue normalises O, adds the cached dense-minus-sparse residual in fp32,
// rounds once to the output type and scatters rows back to the original token
// order when a permutation is given.
//
// Follows the math of the reference's Hopper kernel
// (mcsparse/kernels/flash_mcsa/ops/flash_sparse_attn/cute/flash_fwd_sm90.py:1005-1340,
// softmax.py:126-227) and the gather addressing of topk_gather_kv.py:351-445.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.cuh"
#include "ptx.cuh"

namespace mcs {

namespace {

constexpr int kTileN = 128;          // KV tokens per tile
constexpr int kThreads = 288;        // 4 softmax warps + 4 producer warps + 1 MMA warp
constexpr int kSoftmaxThreads = 128;
constexpr int kProducerThreads = 128;
constexpr int kMmaWarp = 8;
constexpr uint32_t kTmemCols = 256;  // S: [0,128)  O: [128, 128+D)
constexpr float kRescaleThreshold = 8.0f;  // log2 units; P stays <= 2^8

// mbarrier slots
enum { BAR_Q_FULL = 0, BAR_K_FULL, BAR_V_FULL, BAR_K_EMPTY, BAR_V_EMPTY, BAR_S_FULL, BAR_P_READY, BAR_O_FULL,
       BAR_DRAIN, BAR_COUNT };

template <int D>
struct Smem {
  static constexpr int kBlocks = D / 64;                 // 64-element (128-byte) column blocks
  static constexpr int kTileBytes = kBlocks * 16384;     // 128 rows x D x 2 bytes
  static constexpr int kQ = 0;
  static constexpr int kK = kTileBytes;
  static constexpr int kV = 2 * kTileBytes;
  static constexpr int kBars = 3 * kTileBytes;
  static constexpr int kTmemSlot = kBars + BAR_COUNT * 8;
  static constexpr int kTotal = kTmemSlot + 16;
  static constexpr int kDynamic = kTotal + 1024;         // slack for 1024-byte alignment
};

// Byte offset of 16-byte chunk `c` of row `row` inside a swizzled operand tile.
__device__ __forceinline__ uint32_t swz_off(int row, int c) {
  return static_cast<uint32_t>((c >> 3) * 16384 + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}

// One warp copies 32 rows of D 16-bit elements.  `row_ptr_of_lane` is the global
// address of row (row0 + lane); rows with a null pointer are zero-filled.
template <int D>
__device__ __forceinline__ void warp_gather_rows(uint32_t s_tile, int row0, const uint8_t* row_ptr_of_lane,
                                                 const uint8_t* any_valid, int lane) {
  constexpr int kChunks = D / 8;             // 16-byte chunks per row
  constexpr int kRowsPerInstr = 32 / kChunks;
  const int sub = lane / kChunks;
  const int c = lane % kChunks;
#pragma unroll
  for (int i = 0; i < 32 / kRowsPerInstr; ++i) {
    const int rl = i * kRowsPerInstr + sub;
    const unsigned long long p =
        __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(row_ptr_of_lane), rl);
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p);
    const uint32_t dst = s_tile + swz_off(row0 + rl, c);
    if (src != nullptr) {
      cp_async16(dst, src + c * 16);
    } else {
      cp_async16_zfill(dst, any_valid, 0);
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

template <int D, bool kFp16>
__global__ void __launch_bounds__(kThreads, 2) gather_attn_kernel(const GatherAttnParams p) {
  using L = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t sQ = s_base + L::kQ, sK = s_base + L::kK, sV = s_base + L::kV;
  const uint32_t bars = s_base + L::kBars;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  auto bar = [&](int i) { return bars + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- work assignment: m fastest so that resident CTAs share one head's K/V in L2
  const int M = p.M;
  const int m = blockIdx.x % M;
  const int bh = blockIdx.x / M;
  const int h = bh % p.H;
  const int b = bh / p.H;
  const int row_base = m * p.group_rows;
  const int rows_valid = min(p.group_rows, p.Sq - row_base);
  const int max_tiles = p.gather_len / kTileN;
  int T = max_tiles;
  if (p.gl != nullptr) T = min(max(p.gl[(size_t)bh * M + m], 1), max_tiles);
  const int32_t* gi = p.gi + ((size_t)bh * M + m) * p.gather_len;

  // ---- setup
  if (tid == 0) {
    mbar_init(bar(BAR_Q_FULL), kProducerThreads);
    mbar_init(bar(BAR_K_FULL), kProducerThreads);
    mbar_init(bar(BAR_V_FULL), kProducerThreads);
    mbar_init(bar(BAR_K_EMPTY), 1);
    mbar_init(bar(BAR_V_EMPTY), 1);
    mbar_init(bar(BAR_S_FULL), 1);
    mbar_init(bar(BAR_P_READY), kSoftmaxThreads);
    mbar_init(bar(BAR_O_FULL), 1);
    mbar_init(bar(BAR_DRAIN), 1);
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
  const uint32_t tS = tmem;          // fp32 scores, 128 columns; P (16-bit) reuses columns [0,64)
  const uint32_t tO = tmem + 128;    // fp32 output accumulator, D columns

  if (warp < 4) {
    // =====================================================================
    // softmax / correction / epilogue: thread == query row == TMEM lane
    // =====================================================================
    const uint32_t lane_addr = (static_cast<uint32_t>(warp) * 32u) << 16;
    const float scale_log2 = p.scale_log2;
    float m_run = -INFINITY;   // running (possibly stale) row max, log2 domain
    float l_run = 0.f;         // running row sum relative to m_run
    bool ok = true;
#pragma unroll 1
    for (int t = 0; t < T && ok; ++t) {
      ok = mbar_wait(bar(BAR_S_FULL), t & 1, p.status, 10);
      if (!ok) break;
      tc_fence_after();
      // pass 1: row max of this tile
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + lane_addr + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
      }
      const float m_new = fmaxf(m_run, mx * scale_log2);
      if (t == 0) {
        m_run = m_new;
      } else {
        const bool need = (m_new - m_run) > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? ex2_approx(m_run - m_new) : 1.f;
          if (need) m_run = m_new;
          l_run *= alpha;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + lane_addr + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tO + lane_addr + c * 32, r);
          }
        }
      }
      // pass 2: P = exp2(S*scale - m), row sum, write P as packed 16-bit values
      const float neg_m = -m_run;
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + lane_addr + c * 32, r);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * i]), scale_log2, neg_m));
          const float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), scale_log2, neg_m));
          lsum += p0 + p1;
          pk[i] = pack16<kFp16>(p0, p1);
        }
        tmem_st16(tS + lane_addr + c * 16, pk);
      }
      l_run += lsum;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(BAR_P_READY));
    }
    // ---- epilogue
    if (ok) ok = mbar_wait(bar(BAR_O_FULL), 0, p.status, 11);
    if (ok) {
      tc_fence_after();
      const int r_in = warp * 32 + lane;
      const bool valid = r_in < rows_valid;
      const int row = row_base + r_in;                      // position in (permuted) query order
      long long orow = row;
      if (valid && p.perm != nullptr) orow = p.perm[(size_t)bh * p.Sq + row];
      const float inv_l = 1.f / l_run;
      uint8_t* optr = reinterpret_cast<uint8_t*>(p.out) +
                      2 * ((size_t)b * p.o_stride[0] + (size_t)orow * p.o_stride[1] + (size_t)h * p.o_stride[2]);
      const uint8_t* rptr = nullptr;
      if (p.residual != nullptr)
        rptr = reinterpret_cast<const uint8_t*>(p.residual) +
               2 * ((size_t)b * p.r_stride[0] + (size_t)h * p.r_stride[1] + (size_t)row * p.r_stride[2]);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + lane_addr + c * 32, r);
        tmem_wait_ld();
        if (valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 res = make_uint4(0, 0, 0, 0);
            if (rptr != nullptr) res = *reinterpret_cast<const uint4*>(rptr + c * 64 + q4 * 16);
            const uint32_t rw[4] = {res.x, res.y, res.z, res.w};
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 rr = unpack16<kFp16>(rw[j]);
              const float o0 = fmaf(__uint_as_float(r[q4 * 8 + 2 * j]), inv_l, rr.x);
              const float o1 = fmaf(__uint_as_float(r[q4 * 8 + 2 * j + 1]), inv_l, rr.y);
              ow[j] = pack16<kFp16>(o0, o1);
            }
            *reinterpret_cast<uint4*>(optr + c * 64 + q4 * 16) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        }
      }
      if (valid && p.lse != nullptr) {
        // natural-log LSE of the scaled logits
        p.lse[(size_t)bh * p.Sq + orow] = (m_run + lg2_approx(l_run)) * 0.6931471805599453f;
      }
    }
    tc_fence_before();
  } else if (warp < 8) {
    // =====================================================================
    // producers: gather Q once, then K/V tiles
    // =====================================================================
    const int pw = warp - 4;
    const int row0 = pw * 32;
    const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q);
    const uint8_t* kb = reinterpret_cast<const uint8_t*>(p.k) + 2 * ((size_t)b * p.k_stride[0] + (size_t)h * p.k_stride[2]);
    const uint8_t* vb = reinterpret_cast<const uint8_t*>(p.v) + 2 * ((size_t)b * p.v_stride[0] + (size_t)h * p.v_stride[2]);
    const size_t k_row = 2 * (size_t)p.k_stride[1], v_row = 2 * (size_t)p.v_stride[1];
    {
      const int r_in = row0 + lane;
      const uint8_t* qrow = nullptr;
      if (r_in < rows_valid) {
        long long src_row = row_base + r_in;
        if (p.perm != nullptr) src_row = p.perm[(size_t)bh * p.Sq + src_row];
        qrow = qb + 2 * ((size_t)b * p.q_stride[0] + (size_t)src_row * p.q_stride[1] + (size_t)h * p.q_stride[2]);
      }
      warp_gather_rows<D>(sQ, row0, qrow, qb, lane);
      cp_async_commit();
    }
    int idx = min(max(gi[row0 + lane], 0), p.Sk - 1);
    bool ok = true;
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
      if (t > 0) {
        ok = mbar_wait(bar(BAR_K_EMPTY), (t - 1) & 1, p.status, 20);
        if (!ok) break;
      }
      warp_gather_rows<D>(sK, row0, kb + (size_t)idx * k_row, kb, lane);
      cp_async_commit();
      if (t > 0) {
        ok = mbar_wait(bar(BAR_V_EMPTY), (t - 1) & 1, p.status, 21);
        if (!ok) break;
      }
      warp_gather_rows<D>(sV, row0, vb + (size_t)idx * v_row, vb, lane);
      cp_async_commit();
      if (t + 1 < T) idx = min(max(gi[(t + 1) * kTileN + row0 + lane], 0), p.Sk - 1);
      if (t == 0) {
        cp_async_wait<2>();
        fence_proxy_async_smem();
        mbar_arrive(bar(BAR_Q_FULL));
      }
      cp_async_wait<1>();
      fence_proxy_async_smem();
      mbar_arrive(bar(BAR_K_FULL));
      cp_async_wait<0>();
      fence_proxy_async_smem();
      mbar_arrive(bar(BAR_V_FULL));
    }
    cp_async_wait<0>();
  } else {
    // =====================================================================
    // MMA issuer: one thread
    // =====================================================================
    if (lane == 0) {
      constexpr uint32_t kFmt = kFp16 ? 0u : 1u;
      constexpr uint32_t idesc_qk = mma_idesc(kFmt, kFmt, 0, 0, 128, kTileN);
      constexpr uint32_t idesc_pv = mma_idesc(kFmt, kFmt, 0, 1, 128, D);
      bool ok = mbar_wait(bar(BAR_Q_FULL), 0, p.status, 30);
#pragma unroll 1
      for (int t = 0; t < T && ok; ++t) {
        ok = mbar_wait(bar(BAR_K_FULL), t & 1, p.status, 31);
        if (!ok) break;
        fence_proxy_async_smem();
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
          const uint32_t koff = (j >> 2) * 16384 + (j & 3) * 32;
          mma_f16_ss(tS, smem_desc_sw128(sQ + koff, 16, 1024), smem_desc_sw128(sK + koff, 16, 1024), idesc_qk,
                     j > 0);
        }
        tc_commit(bar(BAR_K_EMPTY));
        tc_commit(bar(BAR_S_FULL));
        ok = mbar_wait(bar(BAR_V_FULL), t & 1, p.status, 32);
        if (!ok) break;
        ok = mbar_wait(bar(BAR_P_READY), t & 1, p.status, 33);
        if (!ok) break;
        fence_proxy_async_smem();
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < kTileN / 16; ++j) {
          // A: 16 packed 16-bit values = 8 TMEM columns per k-step; B: 16 KV rows = 2048 bytes
          mma_f16_ts(tO, tS + j * 8, smem_desc_sw128(sV + j * 2048, 16384, 1024), idesc_pv, (t > 0) || (j > 0));
        }
        tc_commit(bar(BAR_V_EMPTY));
        if (t == T - 1) tc_commit(bar(BAR_O_FULL));
      }
      if (!ok) {
        // error path: let outstanding MMAs retire before tensor memory is released
        tc_commit(bar(BAR_DRAIN));
        mbar_wait_quiet(bar(BAR_DRAIN), 0, 1 << 20);
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

template <int D, bool kFp16>
int launch(const GatherAttnParams& p, cudaStream_t stream) {
  using L = Smem<D>;
  auto kern = gather_attn_kernel<D, kFp16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
  if (e != cudaSuccess) return -8;
  const long long grid = (long long)p.B * p.H * p.M;
  kern<<<(unsigned)grid, kThreads, L::kDynamic, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace

int launch_gather_attn_16bit(const GatherAttnParams& p, bool fp16, cudaStream_t stream) {
  if (p.D == 128) return fp16 ? launch<128, true>(p, stream) : launch<128, false>(p, stream);
  if (p.D == 64) return fp16 ? launch<64, true>(p, stream) : launch<64, false>(p, stream);
  return -3;
}

}  // namespace mcs
