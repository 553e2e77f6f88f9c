// Anchor-step group mass for sm_100a:
//
//   mass[b,h,m,j] = sum_{i in query group m} exp(scale * q_i . k_j - lse_i)        (fp32)
//
// i.e. the exact attention probability mass that query group m puts on key token j, given
// the log-sum-exp of every query row from a dense attention pass.  Optionally divided by
// the number of rows in the group (the reference's "mean" convention).
//
// Restates the reference's Triton kernel
// (mcsparse/kernels/flash_mcsa/ops/triton/block_probs.py:27-89), with an fp32 result instead
// of one rounded to bf16.
//
// One CTA per (batch*head, group).  The 128 query rows of the group stay resident in shared
// memory; the CTA streams all key tiles of the head.  The product is computed TRANSPOSED,
// S^T = K_tile Q^T, so that a TMEM lane is a key token and the sum over the group's queries
// runs along the columns inside one thread: no cross-thread reduction at all.
//
// "- lse_i" is folded into the MMA: the contraction is extended by one 16-wide k-step whose K
// columns are (1, 1, 1, 0, ...) and whose Q columns are (-hi, -mid, -lo, 0, ...), a three-term
// bf16 split of lse_i / scale, exact to fp32 precision.  The tensor core then delivers
// q_i . k_j - lse_i / scale and each element costs one multiply, one ex2 and one add.
// The kernel is bound by the ex2 throughput of the SFU (16 per clock per SM); a quarter of the exponentials
// are therefore evaluated by a polynomial on the FMA pipe.
//
// Roles: warps 0-7 exponentiate and sum (two threads per key token: warps w and w+4 share a TMEM
// lane group and take 64 query columns each, so that every SM sub-partition has two warps feeding
// its SFU; the two partial sums meet in shared memory), warp 8 issues the MMAs (converged, one
// elected lane executes the tcgen05 instructions), warps 9-12 prepare the query operand
// and stream the key tiles into a 3-slot ring: by TMA (one elected thread, boxes of 128 rows x 128 bytes)
// when a tensor map can describe K's strides, else with cp.async.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.cuh"
#include "ptx.cuh"

namespace mcs {

namespace {

constexpr int kTile = 128;
constexpr int kThreads = 416;
constexpr int kExpWarps = 8;
constexpr int kProducerThreads = 128;
constexpr int kMmaWarp = 8;
constexpr int kProducerWarp0 = 9;
constexpr int kRing = 3;
constexpr uint32_t kTmemCols = 256;   // two score buffers of 128 columns

enum { BAR_FULL = 0, BAR_EMPTY = BAR_FULL + kRing, BAR_Q_FULL = BAR_EMPTY + kRing, BAR_S_FULL, BAR_S_FREE = BAR_S_FULL + 2,
       BAR_PART = BAR_S_FREE + 2,      // [4 lane groups][2 bufs]: partial sums of the upper column half are in shared memory
       BAR_DRAIN = BAR_PART + 8, BAR_COUNT };

// D is the head dimension rounded up to the tile layouts this kernel has: 64, 128, 192 or 256 (the true head
// dimension, any multiple of 8 up to 256, is a run-time value; rows are zero-padded on their way into shared memory)
template <int D>
struct Smem {
  static constexpr int kBlocks = D / 64;
  static constexpr int kTileBytes = kBlocks * 16384;
  static constexpr int kRingN = D == 256 ? 2 : kRing;        // key-tile slots that fit beside the query tile
  static constexpr int kQ = 0;                              // group's query rows (B operand)
  static constexpr int kQx = kTileBytes;                    // extra k-step of Q: 128 rows x 128 B (first 32 B used)
  static constexpr int kKx = kQx + 16384;                   // extra k-step of K: constant (1,1,1,0...)
  static constexpr int kRingOff = kKx + 16384;
  static constexpr int kBars = kRingOff + kRingN * kTileBytes;
  static constexpr int kPart = kBars + BAR_COUNT * 8;       // float [2][128]: partial sums of the upper column half
  static constexpr int kTmemSlot = kPart + 2 * 128 * 4;
  static constexpr int kTotal = kTmemSlot + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

static_assert(Smem<192>::kDynamic <= 232448 && Smem<256>::kDynamic <= 232448, "padded layouts must fit 227 KB");

__device__ __forceinline__ uint32_t swz(int row, int c) {   // 16-byte chunk c of row, 128-byte swizzle
  return static_cast<uint32_t>((c >> 3) * 16384 + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}

template <int D, bool kFp16, int kPoly>
__global__ void __launch_bounds__(kThreads, 1) group_mass_kernel(const GroupMassParams p, const __grid_constant__ KeyTileMap kmap) {
  // key tiles are 128 consecutive rows: with a valid tensor map one elected thread loads them by TMA
  const bool use_tma = kmap.valid != 0;
  using L = Smem<D>;
  constexpr bool kWide = D > 128;                       // padded layouts: the true head dimension is p.D < D
  constexpr int R = L::kRingN;
  const int d_chunks = p.D / 8;                          // 16-byte chunks of a real row
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bars = s_base + L::kBars;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  auto bar = [&](int i) { return bars + 8u * i; };
  auto sRing = [&](int slot) { return s_base + L::kRingOff + slot * L::kTileBytes; };
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);      // provably warp-uniform

  const int m = blockIdx.x % p.M;
  const int bh = blockIdx.x / p.M;
  const int h = bh % p.H, b = bh / p.H;
  const int row_base = m * p.group_rows;
  const int rows_valid = min(p.group_rows, p.Lq - row_base);
  const int n_tiles = (p.Lk + kTile - 1) / kTile;

  if (tid == 0) {
    for (int i = 0; i < R; ++i) {
      mbar_init(bar(BAR_FULL + i), use_tma ? 1 : kProducerThreads);
      mbar_init(bar(BAR_EMPTY + i), 1);
    }
    mbar_init(bar(BAR_Q_FULL), 2 * kProducerThreads);   // per thread: its cp.async rows + its plain stores
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_S_FULL + i), 1);
      mbar_init(bar(BAR_S_FREE + i), kExpWarps);
    }
    for (int i = 0; i < 8; ++i) mbar_init(bar(BAR_PART + i), 1);
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

  if (warp < kExpWarps) {
    // ===================================================================== exp + column sum
    const int lg = warp & 3, x = warp >> 2;            // TMEM lane group, column half
    const int j_in = lg * 32 + lane;                   // key token inside the tile == TMEM lane
    const uint32_t lane_addr = (static_cast<uint32_t>(lg) * 32u) << 16;
    const float c = p.scale_log2;
    const float xmin = -125.f / c;
    const float norm = p.normalize ? 1.f / static_cast<float>(rows_valid) : 1.f;
    float* out = p.mass + ((size_t)bh * p.M + m) * p.Lk;
    float* part = reinterpret_cast<float*>(smem + L::kPart);
    bool ok = true;
#pragma unroll 1
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int buf = t & 1;
      ok = mbar_wait(bar(BAR_S_FULL + buf), (t >> 1) & 1, p.status, 40);
      if (!ok) break;
      tc_fence_after();
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t r[32];
        tmem_ld32(tmem + buf * 128 + x * 64 + q * 32 + lane_addr, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          // kPoly of every eight exponentials are computed on the FMA pipe instead of the special-function unit,
          // which bounds this kernel (see ex2_poly3_scaled); their positions are spread over the four partial sums.
          // Two of eight measured best (7.84 ms against 8.29 ms with none and 8.10 / 8.36 ms with three / four at
          // H=24, L=32,760: beyond a quarter the extra instructions cost more issue slots than the unit gains).
          auto e = [&](int k) {
            const float v = __uint_as_float(r[i + k]);
            const bool poly = (kPoly >= 1 && k == 3) || (kPoly >= 2 && k == 6) || (kPoly >= 3 && k == 1) || (kPoly >= 4 && k == 4);
            return poly ? ex2_poly3_scaled(v, c, xmin) : ex2_approx(v * c);
          };
          a0 += e(0); a1 += e(1); a2 += e(2); a3 += e(3);
          a0 += e(4); a1 += e(5); a2 += e(6); a3 += e(7);
        }
      }
      tc_fence_before();
      const float sum = (a0 + a1) + (a2 + a3);
      // The two halves of a row meet in shared memory, double-buffered by tile parity and handed over
      // through an mbarrier (a bounded wait, unlike a named barrier).  The lower half releases the score
      // buffer only after it has read the partner's sums, so the partner's write two tiles later (which
      // needs that release to get its next scores) cannot overtake the read.  (Copying all 64 values to
      // registers first and releasing the score buffer before the exponentials measured 10% slower.)
      if (x == 1) {
        part[buf * 128 + j_in] = sum;
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar(BAR_PART + 2 * lg + buf));
          mbar_arrive(bar(BAR_S_FREE + buf));              // one arrival per warp
        }
      } else {
        ok = mbar_wait(bar(BAR_PART + 2 * lg + buf), (t >> 1) & 1, p.status, 45);
        if (!ok) break;
        const int j = t * kTile + j_in;
        if (j < p.Lk) out[j] = (sum + part[buf * 128 + j_in]) * norm;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_S_FREE + buf));
      }
    }
    tc_fence_before();
  } else if (warp == kMmaWarp) {
    // ===================================================================== MMA issuer
    {
      const bool leader = elect_one();
      constexpr uint32_t kFmt = kFp16 ? 0u : 1u;
      constexpr uint32_t idesc = mma_idesc(kFmt, kFmt, 0, 0, 128, 128);
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kLbo = (16u >> 4) << 16;
      auto desc = [&](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
      const uint32_t qlo = (((s_base + L::kQ) & 0x3FFFFu) >> 4) | kLbo;
      const uint32_t qxlo = (((s_base + L::kQx) & 0x3FFFFu) >> 4) | kLbo;
      const uint32_t kxlo = (((s_base + L::kKx) & 0x3FFFFu) >> 4) | kLbo;
      bool ok = mbar_wait(bar(BAR_Q_FULL), 0, p.status, 41);
      int slot = 0, phase = 0;
#pragma unroll 1
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int buf = t & 1;
        if (t >= 2) ok = mbar_wait(bar(BAR_S_FREE + buf), ((t >> 1) - 1) & 1, p.status, 42);
        ok = ok && mbar_wait(bar(BAR_FULL + slot), phase, p.status, 43);
        if (!ok) break;
        fence_proxy_async_smem();
        tc_fence_after();
        const uint32_t tS = tmem + buf * 128;
        const uint32_t klo = ((sRing(slot) & 0x3FFFFu) >> 4) | kLbo;
        if constexpr (kWide) {
          // the k-steps that hold real columns (the last one zero-padded to 16)
          const int ksteps = (p.D + 15) / 16;
#pragma unroll 1
          for (int j = 0; j < ksteps; ++j) {
            const uint32_t koff = (j >> 2) * (16384 >> 4) + (j & 3) * 2;
            if (leader) mma_f16_ss(tS, desc(klo + koff), desc(qlo + koff), idesc, j > 0);
          }
        } else {
#pragma unroll
          for (int j = 0; j < D / 16; ++j) {
            const uint32_t koff = (j >> 2) * (16384 >> 4) + (j & 3) * 2;
            if (leader) mma_f16_ss(tS, desc(klo + koff), desc(qlo + koff), idesc, j > 0);     // A = K tile, B = Q group
          }
        }
        if (leader) {
          mma_f16_ss(tS, desc(kxlo), desc(qxlo), idesc, 1);                     // extra k-step: - lse / scale
          tc_commit(bar(BAR_EMPTY + slot));
          tc_commit(bar(BAR_S_FULL + buf));
        }
        if (++slot == R) { slot = 0; phase ^= 1; }
      }
      if (!ok) {
        if (leader) tc_commit(bar(BAR_DRAIN));
        mbar_wait_quiet(bar(BAR_DRAIN), 0, 1 << 20);
      }
    }
    __syncwarp();
    tc_fence_before();
  } else {
    // ===================================================================== producers
    const int pw = warp - kProducerWarp0;
    const int ptid = pw * 32 + lane;                    // 0..127: also the row this thread prepares
    const int row0 = pw * 32;
    // one lane per 16-byte chunk of a row; the padded layouts give every lane one of 32 chunk positions, of which
    // D / 8 exist in the tile (the others idle) and p.D / 8 hold data (the rest is zero-filled)
    constexpr int kChunks = kWide ? 32 : D / 8;
    constexpr int kRowsPerInstr = 32 / kChunks;
    const int sub = lane / kChunks, cch = lane % kChunks;
    const bool c_in_tile = !kWide || cch < D / 8;
    const bool c_live = !kWide || cch < d_chunks;
    // ---- constant extra K block, extra Q block, Q rows
    {
      // K extra: every row (1, 1, 1, 0, ...); Q extra: (-hi, -mid, -lo, 0, ...) of lse / scale
      const uint32_t one = kFp16 ? 0x3C00u : 0x3F80u;
      uint8_t* kx = smem + L::kKx;
      uint8_t* qx = smem + L::kQx;
      const int r = ptid;
      uint4 kv0 = make_uint4(one | (one << 16), one, 0, 0);
      float x = 3.0e38f;                                 // padding rows: exp(-huge) = 0
      if (kFp16) x = 60000.f;
      if (r < rows_valid) x = p.lse[(size_t)bh * p.Lq + row_base + r] * p.inv_scale;
      uint32_t w0, w1;
      if (kFp16) {
        const __half hi = __float2half_rn(x);
        const float r1 = x - __half2float(hi);
        const __half mid = __float2half_rn(r1);
        const __half lo = __float2half_rn(r1 - __half2float(mid));
        w0 = (uint32_t)__half_as_ushort(__hneg(hi)) | ((uint32_t)__half_as_ushort(__hneg(mid)) << 16);
        w1 = (uint32_t)__half_as_ushort(__hneg(lo));
      } else {
        const __nv_bfloat16 hi = __float2bfloat16_rn(x);
        const float r1 = x - __bfloat162float(hi);
        const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
        const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
        w0 = (uint32_t)__bfloat16_as_ushort(__hneg(hi)) | ((uint32_t)__bfloat16_as_ushort(__hneg(mid)) << 16);
        w1 = (uint32_t)__bfloat16_as_ushort(__hneg(lo));
      }
      // chunks 0 and 1 of the row carry the 16 columns of the k-step; the rest of the 128-byte row is unused
      *reinterpret_cast<uint4*>(kx + swz(r, 0)) = kv0;
      *reinterpret_cast<uint4*>(kx + swz(r, 1)) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(qx + swz(r, 0)) = make_uint4(w0, w1, 0, 0);
      *reinterpret_cast<uint4*>(qx + swz(r, 1)) = make_uint4(0, 0, 0, 0);
      fence_proxy_async_smem();
      mbar_arrive(bar(BAR_Q_FULL));                      // release: the plain stores above
      // Q rows (through the permutation if given)
      int src = -1;
      if (r < rows_valid) {
        src = row_base + r;
        if (p.perm != nullptr) src = static_cast<int>(p.perm[(size_t)bh * p.Lq + src]);
      }
      const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q) + 2 * ((size_t)b * p.q_stride[0] + (size_t)h * p.q_stride[2]) + cch * 16;
      const size_t q_row = 2 * (size_t)p.q_stride[1];
#pragma unroll
      for (int i = 0; i < 32 / kRowsPerInstr; ++i) {
        const int rl = i * kRowsPerInstr + sub;
        const int id = __shfl_sync(0xffffffffu, src, rl);
        const uint32_t dst = s_base + L::kQ + swz(row0 + rl, cch);
        if (c_in_tile) {
          if (id >= 0 && c_live) cp_async16(dst, qb + (size_t)id * q_row);
          else cp_async16_zfill(dst, p.q, 0);
        }
      }
      cp_async_arrive_noinc(bar(BAR_Q_FULL));
    }
    // ---- key tiles: contiguous rows t*128 .. t*128+127 of this head
    int n_tiles_cp = n_tiles;       // tiles copied with cp.async (none when TMA is used)
    const uint8_t* kb = reinterpret_cast<const uint8_t*>(p.k) + 2 * ((size_t)b * p.k_stride[0] + (size_t)h * p.k_stride[2]) + cch * 16;
    const size_t k_row = 2 * (size_t)p.k_stride[1];
    int slot = 0, phase = 0;
    bool wrapped = false, ok = true;
    const bool tma_leader = elect_one();
    if (use_tma) {
      // one thread of producer warp 0 issues every tile as D / 64 boxes of 128 rows x 128 bytes; rows beyond the
      // end of the sequence arrive as zeros
      if (pw == 0) {
        int co[4] = {0, 0, 0, 0};
        co[kmap.pos_h] = h;
        co[kmap.pos_b] = b;
#pragma unroll 1
        for (int t = 0; t < n_tiles && ok; ++t) {
          if (wrapped) ok = mbar_wait(bar(BAR_EMPTY + slot), phase ^ 1, p.status, 44);
          if (!ok) break;
          if (tma_leader) {
            mbar_arrive_expect_tx(bar(BAR_FULL + slot), L::kTileBytes);
            co[kmap.pos_row] = t * kTile;
#pragma unroll
            for (int cb = 0; cb < L::kBlocks; ++cb)
              tma_load_4d(sRing(slot) + cb * 16384, kmap.k, cb * 64, co[1], co[2], co[3], bar(BAR_FULL + slot));
          }
          if (++slot == R) { slot = 0; phase ^= 1; wrapped = true; }
        }
      }
      n_tiles_cp = 0;
    }
#pragma unroll 1
    for (int t = 0; t < n_tiles_cp && ok; ++t) {
      if (wrapped) ok = mbar_wait(bar(BAR_EMPTY + slot), phase ^ 1, p.status, 44);
      if (!ok) break;
      const uint32_t dst0 = sRing(slot);
#pragma unroll
      for (int i = 0; i < 32 / kRowsPerInstr; ++i) {
        const int rl = row0 + i * kRowsPerInstr + sub;
        const int krow = t * kTile + rl;
        const uint32_t dst = dst0 + swz(rl, cch);
        if (c_in_tile) {
          if (krow < p.Lk && c_live) cp_async16(dst, kb + (size_t)krow * k_row);
          else cp_async16_zfill(dst, p.k, 0);
        }
      }
      cp_async_arrive_noinc(bar(BAR_FULL + slot));
      if (++slot == R) { slot = 0; phase ^= 1; wrapped = true; }
    }
    cp_async_wait_all();
  }

  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, bool kFp16, int kPoly = 2>
int launch(const GroupMassParams& p, cudaStream_t stream) {
  using L = Smem<D>;
  auto kern = group_mass_kernel<D, kFp16, kPoly>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) != cudaSuccess) return -8;
  const long long grid = (long long)p.B * p.H * p.M;
  KeyTileMap kmap{};
  // (the map carries the true head dimension: boxes that reach beyond it are zero-filled by the copy engine)
  kmap.valid = encode_tile_map(p.k, p.k_stride, p.B, p.Lk, p.H, p.D, kmap.k, kmap.pos_h, kmap.pos_row, kmap.pos_b);
  kern<<<(unsigned)grid, kThreads, L::kDynamic, stream>>>(p, kmap);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace

int launch_group_mass(const GroupMassParams& p, bool fp16, cudaStream_t stream) {
  if (p.D == 128) return fp16 ? launch<128, true>(p, stream) : launch<128, false>(p, stream);
  if (p.D == 64) return fp16 ? launch<64, true>(p, stream) : launch<64, false>(p, stream);
  // every other multiple of 8 up to 256 (the reference's head-dimension table has 96, 144, 160, 192, 256): padded layouts
  if (p.D < 8 || p.D > 256 || p.D % 8 != 0) return -3;
  if (p.D <= 192) return fp16 ? launch<192, true>(p, stream) : launch<192, false>(p, stream);
  return fp16 ? launch<256, true>(p, stream) : launch<256, false>(p, stream);
}

}  // namespace mcs
