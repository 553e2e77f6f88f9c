// Fast PDDP query grouping (recursive principal-direction bisection) for sm_100a.
//
// Restates mcsparse/kernels/flash_mcsa/pca_group.py:141-243.  Tokens of each (batch, head) are
// reordered so that every aligned block of C tokens holds similar vectors: at each level every
// node (a contiguous interval of the current order) computes the principal direction of its
// centred rows with a few power iterations on the Gram matrix X^T X - s s^T / n, sorts its rows
// by their projection on that direction and is split at the block-aligned midpoint.
//
// Per level, with no host synchronisation anywhere (the tree shape depends only on N and C):
//   gram     tcgen05: G += X_tile^T X_tile over 128-row tiles gathered through the current
//            permutation.  The SAME shared-memory tile serves as both MMA operands (MN-major A and
//            MN-major B); a second, 16-column MMA against a tile of ones yields the column sums s.
//            Big nodes are split into chunks of 2048 rows whose partial results are summed in a
//            fixed order by the next kernel (deterministic, no atomics).
//   power    one CTA per node: reduce partials, centre, normalise the start vector, iterate.
//   project  a = x . v in fp32 per row (one warp per row), emitted as 64-bit sort keys
//            (order-preserving float bits << 32 | position inside the node): unique keys, so the
//            sort is stable by construction; the fp32 projections can be dumped for checking.
//   sort     bitonic network over power-of-two padded segments: shared-memory stages, plus
//            global compare-exchange steps when a segment exceeds one CTA's tile.
//   scatter  new order written back through the sorted positions.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <vector>

#include "kernels.cuh"
#include "ptx.cuh"

namespace mcs {

namespace {

constexpr int kChunkRows = 2048;        // rows per gram work item
constexpr int kSortTile = 4096;         // keys per CTA in the shared-memory sort stages
constexpr int kMaxNodes = 4096;

// ------------------------------------------------------------------------------------------
// Tree shape (pure function of N, C): used identically on host (launch sizes) and device (tables).
// ------------------------------------------------------------------------------------------
struct LevelShape {
  int nodes;        // nodes at this level
  int items;        // gram work items (sum over nodes of ceil(size / kChunkRows))
  int pad;          // power of two >= largest node size
};

__host__ __device__ inline int next_pow2(int v) { int p = 1; while (p < v) p <<= 1; return p; }

// Fills block-interval arrays for successive levels.  lo/hi hold the current level (in blocks).
// Returns false when no interval has more than one block (no further level).
__host__ __device__ inline bool any_splittable(const int* lo, const int* hi, int n) {
  for (int i = 0; i < n; ++i) if (hi[i] - lo[i] > 1) return true;
  return false;
}
__host__ __device__ inline int split_level(const int* lo, const int* hi, int n, int* lo2, int* hi2) {
  int m = 0;
  for (int i = 0; i < n; ++i) {
    if (hi[i] - lo[i] <= 1) { lo2[m] = lo[i]; hi2[m] = hi[i]; ++m; }
    else {
      const int mid = lo[i] + (hi[i] - lo[i]) / 2;
      lo2[m] = lo[i]; hi2[m] = mid; ++m;
      lo2[m] = mid; hi2[m] = hi[i]; ++m;
    }
  }
  return m;
}

// Device tables of one level, laid out consecutively in the workspace.
struct LevelTables {
  int* node_start;   // [nodes] token start
  int* node_size;    // [nodes]
  int* node_item0;   // [nodes] first gram item of the node
  int* item_node;    // [items]
  int* item_row0;    // [items] first row (relative to node start)
};

__global__ void pddp_tables_kernel(int N, int C, int* tab, int max_levels, int stride) {
  // single thread: fills, for every level, node_start/node_size/node_item0/item_node/item_row0
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int K = (N + C - 1) / C;
  // two scratch interval lists live at the end of the table area
  int* lo = tab + (size_t)max_levels * stride;
  int* hi = lo + kMaxNodes;
  int* lo2 = hi + kMaxNodes;
  int* hi2 = lo2 + kMaxNodes;
  int n = 1; lo[0] = 0; hi[0] = K;
  for (int lv = 0; lv < max_levels && any_splittable(lo, hi, n); ++lv) {
    int* t = tab + (size_t)lv * stride;
    int* node_start = t, *node_size = t + kMaxNodes, *node_item0 = t + 2 * kMaxNodes;
    int* item_node = t + 3 * kMaxNodes, *item_row0 = item_node + (stride - 3 * kMaxNodes) / 2;
    int items = 0;
    for (int i = 0; i < n; ++i) {
      const int s = lo[i] * C, e = min(hi[i] * C, N);
      node_start[i] = s; node_size[i] = e - s; node_item0[i] = items;
      for (int r = 0; r < e - s; r += kChunkRows) { item_node[items] = i; item_row0[items] = r; ++items; }
    }
    const int m = split_level(lo, hi, n, lo2, hi2);
    for (int i = 0; i < m; ++i) { lo[i] = lo2[i]; hi[i] = hi2[i]; }
    n = m;
  }
}

__device__ __forceinline__ LevelTables level_tables(int* tab, int lv, int stride) {
  int* t = tab + (size_t)lv * stride;
  LevelTables T;
  T.node_start = t; T.node_size = t + kMaxNodes; T.node_item0 = t + 2 * kMaxNodes;
  T.item_node = t + 3 * kMaxNodes; T.item_row0 = T.item_node + (stride - 3 * kMaxNodes) / 2;
  return T;
}

__device__ __forceinline__ uint32_t swz(int row, int c) {
  return static_cast<uint32_t>((c >> 3) * 16384 + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}

// ------------------------------------------------------------------------------------------
// gram: partial[bh][item] = (G 128x128, s 128) over the item's rows
// ------------------------------------------------------------------------------------------
constexpr int kGramThreads = 160;       // 4 load/epilogue warps + 1 MMA warp
constexpr int kGramSmem = 2 * 32768 + 16384 + 256 + 1024;
constexpr int kPartialFloats = 128 * 128 + 128;

template <bool kFp16>
__global__ void __launch_bounds__(kGramThreads, 1) pddp_gram_kernel(PddpParams p, int lv, const int* perm_in) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t sOnes = s_base + 65536;
  const uint32_t bars = s_base + 65536 + 16384;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 65536 + 16384 + 128);
  auto bar = [&](int i) { return bars + 8u * i; };   // 0,1 full; 2,3 empty; 4 done
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const LevelTables T = level_tables(p.tables, lv, p.table_stride);
  const int item = blockIdx.x, bh = blockIdx.y;
  const int node = T.item_node[item];
  const int row_begin = T.item_row0[item];
  const int rows = min(kChunkRows, T.node_size[node] - row_begin);
  const int pos0 = T.node_start[node] + row_begin;
  const int n_tiles = (rows + 127) / 128;
  const int D = p.D;

  if (tid == 0) {
    mbar_init(bar(0), 128); mbar_init(bar(1), 128); mbar_init(bar(2), 1); mbar_init(bar(3), 1); mbar_init(bar(4), 1);
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(smem_u32(tmem_slot), 256); tmem_relinquish(); }
  // ones tile: rows 0..15 (N = 16), 16 K-columns of 1.0 (K-major, 128-byte swizzled rows)
  if (tid < 16) {
    const uint32_t one2 = kFp16 ? 0x3C003C00u : 0x3F803F80u;
    *reinterpret_cast<uint4*>(smem + 65536 + swz(tid, 0)) = make_uint4(one2, one2, one2, one2);
    *reinterpret_cast<uint4*>(smem + 65536 + swz(tid, 1)) = make_uint4(one2, one2, one2, one2);
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) {
    // ---- gather rows of each tile through the permutation
    const int chunks = D / 8;                    // 16-byte chunks per row (8 or 16)
    const uint8_t* xb = reinterpret_cast<const uint8_t*>(p.x) + 2 * (size_t)bh * p.x_stride_bh;
    const size_t row_bytes = 2 * (size_t)p.x_stride_row;
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int buf = t & 1;
      if (t >= 2) ok = mbar_wait(bar(2 + buf), ((t >> 1) - 1) & 1, p.status, 60);
      if (!ok) break;
      const int r = t * 128 + tid;               // row of the item handled by this thread
      const uint8_t* src = nullptr;
      if (r < rows) src = xb + (size_t)perm_in[(size_t)bh * p.N + pos0 + r] * row_bytes;
      const uint32_t dst = s_base + buf * 32768;
#pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        if (src != nullptr && c < chunks) cp_async16(dst + swz(tid, c), src + c * 16);
        else cp_async16_zfill(dst + swz(tid, c), xb, 0);
      }
      cp_async_arrive_noinc(bar(buf));
    }
    cp_async_wait_all();
    // ---- epilogue: thread d owns feature row d of G (TMEM lane d)
    if (ok) ok = mbar_wait(bar(4), 0, p.status, 61);
    if (ok) {
      tc_fence_after();
      float* out = p.partial + ((size_t)bh * p.max_items + item) * kPartialFloats;
      const uint32_t lane_addr = (static_cast<uint32_t>(warp) * 32u) << 16;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_addr + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) out[(size_t)tid * 128 + c * 32 + i] = __uint_as_float(r[i]);
      }
      uint32_t r8[8];
      tmem_ld8(tmem + lane_addr + 128, r8);
      tmem_wait_ld();
      out[128 * 128 + tid] = __uint_as_float(r8[0]);
    }
    tc_fence_before();
  } else {
    if (lane == 0) {
      constexpr uint32_t kFmt = kFp16 ? 0u : 1u;
      constexpr uint32_t idesc_g = mma_idesc(kFmt, kFmt, 1, 1, 128, 128);   // A and B both MN-major
      constexpr uint32_t idesc_s = mma_idesc(kFmt, kFmt, 1, 0, 128, 16);    // B = ones, K-major
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      auto desc = [&](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
      const uint32_t ones_lo = ((sOnes & 0x3FFFFu) >> 4) | (1u << 16);
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int buf = t & 1;
        ok = mbar_wait(bar(buf), (t >> 1) & 1, p.status, 62);
        if (!ok) break;
        fence_proxy_async_smem();
        tc_fence_after();
        const uint32_t xlo = (((s_base + buf * 32768) & 0x3FFFFu) >> 4) | ((16384u >> 4) << 16);
#pragma unroll
        for (int j = 0; j < 8; ++j) {             // 16 rows per k-step
          const uint64_t dx = desc(xlo + j * (2048 >> 4));
          mma_f16_ss(tmem, dx, dx, idesc_g, (t > 0) || (j > 0));
          mma_f16_ss(tmem + 128, dx, desc(ones_lo), idesc_s, (t > 0) || (j > 0));
        }
        tc_commit(bar(2 + buf));
      }
      if (ok) tc_commit(bar(4));
      else { tc_commit(bar(4)); mbar_wait_quiet(bar(4), 0, 1 << 20); }
    }
    __syncwarp();
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

// ------------------------------------------------------------------------------------------
// power: v[bh][node] = principal direction of the node (pow_iters normalised mat-vecs)
// ------------------------------------------------------------------------------------------

// 512 threads: thread (d, q) = (tid & 127, tid >> 7) owns element d and the Gram rows e = q (mod 4).  The
// arithmetic is exactly that of a 128-thread version with four accumulators per element (a_q summed over
// e = q, q+4, ... in increasing order, combined as (a0 + a1) + (a2 + a3)), so results do not depend on the
// thread count; four times the threads only shorten the dependent load and FMA chains, which is what the
// deep levels with thousands of small nodes are bound by.
__global__ void __launch_bounds__(512, 1) pddp_power_kernel(PddpParams p, int lv, int nodes, const float* v0) {
  extern __shared__ __align__(16) float sm[];
  float* G = sm;                 // 128 x 128, symmetric
  float* vec = sm + 128 * 128;   // 128
  float* partial = vec + 128;    // 4 x 128
  float* red = partial + 512;    // 4
  const LevelTables T = level_tables(p.tables, lv, p.table_stride);
  const int node = blockIdx.x, bh = blockIdx.y, d = threadIdx.x & 127, q = threadIdx.x >> 7;
  const int size = T.node_size[node];
  const int item0 = T.node_item0[node];
  const int n_items = (size + kChunkRows - 1) / kChunkRows;
  const float* part = p.partial + ((size_t)bh * p.max_items + item0) * kPartialFloats;
  // fixed-order reduction of the partial Gram matrices
  float s_d = 0.f;
  for (int it = 0; it < n_items; ++it) s_d += part[(size_t)it * kPartialFloats + 128 * 128 + d];
  if (q == 0) vec[d] = s_d;
  __syncthreads();
  const float inv_n = 1.f / (float)size;
  for (int e = q; e < 128; e += 4) {
    float g = 0.f;
    for (int it = 0; it < n_items; ++it) g += part[(size_t)it * kPartialFloats + (size_t)e * 128 + d];   // G[e][d], coalesced
    G[e * 128 + d] = g - vec[e] * s_d * inv_n;
  }
  __syncthreads();
  // sum over the 128 elements, identical in all four thread groups: warp sums, then (r0 + r1) + (r2 + r3)
  auto sum_128 = [&](float x) {
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    __syncthreads();
    if (q == 0 && (threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
    __syncthreads();
    return (red[0] + red[1]) + (red[2] + red[3]);
  };
  const bool live = d < p.D;
  float v = live ? v0[((size_t)bh * nodes + node) * p.D + d] : 0.f;
  float nrm = sqrtf(sum_128(v * v));
  v /= fmaxf(nrm, 1e-12f);
  for (int iter = 0; iter < p.pow_iters; ++iter) {
    __syncthreads();
    if (q == 0) vec[d] = v;
    __syncthreads();
    float a = 0.f;
#pragma unroll 8
    for (int e = q; e < 128; e += 4) a += G[e * 128 + d] * vec[e];     // G symmetric: G[e][d], conflict-free
    partial[q * 128 + d] = a;
    __syncthreads();
    v = (partial[d] + partial[128 + d]) + (partial[256 + d] + partial[384 + d]);
    nrm = sqrtf(sum_128(v * v));
    v /= fmaxf(nrm, 1e-12f);
  }
  if (q == 0) p.dir[((size_t)bh * p.dir_nodes + node) * 128 + d] = v;
}

// ------------------------------------------------------------------------------------------
// project: fp32 projection of every row on its node's direction -> 64-bit sort keys
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_key(float f) {
  uint32_t u = __float_as_uint(f);
  if (f == 0.f) u = 0u;                                        // -0 == +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kProjRows = 8;     // rows per warp: eight independent row loads in flight per lane

template <bool kFp16>
__global__ void __launch_bounds__(256) pddp_project_kernel(PddpParams p, int lv, int nodes, int pad, const int* perm_in,
                                                           float* proj_out) {
  const LevelTables T = level_tables(p.tables, lv, p.table_stride);
  const int bh = blockIdx.y;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  // one warp per kProjRows consecutive slots of the padded key array (slot = node * pad + r); pad is a
  // multiple of kProjRows, so the slots of a warp belong to one node
  const long long total = (long long)nodes * pad;
  const long long slot0 = warp * kProjRows;
  if (slot0 >= total) return;
  const int node = (int)(slot0 / pad), r0 = (int)(slot0 % pad);
  unsigned long long* keys = p.keys + (size_t)bh * p.key_stride;
  const int nsize = T.node_size[node];
  const int pos0 = T.node_start[node] + r0;
  const bool lane_live = lane * 4 < p.D;
  float4 vv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (lane_live) vv = *reinterpret_cast<const float4*>(p.dir + ((size_t)bh * p.dir_nodes + node) * 128 + lane * 4);
  // row ids of this warp's slots (lane i holds slot i), then all row loads before any arithmetic
  int my_id = -1;
  if (lane < kProjRows && r0 + lane < nsize) my_id = perm_in[(size_t)bh * p.N + pos0 + lane];
  uint2 w[kProjRows];
#pragma unroll
  for (int i = 0; i < kProjRows; ++i) {
    const int id = __shfl_sync(0xffffffffu, my_id, i);
    w[i] = make_uint2(0u, 0u);
    if (id >= 0 && lane_live)
      w[i] = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.x) +
                                            2 * ((size_t)bh * p.x_stride_bh + (size_t)id * p.x_stride_row) + lane * 8);
  }
#pragma unroll
  for (int i = 0; i < kProjRows; ++i) {
    float acc = 0.f;
    if (lane_live) {
      float2 a, b;
      if (kFp16) {
        a = __half22float2(*reinterpret_cast<const __half2*>(&w[i].x));
        b = __half22float2(*reinterpret_cast<const __half2*>(&w[i].y));
      } else {
        a = make_float2(bf16_lo(w[i].x), bf16_hi(w[i].x));
        b = make_float2(bf16_lo(w[i].y), bf16_hi(w[i].y));
      }
      acc = fmaf(a.x, vv.x, fmaf(a.y, vv.y, fmaf(b.x, vv.z, b.y * vv.w)));
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      const int r = r0 + i;
      if (r >= nsize) {
        keys[slot0 + i] = 0xFFFFFFFFFFFFFFFFull;               // padding sorts last
      } else {
        keys[slot0 + i] = ((unsigned long long)float_key(acc) << 32) | (unsigned)r;
        if (proj_out != nullptr) proj_out[(size_t)bh * p.N + pos0 + i] = acc;
      }
    }
  }
}


// ------------------------------------------------------------------------------------------
// Head dimensions other than 64 and 128 (multiples of 8 up to 256): the principal direction by power iterations
// that never form the Gram matrix.  With t_r = x_r . v,
//     (X^T X - s s^T / n) v  =  sum_r x_r t_r  -  s (sum_r t_r) / n,
// so one pass over the node's rows per iteration gives the next vector.  The rows are read pow_iters times per level
// instead of once, which is the price of staying clear of a 256 x 256 Gram matrix per node; this path serves the
// uncommon head dimensions, the tensor-core Gram path above the common ones.  Partial sums of a node's chunks are
// combined in chunk order by the next kernel: deterministic, no atomics.
// ------------------------------------------------------------------------------------------
constexpr int kWideD = 256;
constexpr int kWideFloats = 2 * kWideD + 8;      // per chunk: sum_r x_r t_r [256], sum_r x_r [256], sum_r t_r

__device__ __forceinline__ float block_sum_256(float x, float* red) {
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += red[w];
  return t;
}

// v = v0 / |v0| for every node of the level (zeros beyond D)
__global__ void __launch_bounds__(256) pddp_wide_init_kernel(PddpParams p, int nodes, const float* v0, float* wdir) {
  __shared__ float red[8];
  const int node = blockIdx.x, bh = blockIdx.y, d = threadIdx.x;
  float v = d < p.D ? v0[((size_t)bh * nodes + node) * p.D + d] : 0.f;
  const float nrm = sqrtf(block_sum_256(v * v, red));
  wdir[((size_t)bh * p.dir_nodes + node) * kWideD + d] = v / fmaxf(nrm, 1e-12f);
}

template <bool kFp16>
__device__ __forceinline__ void unpack8(const uint4& w, float (&x)[8]) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kFp16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    } else {
      x[2 * i] = bf16_lo(u[i]); x[2 * i + 1] = bf16_hi(u[i]);
    }
  }
}

// One CTA per chunk of up to kChunkRows rows of one node: lane l of every warp owns elements 8l .. 8l+7 of a row.
template <bool kFp16>
__global__ void __launch_bounds__(256) pddp_wide_matvec_kernel(PddpParams p, int lv, const int* perm_in, const float* wdir,
                                                               float* wpart) {
  __shared__ float acc_w[8][kWideD];
  __shared__ float acc_s[8][kWideD];
  __shared__ float acc_t[8];
  const LevelTables T = level_tables(p.tables, lv, p.table_stride);
  const int item = blockIdx.x, bh = blockIdx.y;
  const int node = T.item_node[item], row0 = T.item_row0[item];
  const int rows = min(kChunkRows, T.node_size[node] - row0);
  const int start = T.node_start[node] + row0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool live = lane * 8 < p.D;
  float v[8], w[8], sx[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[j] = live ? wdir[((size_t)bh * p.dir_nodes + node) * kWideD + lane * 8 + j] : 0.f;
    w[j] = 0.f; sx[j] = 0.f;
  }
  float st = 0.f;
  const uint8_t* xb = reinterpret_cast<const uint8_t*>(p.x) + 2 * (size_t)bh * p.x_stride_bh + lane * 16;
  constexpr int kIn = 4;                                         // rows in flight per warp
#pragma unroll 1
  for (int r = warp * kIn; r < rows; r += 8 * kIn) {
    uint4 raw[kIn];
#pragma unroll
    for (int i = 0; i < kIn; ++i) {
      raw[i] = make_uint4(0u, 0u, 0u, 0u);
      if (r + i < rows && live) {
        const int id = perm_in[(size_t)bh * p.N + start + r + i];
        raw[i] = *reinterpret_cast<const uint4*>(xb + 2 * (size_t)id * p.x_stride_row);
      }
    }
#pragma unroll
    for (int i = 0; i < kIn; ++i) {
      float x[8];
      unpack8<kFp16>(raw[i], x);
      float t = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) t = fmaf(x[j], v[j], t);
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
#pragma unroll
      for (int j = 0; j < 8; ++j) { w[j] = fmaf(x[j], t, w[j]); sx[j] += x[j]; }
      st += t;                                                   // (rows beyond the chunk are zero rows: t = 0)
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { acc_w[warp][lane * 8 + j] = w[j]; acc_s[warp][lane * 8 + j] = sx[j]; }
  if (lane == 0) acc_t[warp] = st;
  __syncthreads();
  float* out = wpart + ((size_t)bh * p.max_items + item) * kWideFloats;
  const int d = threadIdx.x;
  float a = 0.f, b = 0.f;
#pragma unroll
  for (int q = 0; q < 8; ++q) { a += acc_w[q][d]; b += acc_s[q][d]; }          // warps in fixed order
  out[d] = a;
  out[kWideD + d] = b;
  if (d == 0) {
    float t = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) t += acc_t[q];
    out[2 * kWideD] = t;
  }
}

// next vector of every node: chunks combined in order, centred, normalised
__global__ void __launch_bounds__(256) pddp_wide_step_kernel(PddpParams p, int lv, float* wdir, const float* wpart) {
  __shared__ float red[8];
  const LevelTables T = level_tables(p.tables, lv, p.table_stride);
  const int node = blockIdx.x, bh = blockIdx.y, d = threadIdx.x;
  const int size = T.node_size[node];
  const int item0 = T.node_item0[node];
  const int n_items = (size + kChunkRows - 1) / kChunkRows;
  const float* part = wpart + ((size_t)bh * p.max_items + item0) * kWideFloats;
  float wr = 0.f, s = 0.f, t = 0.f;
  for (int it = 0; it < n_items; ++it) {
    wr += part[(size_t)it * kWideFloats + d];
    s += part[(size_t)it * kWideFloats + kWideD + d];
    t += part[(size_t)it * kWideFloats + 2 * kWideD];
  }
  float v = wr - s * (t / (float)size);
  const float nrm = sqrtf(block_sum_256(v * v, red));
  wdir[((size_t)bh * p.dir_nodes + node) * kWideD + d] = v / fmaxf(nrm, 1e-12f);
}

// projection of every row on its node's direction, eight elements per lane (the counterpart of pddp_project_kernel)
template <bool kFp16>
__global__ void __launch_bounds__(256) pddp_wide_project_kernel(PddpParams p, int lv, int nodes, int pad, const int* perm_in,
                                                                const float* wdir, float* proj_out) {
  const LevelTables T = level_tables(p.tables, lv, p.table_stride);
  const int bh = blockIdx.y;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)nodes * pad;
  const long long slot0 = warp * kProjRows;
  if (slot0 >= total) return;
  const int node = (int)(slot0 / pad), r0 = (int)(slot0 % pad);
  unsigned long long* keys = p.keys + (size_t)bh * p.key_stride;
  const int nsize = T.node_size[node];
  const int pos0 = T.node_start[node] + r0;
  const bool live = lane * 8 < p.D;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = live ? wdir[((size_t)bh * p.dir_nodes + node) * kWideD + lane * 8 + j] : 0.f;
  int my_id = -1;
  if (lane < kProjRows && r0 + lane < nsize) my_id = perm_in[(size_t)bh * p.N + pos0 + lane];
  uint4 raw[kProjRows];
#pragma unroll
  for (int i = 0; i < kProjRows; ++i) {
    const int id = __shfl_sync(0xffffffffu, my_id, i);
    raw[i] = make_uint4(0u, 0u, 0u, 0u);
    if (id >= 0 && live)
      raw[i] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.x) +
                                              2 * ((size_t)bh * p.x_stride_bh + (size_t)id * p.x_stride_row) + lane * 16);
  }
#pragma unroll
  for (int i = 0; i < kProjRows; ++i) {
    float x[8];
    unpack8<kFp16>(raw[i], x);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc = fmaf(x[j], v[j], acc);
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      const int r = r0 + i;
      if (r >= nsize) {
        keys[slot0 + i] = 0xFFFFFFFFFFFFFFFFull;
      } else {
        keys[slot0 + i] = ((unsigned long long)float_key(acc) << 32) | (unsigned)r;
        if (proj_out != nullptr) proj_out[(size_t)bh * p.N + pos0 + i] = acc;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// sort: bitonic network over segments of `pad` keys (power of two), ascending inside each segment
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void cmpx(unsigned long long& a, unsigned long long& b, bool asc) {
  if ((a > b) == asc) { const unsigned long long t = a; a = b; b = t; }
}

// All stages with compare distance < tile, for k from k_lo to k_hi (k_hi <= pad), on tiles of
// min(pad, kSortTile) keys held in shared memory.  For k > tile only the tail (j < tile) is done.
__global__ void __launch_bounds__(1024) pddp_sort_smem_kernel(unsigned long long* keys_all, size_t key_stride, int pad, int tile,
                                                              int k_lo, int k_hi) {
  extern __shared__ __align__(16) unsigned long long sk[];
  unsigned long long* keys = keys_all + (size_t)blockIdx.y * key_stride + (size_t)blockIdx.x * tile;
  const int base = blockIdx.x * tile;                        // index of this tile inside the bh's key array
  for (int i = threadIdx.x; i < tile; i += blockDim.x) sk[i] = keys[i];
  __syncthreads();
  for (int k = k_lo; k <= k_hi; k <<= 1) {
    for (int j = min(k >> 1, tile >> 1); j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < (tile >> 1); t += blockDim.x) {
        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));      // lower index of the pair
        const int gi = (base + i) & (pad - 1);                     // position inside the segment
        const bool asc = (k == pad) || ((gi & k) == 0);
        unsigned long long a = sk[i], b = sk[i + j];
        cmpx(a, b, asc);
        sk[i] = a; sk[i + j] = b;
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < tile; i += blockDim.x) keys[i] = sk[i];
}

// One compare-exchange step at distance j >= tile of stage k.
__global__ void __launch_bounds__(256) pddp_sort_global_kernel(unsigned long long* keys_all, size_t key_stride, long long half_total,
                                                               int pad, int k, int j) {
  unsigned long long* keys = keys_all + (size_t)blockIdx.y * key_stride;
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= half_total) return;
  const long long i = ((t & ~(long long)(j - 1)) << 1) | (t & (j - 1));
  const int gi = (int)(i & (pad - 1));
  const bool asc = (k == pad) || ((gi & k) == 0);
  unsigned long long a = keys[i], b = keys[i + j];
  if ((a > b) == asc) { keys[i] = b; keys[i + j] = a; }
}

// new_perm[start + r] = old_perm[start + sorted position r]
__global__ void __launch_bounds__(256) pddp_scatter_kernel(PddpParams p, int lv, int nodes, int pad, const int* perm_in, int* perm_out) {
  const LevelTables T = level_tables(p.tables, lv, p.table_stride);
  const int bh = blockIdx.y;
  const long long slot = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (slot >= (long long)nodes * pad) return;
  const int node = (int)(slot / pad), r = (int)(slot % pad);
  if (r >= T.node_size[node]) return;
  const unsigned long long key = p.keys[(size_t)bh * p.key_stride + slot];
  const int start = T.node_start[node];
  perm_out[(size_t)bh * p.N + start + r] = perm_in[(size_t)bh * p.N + start + (int)(key & 0xFFFFFFFFull)];
}

__global__ void pddp_iota_kernel(int* perm, long long total, int N) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) perm[i] = (int)(i % N);
}
__global__ void pddp_widen_kernel(const int* perm, long long* out, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = perm[i];
}

}  // namespace

// ------------------------------------------------------------------------------------------
// Host side: tree shape, workspace layout, per-level launches
// ------------------------------------------------------------------------------------------
namespace {

struct Plan {
  int levels = 0;
  int K = 0;
  std::vector<LevelShape> shape;
  int max_items = 0;
  size_t key_stride = 0;          // u64 keys per (batch*head)
  int table_stride = 0;
  // byte offsets inside the workspace
  size_t off_tables = 0, off_perm_a = 0, off_perm_b = 0, off_partial = 0, off_dir = 0, off_keys = 0, total = 0;
};

Plan make_plan(int BH, int N, int C) {
  Plan pl;
  pl.K = (N + C - 1) / C;
  std::vector<int> lo(1, 0), hi(1, pl.K), lo2, hi2;
  while (any_splittable(lo.data(), hi.data(), (int)lo.size())) {
    LevelShape ls{(int)lo.size(), 0, 1};
    int max_size = 1;
    for (size_t i = 0; i < lo.size(); ++i) {
      const int size = std::min(hi[i] * C, N) - lo[i] * C;
      ls.items += (size + kChunkRows - 1) / kChunkRows;
      max_size = std::max(max_size, size);
    }
    ls.pad = std::max(next_pow2(max_size), 8);   // the projection kernel works on whole groups of kProjRows = 8 slots
    pl.shape.push_back(ls);
    pl.max_items = std::max(pl.max_items, ls.items);
    pl.key_stride = std::max(pl.key_stride, (size_t)ls.nodes * ls.pad);
    lo2.assign(2 * lo.size(), 0); hi2.assign(2 * lo.size(), 0);
    const int m = split_level(lo.data(), hi.data(), (int)lo.size(), lo2.data(), hi2.data());
    lo.assign(lo2.begin(), lo2.begin() + m); hi.assign(hi2.begin(), hi2.begin() + m);
  }
  pl.levels = (int)pl.shape.size();
  pl.table_stride = 3 * kMaxNodes + 2 * (pl.max_items + 8);
  auto align = [](size_t v) { return (v + 255) & ~size_t(255); };
  size_t o = 0;
  pl.off_tables = o; o = align(o + ((size_t)std::max(pl.levels, 1) * pl.table_stride + 4 * kMaxNodes) * sizeof(int));
  pl.off_perm_a = o; o = align(o + (size_t)BH * N * sizeof(int));
  pl.off_perm_b = o; o = align(o + (size_t)BH * N * sizeof(int));
  pl.off_partial = o; o = align(o + (size_t)BH * std::max(pl.max_items, 1) * kPartialFloats * sizeof(float));
  pl.off_dir = o; o = align(o + (size_t)BH * pl.K * 128 * sizeof(float));
  pl.off_keys = o; o = align(o + (size_t)BH * std::max(pl.key_stride, (size_t)1) * sizeof(unsigned long long));
  pl.total = o;
  return pl;
}

}  // namespace

size_t pddp_workspace_bytes(int BH, int N, int C) {
  if (BH < 1 || N < 1 || C < 1 || (N + C - 1) / C > kMaxNodes) return 0;
  return make_plan(BH, N, C).total;
}

long long pddp_start_vector_rows(int BH, int N, int C) {
  const Plan pl = make_plan(BH, N, C);
  long long rows = 0;
  for (const auto& ls : pl.shape) rows += (long long)BH * ls.nodes;
  return rows;
}

int launch_pddp(const PddpArgs& a, cudaStream_t stream) {
  const int BH = a.BH, N = a.N, C = a.C;
  const long long total = (long long)BH * N;
  uint8_t* ws = reinterpret_cast<uint8_t*>(a.workspace);
  const Plan pl = make_plan(BH, N, C);
  if (pl.total > a.workspace_bytes) return -7;
  int* perm_a = reinterpret_cast<int*>(ws + pl.off_perm_a);
  int* perm_b = reinterpret_cast<int*>(ws + pl.off_perm_b);
  const int tb = 256;
  pddp_iota_kernel<<<(unsigned)((total + tb - 1) / tb), tb, 0, stream>>>(perm_a, total, N);
  if (pl.levels > 0) {
    PddpParams p{};
    p.x = a.x; p.x_stride_bh = a.x_stride_bh; p.x_stride_row = a.x_stride_row;
    p.N = N; p.D = a.D; p.BH = BH; p.pow_iters = a.pow_iters;
    p.tables = reinterpret_cast<int*>(ws + pl.off_tables); p.table_stride = pl.table_stride;
    p.max_items = std::max(pl.max_items, 1);
    p.partial = reinterpret_cast<float*>(ws + pl.off_partial);
    p.dir = reinterpret_cast<float*>(ws + pl.off_dir); p.dir_nodes = pl.K;
    p.keys = reinterpret_cast<unsigned long long*>(ws + pl.off_keys); p.key_stride = pl.key_stride;
    p.status = a.status;
    pddp_tables_kernel<<<1, 1, 0, stream>>>(N, C, p.tables, pl.levels, pl.table_stride);
    auto gram = a.fp16 ? pddp_gram_kernel<true> : pddp_gram_kernel<false>;
    if (cudaFuncSetAttribute(gram, cudaFuncAttributeMaxDynamicSharedMemorySize, kGramSmem) != cudaSuccess) return -8;
    const int power_smem = (128 * 128 + 128 + 512 + 8) * sizeof(float);
    if (cudaFuncSetAttribute(pddp_power_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, power_smem) != cudaSuccess) return -8;
    const float* v0 = a.start_vectors;
    const bool wide = a.D != 64 && a.D != 128;
    // wide path: per-chunk partial sums first, then the directions (256 floats per node), both inside the partial area
    float* wpart = p.partial;
    float* wdir = p.partial + (size_t)BH * p.max_items * kWideFloats;
    if (wide && ((size_t)BH * p.max_items * kWideFloats + (size_t)BH * pl.K * kWideD) >
                    (size_t)BH * p.max_items * kPartialFloats)
      return -7;
    for (int lv = 0; lv < pl.levels; ++lv) {
      const LevelShape& ls = pl.shape[lv];
      if (a.perm_levels != nullptr)
        cudaMemcpyAsync(a.perm_levels + (size_t)lv * total, perm_a, total * sizeof(int), cudaMemcpyDeviceToDevice, stream);
      const long long slots = (long long)ls.nodes * ls.pad;
      float* proj = a.proj_levels != nullptr ? a.proj_levels + (size_t)lv * total : nullptr;
      const unsigned pgrid = (unsigned)((slots / kProjRows * 32 + 255) / 256);
      if (wide) {
        // Gram-free power iterations (head dimensions other than 64 / 128); partial sums and directions live in the
        // area the Gram partials would use
        pddp_wide_init_kernel<<<dim3(ls.nodes, BH), 256, 0, stream>>>(p, ls.nodes, v0, wdir);
        for (int it = 0; it < a.pow_iters; ++it) {
          if (a.fp16) pddp_wide_matvec_kernel<true><<<dim3(ls.items, BH), 256, 0, stream>>>(p, lv, perm_a, wdir, wpart);
          else pddp_wide_matvec_kernel<false><<<dim3(ls.items, BH), 256, 0, stream>>>(p, lv, perm_a, wdir, wpart);
          pddp_wide_step_kernel<<<dim3(ls.nodes, BH), 256, 0, stream>>>(p, lv, wdir, wpart);
        }
        if (a.fp16) pddp_wide_project_kernel<true><<<dim3(pgrid, BH), 256, 0, stream>>>(p, lv, ls.nodes, ls.pad, perm_a, wdir, proj);
        else pddp_wide_project_kernel<false><<<dim3(pgrid, BH), 256, 0, stream>>>(p, lv, ls.nodes, ls.pad, perm_a, wdir, proj);
      } else {
        gram<<<dim3(ls.items, BH), kGramThreads, kGramSmem, stream>>>(p, lv, perm_a);
        pddp_power_kernel<<<dim3(ls.nodes, BH), 512, power_smem, stream>>>(p, lv, ls.nodes, v0);
        if (a.fp16) pddp_project_kernel<true><<<dim3(pgrid, BH), 256, 0, stream>>>(p, lv, ls.nodes, ls.pad, perm_a, proj);
        else pddp_project_kernel<false><<<dim3(pgrid, BH), 256, 0, stream>>>(p, lv, ls.nodes, ls.pad, perm_a, proj);
      }
      v0 += (size_t)BH * ls.nodes * a.D;
      // bitonic sort of every segment of `pad` keys
      const int tile = std::min(ls.pad, kSortTile);
      const unsigned tiles = (unsigned)(slots / tile);
      const int sthreads = std::max(32, std::min(1024, tile / 2));
      pddp_sort_smem_kernel<<<dim3(tiles, BH), sthreads, (size_t)tile * 8, stream>>>(p.keys, p.key_stride, ls.pad, tile, 2, tile);
      for (int k = tile * 2; k <= ls.pad; k <<= 1) {
        for (int j = k >> 1; j >= tile; j >>= 1)
          pddp_sort_global_kernel<<<dim3((unsigned)((slots / 2 + 255) / 256), BH), 256, 0, stream>>>(p.keys, p.key_stride, slots / 2, ls.pad, k, j);
        pddp_sort_smem_kernel<<<dim3(tiles, BH), sthreads, (size_t)tile * 8, stream>>>(p.keys, p.key_stride, ls.pad, tile, k, k);
      }
      pddp_scatter_kernel<<<dim3((unsigned)((slots + 255) / 256), BH), 256, 0, stream>>>(p, lv, ls.nodes, ls.pad, perm_a, perm_b);
      std::swap(perm_a, perm_b);
    }
  }
  if (a.perm_levels != nullptr)
    cudaMemcpyAsync(a.perm_levels + (size_t)pl.levels * total, perm_a, total * sizeof(int), cudaMemcpyDeviceToDevice, stream);
  pddp_widen_kernel<<<(unsigned)((total + tb - 1) / tb), tb, 0, stream>>>(perm_a, a.perm_out, total);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

int pddp_levels(int N, int C) { return make_plan(1, N, C).levels; }

// ------------------------------------------------------------------------------------------
// Built-in scratch for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand over a workspace: an inference server that has
// given every free byte of the GPU to its own memory pool and forbids further allocations, or
// code on a latency-critical path where cudaMalloc is banned because it synchronises the whole
// device.  For them the library carries one fixed scratch array in its own device image.  It is
// part of the module, so each GPU that loads the library pays for it from load to exit: hence
// the small, fixed size.  In host code the array's name is only a handle, never an address a
// kernel could use; the usable device address comes from cudaGetSymbolAddress, asked once per
// device while that device is current.
// ------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 32u << 20;   // 32 MiB
static __device__ __align__(256) unsigned char g_pddp_static_scratch[kStaticScratchBytes];

size_t pddp_static_scratch_bytes() { return kStaticScratchBytes; }

// Device address of the built-in scratch on the CURRENT device (looked up on the first call per
// device, then cached).  Returns nullptr if the lookup fails.
void* pddp_static_scratch_address() {
  static void* cached[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_pddp_static_scratch) != cudaSuccess) return nullptr;
    cached[dev] = ptr;
  }
  return cached[dev];
}

}  // namespace mcs
