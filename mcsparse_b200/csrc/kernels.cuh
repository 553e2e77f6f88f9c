// Internal launch interfaces shared between the kernels and the C ABI layer.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace mcs {

struct GatherAttnParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  const int32_t* gi;
  const uint16_t* gi16;        // packed indices (instead of gi): low 16 bits ...
  const uint32_t* gi_hi;       // ... and bit 16 as a bit plane, one word per 32 entries
  const int32_t* gl;
  const void* residual;
  const int64_t* perm;
  const float* scale_qk_log2;  // e4m3 only
  const float* scale_v;        // e4m3 only
  int* status;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3], r_stride[3];
  int B, Sq, Sk, H, D, M, gather_len, group_rows;
  float scale_log2;  // softmax_scale * log2(e)
  long long* clock_out;  // optional: {SM cycles, nanoseconds, tiles} of CTA 0's tile loop (mcs_set_clock_buffer)
  // sequence-sharded output (Ulysses): row r' of the output goes to out_peer[r' / out_rows_per_peer] at local
  // row r' % out_rows_per_peer (peer or local memory alike)
  void* out_peer[16];
  float out_sign;           // +1: out = attention + residual; -1: out = residual - attention (residual construction)
  int dense;                // 1: no index list, every query group attends to all Sk keys (tail of the last tile masked)
  int n_out_peers;          // 0 = not sharded
  int out_rows_per_peer;
  int out_group_order;      // 1: with perm, output and lse rows stay in permuted (group) order
};

// Tensor maps of K and V for the dense mode (TMA tile loads of 128 contiguous key rows): 4-D maps with the
// head dimension innermost and (head, row, batch) in the order of ascending stride; pos_* say at which
// coordinate position each of them sits (1..3).  Opaque 128-byte blobs (CUtensorMap), 64-byte aligned.
struct alignas(64) DenseTileMaps {
  unsigned long long k[16];
  unsigned long long v[16];
  int k_pos_h, k_pos_row, k_pos_b;
  int v_pos_h, v_pos_row, v_pos_b;
  int valid;     // 0: maps not built, the dense mode gathers rows with cp.async like the sparse mode
};

// (tensor_map.cu) 4-D tensor map of a (B, S, H, D) tensor of 16-bit elements with element strides {batch, row,
// head}; box = 64 elements x 128 rows, 128-byte swizzle.  `out` receives the 128-byte map, pos_* the coordinate
// positions (1..3) of head, row and batch.  False if the layout cannot be described or the driver has no encoder.
bool encode_tile_map(const void* base, const int64_t* stride, int B, int S, int H, int D, unsigned long long* out,
                     int& pos_h, int& pos_row, int& pos_b);

// Tensor map of K for the group-mass kernel (see DenseTileMaps)
struct alignas(64) KeyTileMap {
  unsigned long long k[16];
  int pos_h, pos_row, pos_b;
  int valid;     // 0: key tiles are copied with cp.async
};

struct GroupMassParams {
  const void* q;        // (B, Lq, H, D) strided
  const void* k;        // (B, Lk, H, D) strided
  const float* lse;     // (B*H, Lq) in group (permuted) order
  const int64_t* perm;  // (B*H, Lq) or null
  float* mass;          // (B*H, M, Lk)
  int* status;
  int64_t q_stride[3], k_stride[3];
  int B, H, Lq, Lk, D, M, group_rows, normalize;
  float scale_log2;     // scale * log2(e)
  float inv_scale;      // 1 / scale
};

struct PddpParams {
  const void* x;
  long long x_stride_bh, x_stride_row;   // elements
  int N, D, BH, pow_iters;
  int* tables; int table_stride; int max_items;
  float* partial;                        // [BH][max_items][128*128 + 128]
  float* dir; int dir_nodes;             // [BH][dir_nodes][128]
  unsigned long long* keys; size_t key_stride;
  int* status;
};
struct PddpArgs {
  const void* x; long long x_stride_bh, x_stride_row;
  int BH, N, D, C, pow_iters; bool fp16;
  const float* start_vectors;            // all levels, level-major: (BH * nodes_l, D) each
  long long* perm_out;                   // (BH, N)
  float* proj_levels;                    // optional (levels, BH, N)
  int* perm_levels;                      // optional (levels + 1, BH, N)
  void* workspace; size_t workspace_bytes;
  int* status;
};
size_t pddp_workspace_bytes(int BH, int N, int C);
long long pddp_start_vector_rows(int BH, int N, int C);
int pddp_levels(int N, int C);
int launch_pddp(const PddpArgs& a, cudaStream_t stream);
size_t pddp_static_scratch_bytes();
void* pddp_static_scratch_address();

int launch_perm_rows(const void* x, void* out, const long long* perm, int BH, int L, int row_bytes, long long x_bh,
                     long long x_row, long long o_bh, long long o_row, bool invert, cudaStream_t stream);

struct TopkParams {
  const float* scores;   // (rows, L)
  int32_t* out;          // (rows, k_total) ascending
  const int32_t* sinks;  // n_sink distinct indices in [0, L)
  long long rows;
  int L, k_total, n_sink;
  const int32_t* k_rows;  // optional per-row budgets (sinks included), clamped to [n_sink, k_total]; entries beyond are zeroed
};
int launch_index_pack17(const int32_t* gi, long long n, uint16_t* lo, uint32_t* hi, cudaStream_t stream);
int launch_index_unpack17(const uint16_t* lo, const uint32_t* hi, long long n, int32_t* gi, cudaStream_t stream);
int launch_topp_count(const float* scores, const int32_t* sinks, int n_sink, long long rows, int L, float topp, int32_t* counts,
                      cudaStream_t stream);

int launch_topk_select(const TopkParams& p, cudaStream_t stream);
int launch_group_mass(const GroupMassParams& p, bool fp16, cudaStream_t stream);
int launch_gather_attn_16bit(const GatherAttnParams& p, bool fp16, cudaStream_t stream);
int launch_gather_attn_e4m3(const GatherAttnParams& p, cudaStream_t stream);
// measurement aid: the K/V row gather of a sparse launch alone (gather_attn.cu)
int launch_gather_rate_probe(const GatherAttnParams& p, int elem_bytes, cudaStream_t stream);
// head dimensions other than 64 and 128 (multiples of 8 up to 256), bf16 / fp16 (gather_attn_wide.cu)
int launch_gather_attn_wide(const GatherAttnParams& p, bool fp16, cudaStream_t stream);
int launch_gather_attn_wide_e4m3(const GatherAttnParams& p, cudaStream_t stream);   // e4m3, multiples of 16 up to 256

// QKV-projection epilogue: RMSNorm + 3-D rotary embedding + store into the (peer) buffers the attention reads (qkv_epilogue.cu)
constexpr int kQkvMaxSegments = 128;
struct QkvEpilogueParams {
  const void* src;            // (rows, n_seg, D) 16-bit, row stride src_row_stride elements
  long long src_row_stride;
  long long rows;
  long long row0;             // destination row of local row 0 (rank * rows in a sequence-sharded layer)
  long long token0;           // grid position (flattened, frame-major) of local row 0
  const float* gamma_q;       // (D) RMSNorm weights of query slices
  const float* gamma_k;       // (D) RMSNorm weights of key slices
  const float2* rope_cs;      // (grid_f + grid_h + grid_w, D / 2) (cos, sin) per axis position and rotation pair
  int n_seg, D;
  int grid_f, grid_h, grid_w; // tokens are numbered frame-major over this grid
  int pairs_t, pairs_h;       // rotation pairs [0, pairs_t) follow the frame, the next pairs_h the row, the rest the column
  float eps;
};
int launch_qkv_epilogue(const QkvEpilogueParams& p, void* const* dst, const long long* dst_row_stride, const int* kind,
                        bool fp16, cudaStream_t stream);

// Sequence-to-head reshard by peer stores (see reshard.cu)
int launch_ulysses_scatter_dma(const void* src, void* const* dst_peers, int n_peers, int rank, long long rows,
                               long long seg_bytes, long long seg_stride_bytes, long long src_row_bytes, cudaStream_t stream);
int launch_ulysses_scatter(const void* src, void* const* dst_peers, int n_peers, int rank, long long rows,
                           long long seg_bytes, long long seg_stride_bytes, long long src_row_bytes, cudaStream_t stream);

}  // namespace mcs
