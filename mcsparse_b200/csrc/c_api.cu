// C ABI of the library: argument validation and dispatch to the kernels.
// Nothing here synchronises, allocates or frees.
#include "../../include/mcsparse_b200.h"

#include <cmath>

#include "kernels.cuh"
#include "ptx.cuh"

namespace {

// One CTA, one thread: spins for a fixed number of SM cycles (bounded) and reports cycles and wall time.
__global__ void sm_clock_probe_kernel(long long* out2) {
  const long long c0 = clock64();
  const unsigned long long g0 = mcs::globaltimer_ns();
  long long c1 = c0;
  for (int i = 0; i < (1 << 20) && c1 - c0 < 40000; ++i) c1 = clock64();
  out2[0] = c1 - c0;
  out2[1] = static_cast<long long>(mcs::globaltimer_ns() - g0);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

static long long* g_clock_out = nullptr;

extern "C" {

void mcs_set_clock_buffer(int64_t* buf3) { g_clock_out = reinterpret_cast<long long*>(buf3); }

int mcs_sm_clock_probe(int64_t* out2, void* stream) {
  if (out2 == nullptr) return MCS_ERR_NULL_POINTER;
  sm_clock_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<long long*>(out2));
  return cudaGetLastError() == cudaSuccess ? 0 : MCS_ERR_LAUNCH_FAILED;
}

int mcs_version(void) { return 1; }
int mcs_built_for_sm(void) { return 100; }

const char* mcs_error_string(int code) {
  switch (code) {
    case 0: return "ok";
    case MCS_ERR_NULL_POINTER: return "required pointer is null";
    case MCS_ERR_BAD_SHAPE: return "invalid shape";
    case MCS_ERR_BAD_HEAD_DIM: return "unsupported head dimension";
    case MCS_ERR_BAD_DTYPE: return "unsupported element type";
    case MCS_ERR_BAD_ALIGNMENT: return "pointer or stride not 16-byte aligned";
    case MCS_ERR_BAD_SCALE: return "softmax scale must be positive and finite";
    case MCS_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case MCS_ERR_LAUNCH_FAILED: return "kernel launch failed";
    case MCS_ERR_UNSUPPORTED: return "unsupported configuration";
    case MCS_ERR_TOO_LARGE: return "size exceeds the supported maximum";
    default: return "unknown error";
  }
}

static int gather_attn_dispatch(const mcs_gather_attn_args* a, void* const* out_peers, int n_peers, int rows_per_peer,
                                bool dense, void* stream, bool negate = false, bool probe = false) {
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->v == nullptr || a->status == nullptr)
    return MCS_ERR_NULL_POINTER;
  if (!dense && a->gi == nullptr && (a->gi16 == nullptr || a->gi_hi == nullptr)) return MCS_ERR_NULL_POINTER;
  if (a->gi16 != nullptr && a->Sk > (1 << 17)) return MCS_ERR_TOO_LARGE;        // packed indices carry 17 bits
  if (n_peers == 0 && a->out == nullptr) return MCS_ERR_NULL_POINTER;
  if (n_peers > 0) {
    if (out_peers == nullptr) return MCS_ERR_NULL_POINTER;
    if (n_peers > 16 || rows_per_peer < 1 || (long long)rows_per_peer * n_peers < a->Sq) return MCS_ERR_BAD_SHAPE;
    for (int i = 0; i < n_peers; ++i) {
      if (out_peers[i] == nullptr) return MCS_ERR_NULL_POINTER;
      if (!aligned16(out_peers[i])) return MCS_ERR_BAD_ALIGNMENT;
    }
  }
  if (a->B < 1 || a->H < 1 || a->Sq < 1 || a->Sk < 1) return MCS_ERR_BAD_SHAPE;
  if (!dense && (a->gather_len < 128 || a->gather_len % 128 != 0)) return MCS_ERR_BAD_SHAPE;
  if (dense && (a->gl != nullptr || a->dtype == MCS_DTYPE_E4M3)) return MCS_ERR_UNSUPPORTED;
  if (a->group_rows < 1 || a->group_rows > 128) return MCS_ERR_BAD_SHAPE;
  if (a->dtype != MCS_DTYPE_BF16 && a->dtype != MCS_DTYPE_FP16 && a->dtype != MCS_DTYPE_E4M3)
    return MCS_ERR_BAD_DTYPE;
  const int esize = a->dtype == MCS_DTYPE_E4M3 ? 1 : 2;
  const int row_align = 16 / esize;  // elements per 16 bytes
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || (a->out != nullptr && !aligned16(a->out)) ||
      (a->residual != nullptr && !aligned16(a->residual)))
    return MCS_ERR_BAD_ALIGNMENT;
  for (int i = 0; i < 3; ++i) {
    if (a->q_stride[i] % row_align || a->k_stride[i] % row_align || a->v_stride[i] % row_align) return MCS_ERR_BAD_ALIGNMENT;
    if (a->o_stride[i] % 8) return MCS_ERR_BAD_ALIGNMENT;
    if (a->residual != nullptr && a->r_stride[i] % 8) return MCS_ERR_BAD_ALIGNMENT;
  }
  const long long groups = ((long long)a->Sq + a->group_rows - 1) / a->group_rows;
  if ((long long)a->B * a->H * groups > 0x7fffffffLL) return MCS_ERR_TOO_LARGE;

  mcs::GatherAttnParams p{};
  p.q = a->q; p.k = a->k; p.v = a->v; p.out = a->out; p.lse = a->lse;
  p.gi = a->gi; p.gl = a->gl;
  if (a->gi == nullptr) { p.gi16 = a->gi16; p.gi_hi = a->gi_hi; } p.residual = a->residual; p.perm = a->perm;
  p.scale_qk_log2 = a->scale_qk_log2; p.scale_v = a->scale_v; p.status = a->status;
  for (int i = 0; i < 3; ++i) {
    p.q_stride[i] = a->q_stride[i]; p.k_stride[i] = a->k_stride[i]; p.v_stride[i] = a->v_stride[i];
    p.o_stride[i] = a->o_stride[i]; p.r_stride[i] = a->r_stride[i];
  }
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.H = a->H; p.D = a->D;
  p.M = (int)groups; p.gather_len = a->gather_len; p.group_rows = a->group_rows;
  if (dense) {
    p.dense = 1;
    p.gi = nullptr; p.gi16 = nullptr; p.gi_hi = nullptr;
    p.gather_len = (a->Sk + 127) / 128 * 128;       // every key tile of the sequence
  }
  if (negate && a->residual == nullptr) return MCS_ERR_NULL_POINTER;
  if (a->flags & ~MCS_ATTN_OUT_GROUP_ORDER) return MCS_ERR_UNSUPPORTED;
  p.out_group_order = (a->flags & MCS_ATTN_OUT_GROUP_ORDER) ? 1 : 0;
  p.out_sign = negate ? -1.f : 1.f;
  p.n_out_peers = n_peers; p.out_rows_per_peer = rows_per_peer;
  for (int i = 0; i < n_peers; ++i) p.out_peer[i] = out_peers[i];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  p.clock_out = g_clock_out;

  if (probe) {
    // measurement aid: only the K/V row gather of this launch (int32 index list, head dimension 64 or 128)
    if (a->gi == nullptr || dense) return MCS_ERR_UNSUPPORTED;
    return mcs::launch_gather_rate_probe(p, esize, s);
  }
  if (a->dtype == MCS_DTYPE_E4M3) {
    if (a->scale_qk_log2 == nullptr || a->scale_v == nullptr) return MCS_ERR_NULL_POINTER;
    if (a->group_rows != 128) return MCS_ERR_BAD_SHAPE;
    if (a->D != 128) {
      // other head dimensions (the reference's FP8 kernel lists 160): the kernel that pads rows into shared memory
      if (a->D < 16 || a->D > 256 || a->D % 16 != 0) return MCS_ERR_BAD_HEAD_DIM;
      return mcs::launch_gather_attn_wide_e4m3(p, s);
    }
    return mcs::launch_gather_attn_e4m3(p, s);
  }
  if (!(a->softmax_scale > 0.f) || !std::isfinite(a->softmax_scale)) return MCS_ERR_BAD_SCALE;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  if (a->D != 64 && a->D != 128) {
    // other head dimensions (96, 144, 160, 192, 256 ...): the kernel that pads rows on their way into shared memory
    if (a->D < 8 || a->D > 256 || a->D % 8 != 0) return MCS_ERR_BAD_HEAD_DIM;
    return mcs::launch_gather_attn_wide(p, a->dtype == MCS_DTYPE_FP16, s);
  }
  return mcs::launch_gather_attn_16bit(p, a->dtype == MCS_DTYPE_FP16, s);
}

int mcs_gather_attn_fwd(const mcs_gather_attn_args* a, void* stream) {
  return gather_attn_dispatch(a, nullptr, 0, 0, false, stream);
}

int mcs_gather_attn_residual_fwd(const mcs_gather_attn_args* a, void* stream) {
  return gather_attn_dispatch(a, nullptr, 0, 0, false, stream, true);
}

int mcs_gather_rate_probe(const mcs_gather_attn_args* a, void* stream) {
  return gather_attn_dispatch(a, nullptr, 0, 0, false, stream, false, true);
}

int mcs_dense_attn_fwd(const mcs_gather_attn_args* a, void* stream) {
  return gather_attn_dispatch(a, nullptr, 0, 0, true, stream);
}

int mcs_gather_attn_fwd_sharded(const mcs_gather_attn_args* a, void* const* out_peers, int32_t n_peers,
                                int32_t rows_per_peer, void* stream) {
  if (n_peers < 1) return MCS_ERR_BAD_SHAPE;
  return gather_attn_dispatch(a, out_peers, n_peers, rows_per_peer, false, stream);
}

static int ulysses_scatter_checked(const void* src, void* const* dst_peers, int32_t n_peers, int32_t rank, int64_t rows,
                                   int64_t seg_bytes, int64_t seg_stride_bytes, int64_t src_row_bytes, void* stream, bool dma) {
  if (src == nullptr || dst_peers == nullptr) return MCS_ERR_NULL_POINTER;
  if (n_peers < 1 || n_peers > 16 || rank < 0 || rank >= n_peers || rows < 0 || seg_bytes < 16) return MCS_ERR_BAD_SHAPE;
  if (seg_stride_bytes < seg_bytes || src_row_bytes < seg_stride_bytes * (n_peers - 1) + seg_bytes) return MCS_ERR_BAD_SHAPE;
  if (seg_bytes % 16 || seg_stride_bytes % 16 || src_row_bytes % 16 || !aligned16(src)) return MCS_ERR_BAD_ALIGNMENT;
  for (int i = 0; i < n_peers; ++i) {
    if (dst_peers[i] == nullptr) return MCS_ERR_NULL_POINTER;
    if (!aligned16(dst_peers[i])) return MCS_ERR_BAD_ALIGNMENT;
  }
  auto* fn = dma ? mcs::launch_ulysses_scatter_dma : mcs::launch_ulysses_scatter;
  return fn(src, dst_peers, n_peers, rank, rows, seg_bytes, seg_stride_bytes, src_row_bytes, static_cast<cudaStream_t>(stream));
}

int mcs_ulysses_scatter(const void* src, void* const* dst_peers, int32_t n_peers, int32_t rank, int64_t rows,
                        int64_t seg_bytes, int64_t seg_stride_bytes, int64_t src_row_bytes, void* stream) {
  return ulysses_scatter_checked(src, dst_peers, n_peers, rank, rows, seg_bytes, seg_stride_bytes, src_row_bytes, stream, false);
}

int mcs_ulysses_scatter_dma(const void* src, void* const* dst_peers, int32_t n_peers, int32_t rank, int64_t rows,
                            int64_t seg_bytes, int64_t seg_stride_bytes, int64_t src_row_bytes, void* stream) {
  return ulysses_scatter_checked(src, dst_peers, n_peers, rank, rows, seg_bytes, seg_stride_bytes, src_row_bytes, stream, true);
}

int mcs_qkv_norm_rope_scatter(const mcs_qkv_epilogue_args* a, void* stream) {
  if (a == nullptr || a->src == nullptr || a->dst == nullptr || a->dst_row_stride == nullptr || a->kind == nullptr ||
      a->rope_cs == nullptr || a->gamma_q == nullptr || a->gamma_k == nullptr)
    return MCS_ERR_NULL_POINTER;
  if (a->rows < 0 || a->n_seg < 1 || a->n_seg > mcs::kQkvMaxSegments || a->row0 < 0 || a->token0 < 0) return MCS_ERR_BAD_SHAPE;
  if (a->D != 64 && a->D != 128) return MCS_ERR_BAD_HEAD_DIM;
  if (a->dtype != MCS_DTYPE_BF16 && a->dtype != MCS_DTYPE_FP16) return MCS_ERR_BAD_DTYPE;
  if (a->grid_f < 1 || a->grid_h < 1 || a->grid_w < 1 || a->pairs_t < 0 || a->pairs_h < 0 || a->pairs_t + a->pairs_h > a->D / 2)
    return MCS_ERR_BAD_SHAPE;
  if ((int64_t)a->grid_f * a->grid_h * a->grid_w > 0x7fffffffLL) return MCS_ERR_TOO_LARGE;
  if (a->token0 + a->rows > (int64_t)a->grid_f * a->grid_h * a->grid_w) return MCS_ERR_BAD_SHAPE;
  if (a->src_row_stride < (int64_t)a->n_seg * a->D || a->src_row_stride % 8 || !aligned16(a->src)) return MCS_ERR_BAD_ALIGNMENT;
  if (!(a->eps >= 0.f) || !std::isfinite(a->eps)) return MCS_ERR_BAD_SCALE;
  long long strides[mcs::kQkvMaxSegments];
  for (int i = 0; i < a->n_seg; ++i) {
    if (a->dst[i] == nullptr) return MCS_ERR_NULL_POINTER;
    if (!aligned16(a->dst[i]) || a->dst_row_stride[i] % 8 || a->dst_row_stride[i] < a->D) return MCS_ERR_BAD_ALIGNMENT;
    if (a->kind[i] < 0 || a->kind[i] > 2) return MCS_ERR_BAD_SHAPE;
    strides[i] = a->dst_row_stride[i];
  }
  mcs::QkvEpilogueParams p{};
  p.src = a->src; p.src_row_stride = a->src_row_stride; p.rows = a->rows; p.row0 = a->row0; p.token0 = a->token0;
  p.gamma_q = a->gamma_q; p.gamma_k = a->gamma_k; p.rope_cs = reinterpret_cast<const float2*>(a->rope_cs);
  p.n_seg = a->n_seg; p.D = a->D; p.grid_f = a->grid_f; p.grid_h = a->grid_h; p.grid_w = a->grid_w;
  p.pairs_t = a->pairs_t; p.pairs_h = a->pairs_h; p.eps = a->eps;
  return mcs::launch_qkv_epilogue(p, a->dst, strides, a->kind, a->dtype == MCS_DTYPE_FP16, static_cast<cudaStream_t>(stream));
}

int mcs_group_mass(const mcs_group_mass_args* a, void* stream) {
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->lse == nullptr || a->mass == nullptr || a->status == nullptr)
    return MCS_ERR_NULL_POINTER;
  if (a->B < 1 || a->H < 1 || a->Lq < 1 || a->Lk < 1) return MCS_ERR_BAD_SHAPE;
  if (a->group_rows < 1 || a->group_rows > 128) return MCS_ERR_BAD_SHAPE;
  if (a->dtype != MCS_DTYPE_BF16 && a->dtype != MCS_DTYPE_FP16) return MCS_ERR_BAD_DTYPE;
  if (a->D < 8 || a->D > 256 || a->D % 8 != 0) return MCS_ERR_BAD_HEAD_DIM;   // 64 and 128 native, others on padded layouts
  if (!(a->softmax_scale > 0.f) || !std::isfinite(a->softmax_scale)) return MCS_ERR_BAD_SCALE;
  if (!aligned16(a->q) || !aligned16(a->k)) return MCS_ERR_BAD_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if (a->q_stride[i] % 8 || a->k_stride[i] % 8) return MCS_ERR_BAD_ALIGNMENT;
  const long long groups = ((long long)a->Lq + a->group_rows - 1) / a->group_rows;
  if ((long long)a->B * a->H * groups > 0x7fffffffLL) return MCS_ERR_TOO_LARGE;
  mcs::GroupMassParams p{};
  p.q = a->q; p.k = a->k; p.lse = a->lse; p.perm = a->perm; p.mass = a->mass; p.status = a->status;
  for (int i = 0; i < 3; ++i) { p.q_stride[i] = a->q_stride[i]; p.k_stride[i] = a->k_stride[i]; }
  p.B = a->B; p.H = a->H; p.Lq = a->Lq; p.Lk = a->Lk; p.D = a->D; p.M = (int)groups;
  p.group_rows = a->group_rows; p.normalize = a->normalize;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.inv_scale = 1.0f / a->softmax_scale;
  return mcs::launch_group_mass(p, a->dtype == MCS_DTYPE_FP16, static_cast<cudaStream_t>(stream));
}

int mcs_topk_select(const float* scores, int32_t* out, const int32_t* sinks, int32_t n_sink, int64_t rows,
                    int32_t L, int32_t k_total, void* stream) {
  if (scores == nullptr || out == nullptr || (n_sink > 0 && sinks == nullptr)) return MCS_ERR_NULL_POINTER;
  if (rows < 0 || L < 1 || n_sink < 0 || n_sink > 64 || k_total < n_sink || k_total > L) return MCS_ERR_BAD_SHAPE;
  if (rows == 0) return 0;
  mcs::TopkParams p{scores, out, sinks, (long long)rows, L, k_total, n_sink, nullptr};
  return mcs::launch_topk_select(p, static_cast<cudaStream_t>(stream));
}

int mcs_index_pack17(const int32_t* gi, int64_t n, uint16_t* lo, uint32_t* hi, void* stream) {
  if (gi == nullptr || lo == nullptr || hi == nullptr) return MCS_ERR_NULL_POINTER;
  if (n < 0 || n % 128 != 0) return MCS_ERR_BAD_SHAPE;
  return mcs::launch_index_pack17(gi, (long long)n, lo, hi, static_cast<cudaStream_t>(stream));
}

int mcs_index_unpack17(const uint16_t* lo, const uint32_t* hi, int64_t n, int32_t* gi, void* stream) {
  if (gi == nullptr || lo == nullptr || hi == nullptr) return MCS_ERR_NULL_POINTER;
  if (n < 0 || n % 128 != 0) return MCS_ERR_BAD_SHAPE;
  return mcs::launch_index_unpack17(lo, hi, (long long)n, gi, static_cast<cudaStream_t>(stream));
}

int mcs_topk_select_var(const float* scores, int32_t* out, const int32_t* sinks, int32_t n_sink, int64_t rows, int32_t L,
                        int32_t k_max, const int32_t* k_rows, void* stream) {
  if (scores == nullptr || out == nullptr || k_rows == nullptr || (n_sink > 0 && sinks == nullptr)) return MCS_ERR_NULL_POINTER;
  if (rows < 0 || L < 1 || n_sink < 0 || n_sink > 64 || k_max < n_sink || k_max > L) return MCS_ERR_BAD_SHAPE;
  if (rows == 0) return 0;
  mcs::TopkParams p{scores, out, sinks, (long long)rows, L, k_max, n_sink, k_rows};
  return mcs::launch_topk_select(p, static_cast<cudaStream_t>(stream));
}

int mcs_topp_count(const float* scores, const int32_t* sinks, int32_t n_sink, int64_t rows, int32_t L, float topp, int32_t* counts,
                   void* stream) {
  if (scores == nullptr || counts == nullptr || (n_sink > 0 && sinks == nullptr)) return MCS_ERR_NULL_POINTER;
  if (rows < 0 || L < 1 || n_sink < 0 || n_sink > 64 || n_sink >= L) return MCS_ERR_BAD_SHAPE;
  if (!(topp > 0.f) || !(topp <= 1.f)) return MCS_ERR_BAD_SCALE;
  return mcs::launch_topp_count(scores, sinks, n_sink, (long long)rows, L, topp, counts, static_cast<cudaStream_t>(stream));
}

int64_t mcs_pddp_workspace_bytes(int32_t BH, int32_t N, int32_t C) { return (int64_t)mcs::pddp_workspace_bytes(BH, N, C); }
int64_t mcs_pddp_start_vector_rows(int32_t BH, int32_t N, int32_t C) {
  if (BH < 1 || N < 1 || C < 1) return 0;
  return mcs::pddp_start_vector_rows(BH, N, C);
}
int32_t mcs_pddp_levels(int32_t N, int32_t C) { return (N < 1 || C < 1) ? 0 : mcs::pddp_levels(N, C); }

int mcs_pddp_perm(const mcs_pddp_args* a, void* stream) {
  if (a == nullptr || a->x == nullptr || a->perm_out == nullptr || a->workspace == nullptr || a->status == nullptr)
    return MCS_ERR_NULL_POINTER;
  if (a->BH < 1 || a->N < 1 || a->C < 1 || a->pow_iters < 0) return MCS_ERR_BAD_SHAPE;
  if (a->D < 8 || a->D > 256 || a->D % 8 != 0) return MCS_ERR_BAD_HEAD_DIM;   // 64 / 128: tensor-core Gram path; others: Gram-free path
  if (a->dtype != MCS_DTYPE_BF16 && a->dtype != MCS_DTYPE_FP16) return MCS_ERR_BAD_DTYPE;
  if (!aligned16(a->x) || a->x_stride_bh % 8 || a->x_stride_row % 8) return MCS_ERR_BAD_ALIGNMENT;
  const size_t need = mcs::pddp_workspace_bytes(a->BH, a->N, a->C);
  if (need == 0) return MCS_ERR_TOO_LARGE;
  if ((int64_t)need > a->workspace_bytes) return MCS_ERR_WORKSPACE_TOO_SMALL;
  if (a->start_vectors == nullptr && mcs::pddp_levels(a->N, a->C) > 0) return MCS_ERR_NULL_POINTER;
  mcs::PddpArgs p{};
  p.x = a->x; p.x_stride_bh = a->x_stride_bh; p.x_stride_row = a->x_stride_row;
  p.BH = a->BH; p.N = a->N; p.D = a->D; p.C = a->C; p.pow_iters = a->pow_iters; p.fp16 = a->dtype == MCS_DTYPE_FP16;
  p.start_vectors = a->start_vectors; p.perm_out = reinterpret_cast<long long*>(a->perm_out);
  p.proj_levels = a->proj_levels; p.perm_levels = a->perm_levels;
  p.workspace = a->workspace; p.workspace_bytes = (size_t)a->workspace_bytes; p.status = a->status;
  return mcs::launch_pddp(p, static_cast<cudaStream_t>(stream));
}

int64_t mcs_pddp_static_scratch_bytes(void) { return (int64_t)mcs::pddp_static_scratch_bytes(); }

int mcs_pddp_perm_static(const mcs_pddp_args* a, void* stream) {
  if (a == nullptr) return MCS_ERR_NULL_POINTER;
  if (a->BH < 1 || a->N < 1 || a->C < 1) return MCS_ERR_BAD_SHAPE;
  const size_t need = mcs::pddp_workspace_bytes(a->BH, a->N, a->C);
  if (need == 0 || need > mcs::pddp_static_scratch_bytes()) return MCS_ERR_TOO_LARGE;   // beyond the built-in scratch
  void* scratch = mcs::pddp_static_scratch_address();     // first call on a device resolves the symbol
  if (scratch == nullptr) return MCS_ERR_LAUNCH_FAILED;
  mcs_pddp_args b = *a;
  b.workspace = scratch;
  b.workspace_bytes = (int64_t)mcs::pddp_static_scratch_bytes();
  return mcs_pddp_perm(&b, stream);
}

static int perm_rows(const void* x, void* out, const int64_t* perm, int32_t BH, int32_t L, int32_t row_bytes, int64_t x_bh,
                     int64_t x_row, int64_t o_bh, int64_t o_row, bool invert, void* stream) {
  if (x == nullptr || out == nullptr || perm == nullptr) return MCS_ERR_NULL_POINTER;
  if (BH < 1 || L < 1 || row_bytes < 16) return MCS_ERR_BAD_SHAPE;
  if (row_bytes % 16 || x_bh % 16 || x_row % 16 || o_bh % 16 || o_row % 16 || !aligned16(x) || !aligned16(out))
    return MCS_ERR_BAD_ALIGNMENT;
  return mcs::launch_perm_rows(x, out, reinterpret_cast<const long long*>(perm), BH, L, row_bytes, x_bh, x_row, o_bh, o_row, invert,
                               static_cast<cudaStream_t>(stream));
}
int mcs_perm_apply(const void* x, void* out, const int64_t* perm, int32_t BH, int32_t L, int32_t row_bytes, int64_t x_bh,
                   int64_t x_row, int64_t o_bh, int64_t o_row, void* stream) {
  return perm_rows(x, out, perm, BH, L, row_bytes, x_bh, x_row, o_bh, o_row, false, stream);
}
int mcs_perm_invert(const void* x, void* out, const int64_t* perm, int32_t BH, int32_t L, int32_t row_bytes, int64_t x_bh,
                    int64_t x_row, int64_t o_bh, int64_t o_row, void* stream) {
  return perm_rows(x, out, perm, BH, L, row_bytes, x_bh, x_row, o_bh, o_row, true, stream);
}

}  // extern "C"
