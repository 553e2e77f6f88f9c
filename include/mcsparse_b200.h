/*
 * mcsparse_b200 — C ABI of the B200 (sm_100a) token-sparse attention hot path.
 *
 * Every entry point takes plain device pointers, sizes and element strides, and
 * a CUDA stream (passed as void* so that the header needs no CUDA include).
 * Conventions:
 *   - return value 0 = launched; negative = argument error, nothing launched
 *     (see mcs_error_string);
 *   - entry points never synchronise, never allocate and never free; scratch
 *     memory, where a kernel needs it, is passed in by the caller together with
 *     its size (query the size with the matching *_workspace_bytes function);
 *   - `status` is a caller-owned int32 in device memory, zero-initialised once.
 *     Kernels that wait on hardware barriers bound every wait; if a wait
 *     expires they store a non-zero code there and return cleanly.  A caller
 *     that wants the check reads the word after synchronising its stream;
 *   - all tensors keep the layouts of the reference's Python entry points so a
 *     binding only forwards data_ptr()/stride().
 *
 * Each declaration cites the reference interface it replaces, by the path of
 * the file inside the mcsparse project.
 */
#ifndef MCSPARSE_B200_H_
#define MCSPARSE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of q/k/v. */
#define MCS_DTYPE_BF16 0
#define MCS_DTYPE_FP16 1
#define MCS_DTYPE_E4M3 2

/* Argument errors (returned, never stored in the status word). */
#define MCS_ERR_NULL_POINTER (-1)
#define MCS_ERR_BAD_SHAPE (-2)
#define MCS_ERR_BAD_HEAD_DIM (-3)
#define MCS_ERR_BAD_DTYPE (-4)
#define MCS_ERR_BAD_ALIGNMENT (-5)
#define MCS_ERR_BAD_SCALE (-6)
#define MCS_ERR_WORKSPACE_TOO_SMALL (-7)
#define MCS_ERR_LAUNCH_FAILED (-8)
#define MCS_ERR_UNSUPPORTED (-9)
#define MCS_ERR_TOO_LARGE (-10)

/* Library version and the compute capability the kernels were built for (100). */
int mcs_version(void);
int mcs_built_for_sm(void);
const char* mcs_error_string(int code);

/*
 * Gather-KV sparse flash-attention forward (bf16 / fp16 / e4m3 inputs).
 *
 * Replaces: mcsparse/kernels/flash_mcsa/ops/flash_sparse_attn/cute/interface.py:108-340
 * (flash_attn_gather_kv_func) and :346-570 (flash_attn_gather_kv_fp8_func); also
 * absorbs the copies its caller makes around it,
 * mcsparse/kernels/flash_mcsa/token_sparse.py:1436-1459 (_sp layout copies),
 * :1095-1112 (residual add), and mcsparse/kernels/flash_mcsa/pca_group.py:40-61
 * (apply_perm / invert_perm) when `perm` is given.
 *
 * For query group m = row / group_rows of (batch b, head h), the key set is the
 * multiset gi[b,h,m, 0 : T*128], T = gl[b,h,m] if gl != NULL else gather_len/128.
 *   out[b, row', h, :] = softmax_j(scale * q_row . k[gi_j]) @ v[gi_j]  (+ residual[b,h,row,:])
 * where, with perm != NULL, "row" counts positions in the permuted query order,
 * the query vector is q[b, perm[b*H+h, row], h, :] and row' = perm[b*H+h, row]
 * (the output is written back in the original token order); without perm,
 * row' = row.  lse (optional) is the natural-log log-sum-exp of the scaled logits,
 * stored at [b, h, row'].
 *
 * For MCS_DTYPE_E4M3: logits are (q8.k8) * scale_qk_log2[b,h,m] in the log2 domain,
 * the output is multiplied by scale_v[b,h], out/residual are bf16.
 */
typedef struct mcs_gather_attn_args {
  const void* q;        /* (B, Sq, H, D) element strides q_stride[0..2], last dim contiguous */
  const void* k;        /* (B, Sk, H, D) */
  const void* v;        /* (B, Sk, H, D) */
  void* out;            /* (B, Sq, H, D), bf16/fp16 (bf16 for e4m3 inputs) */
  float* lse;           /* (B, H, Sq) contiguous fp32, or NULL */
  const int32_t* gi;    /* (B, H, M, gather_len) contiguous int32 */
  const int32_t* gl;    /* (B, H, M) contiguous int32 tile counts, or NULL */
  const void* residual; /* (B, H, Sq, D) element strides r_stride[0..2] (b, h, row), or NULL */
  const int64_t* perm;  /* (B*H, Sq) contiguous int64, or NULL */
  const float* scale_qk_log2; /* e4m3 only: (B, H, M) contiguous fp32 */
  const float* scale_v;       /* e4m3 only: (B, H) contiguous fp32 */
  int32_t* status;      /* device int32, see file comment */
  int64_t q_stride[3];  /* batch, sequence, head (elements) */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int64_t r_stride[3];  /* batch, head, row (elements) */
  int32_t B, Sq, Sk, H, D;  /* D: 16-bit types: a multiple of 8 up to 256 (64 and 128 on the persistent kernel); e4m3: a multiple of 16 up to 256 (128 on the persistent kernel) */
  int32_t gather_len;   /* multiple of 128 */
  int32_t group_rows;   /* query rows per group, 1..128 (reference: 128) */
  int32_t dtype;        /* MCS_DTYPE_* */
  float softmax_scale;  /* > 0; ignored for e4m3 (scale_qk_log2 carries it) */
  int32_t flags;        /* MCS_ATTN_* bits, 0 for the behaviour described above */
  const uint16_t* gi16; /* with gi == NULL: the same indices in packed form, low 16 bits of every entry ... */
  const uint32_t* gi_hi;/* ... and bit 16 as a bit plane, one 32-bit word per 32 consecutive entries (Sk <= 131,072) */
} mcs_gather_attn_args;

/* With perm != NULL: read the query rows through the permutation but keep out and lse in the permuted
 * (group) order, row' = row.  The anchor step wants exactly that: the dense output and LSE of the
 * regrouped queries without a gathered copy of Q (mcsparse/kernels/flash_mcsa/token_sparse.py:1057-1058
 * makes that copy before the dense pass at :1151). */
#define MCS_ATTN_OUT_GROUP_ORDER 1

int mcs_gather_attn_fwd(const mcs_gather_attn_args* args, void* stream);

/*
 * Residual construction of the anchor step in one pass: out = residual - attention, where args->residual
 * (required) holds the dense attention output in (B, H, Sq, D) layout and the attention is the sparse
 * attention defined above; fp32 subtraction, one rounding.  The result is what later reuse steps pass back
 * as `residual`.
 *
 * Replaces: the sparse pass followed by the elementwise `out_full - out_sparse` of
 * mcsparse/kernels/flash_mcsa/token_sparse.py:1209-1216.
 */
int mcs_gather_attn_residual_fwd(const mcs_gather_attn_args* args, void* stream);

/*
 * Dense attention with log-sum-exp through the same kernel: every query group attends to all Sk keys
 * (args->gi, gl, gather_len are ignored; bf16 / fp16 only; the part of the last 128-key tile beyond Sk is
 * masked).  residual, perm and lse work as above.  This is the input of the anchor step: the dense output
 * (returned on anchor steps, and the minuend of the cached residual) and the per-row LSE that
 * mcs_group_mass needs.
 *
 * Replaces: the FlashAttention-3 call of mcsparse/kernels/flash_mcsa/ops/full_attn.py:88-121 as used by
 * mcsparse/kernels/flash_mcsa/token_sparse.py:1151 (dense pass with LSE in the calibrate branch).
 */
int mcs_dense_attn_fwd(const mcs_gather_attn_args* args, void* stream);

/*
 * The same kernel with a SEQUENCE-SHARDED output: row r' of the output is written to
 * out_peers[r' / rows_per_peer] at local row r' % rows_per_peer (strides args->o_stride, batch and head
 * offsets as usual; args->out is ignored).  out_peers is a host array of n_peers (<= 16) device pointers
 * that this GPU can store to: its own memory and peers' memory mapped into this process (CUDA IPC or
 * virtual-memory handles, NVLink).  This is the head-to-sequence all-to-all of Ulysses context
 * parallelism fused into the attention epilogue: each finished row goes straight to the rank that owns
 * its token, so no reverse all-to-all and no unpack copy exist.
 *
 * Replaces: the second all-to-all of diffusers' _templated_context_parallel_attention around the
 * reference's forward_op (mcsparse/h3/context_parallel.py:220-229).  The caller orders the launch
 * against the peers' later reads (a stream-ordered collective or event exchange); nothing in the kernel
 * waits for another GPU.
 */
int mcs_gather_attn_fwd_sharded(const mcs_gather_attn_args* args, void* const* out_peers, int32_t n_peers,
                                int32_t rows_per_peer, void* stream);

/*
 * Sequence-to-head reshard by peer stores (the first all-to-all of the same path): src holds `rows`
 * local tokens of src_row_bytes each; the seg_bytes at offset r * seg_stride_bytes of a row are the heads
 * wanted by rank r (all of its heads, or a chunk of them when the exchange is pipelined), and are written
 * to dst_peers[r] + (rank * rows + s) * seg_bytes for local row s.  dst_peers is a host array of device
 * pointers this GPU can store to (see above).  16-byte granularity.
 */
int mcs_ulysses_scatter(const void* src, void* const* dst_peers, int32_t n_peers, int32_t rank, int64_t rows,
                        int64_t seg_bytes, int64_t seg_stride_bytes, int64_t src_row_bytes, void* stream);

/*
 * The same reshard, same arguments and result, issued as one strided 2-D device copy per peer on the copy
 * engines instead of a kernel: for head chunks that are exchanged while an attention kernel occupies the SMs.
 */
int mcs_ulysses_scatter_dma(const void* src, void* const* dst_peers, int32_t n_peers, int32_t rank, int64_t rows,
                            int64_t seg_bytes, int64_t seg_stride_bytes, int64_t src_row_bytes, void* stream);

/*
 * Epilogue of the QKV projection of a context-parallel attention layer, fused with the sequence-to-head
 * exchange: for `rows` local tokens and `n_seg` head slices of D elements per token (slice s of token i at
 * src + i * src_row_stride + s * D, 16-bit elements), query (kind 0) and key (kind 1) slices are RMS-normalised
 * over their D elements with weights gamma_q / gamma_k (fp32, x * rsqrt(mean(x^2) + eps) * g) and rotated by the
 * 3-D rotary embedding of the token; value slices (kind 2) are copied.  Slice s of token i is stored at
 * dst[s] + (row0 + i) * dst_row_stride[s] elements: an address in this GPU's memory or a peer's (see
 * mcs_gather_attn_fwd_sharded), so every slice lands directly in the (L, heads, D) buffer of the rank that owns
 * its head.  Token i sits at flattened position token0 + i of a frame-major (grid_f, grid_h, grid_w) grid;
 * rotation pair p of a slice (elements 2p, 2p+1) follows the frame index for p < pairs_t, the grid row for the
 * next pairs_h pairs and the grid column for the rest; rope_cs is a device table of (cos, sin) float pairs of
 * shape (grid_f + grid_h + grid_w, D / 2): row = axis offset + position on that axis, column = pair.
 * dst, dst_row_stride and kind are HOST arrays of n_seg (<= 128) entries.  D is 64 or 128.
 *
 * Replaces: the stretch between the model's QKV projection and the reference's forward_op, i.e. the model's
 * q/k RMSNorm and rotary embedding followed by the first all-to-all of diffusers'
 * _templated_context_parallel_attention (mcsparse/h3/context_parallel.py:165-176, 220-229).
 */
typedef struct mcs_qkv_epilogue_args {
  const void* src;
  const float* gamma_q;
  const float* gamma_k;
  const float* rope_cs;
  void* const* dst;                /* host array, n_seg device pointers */
  const int64_t* dst_row_stride;   /* host array, elements */
  const int32_t* kind;             /* host array: 0 query, 1 key, 2 value */
  int64_t src_row_stride;          /* elements */
  int64_t rows, row0, token0;
  int32_t n_seg, D;
  int32_t grid_f, grid_h, grid_w;
  int32_t pairs_t, pairs_h;
  int32_t dtype;                   /* MCS_DTYPE_BF16 or MCS_DTYPE_FP16 */
  float eps;
} mcs_qkv_epilogue_args;

int mcs_qkv_norm_rope_scatter(const mcs_qkv_epilogue_args* args, void* stream);

/*
 * Anchor-step group mass: mass[b,h,m,j] = sum_{i in group m} exp(scale * q_i . k_j - lse_i), fp32.
 *
 * Replaces: mcsparse/kernels/flash_mcsa/ops/triton/block_probs.py:27-117
 * (_token_probs_kernel_bf16 / _compute_token_probs_bf16_triton) as called from
 * mcsparse/kernels/flash_mcsa/token_sparse.py:590-595 (_compute_token_probs).
 * Differences: the result is fp32 (the reference rounds to bf16, which creates rank ties),
 * and it is the plain sum unless `normalize` is set (then it is divided by the number of rows
 * in the group, the reference's convention).  Groups are `group_rows` consecutive positions
 * of the query order given by `perm` (identity if NULL); `lse` is indexed by position in that
 * order, as the dense pass that produced it ran on the permuted queries
 * (token_sparse.py:1058, 1151).
 */
typedef struct mcs_group_mass_args {
  const void* q;        /* (B, Lq, H, D) element strides q_stride[0..2], bf16/fp16 */
  const void* k;        /* (B, Lk, H, D) */
  const float* lse;     /* (B*H, Lq) contiguous fp32, natural log, softmax scale included */
  const int64_t* perm;  /* (B*H, Lq) contiguous int64, or NULL */
  float* mass;          /* (B*H, M, Lk) contiguous fp32, M = ceil(Lq / group_rows) */
  int32_t* status;
  int64_t q_stride[3];
  int64_t k_stride[3];
  int32_t B, H, Lq, Lk, D;   /* D: a multiple of 8 up to 256 (64 and 128 on the tuned tile layouts) */
  int32_t group_rows;   /* 1..128 */
  int32_t dtype;        /* MCS_DTYPE_BF16 or MCS_DTYPE_FP16 */
  int32_t normalize;    /* 0: sum, 1: divide by rows in group */
  float softmax_scale;  /* > 0 */
} mcs_group_mass_args;

int mcs_group_mass(const mcs_group_mass_args* args, void* stream);

/*
 * Exact top-k token selection with forced sink tokens.
 *
 * Replaces: mcsparse/kernels/flash_mcsa/token_sparse.py:755-945 (_select_topk_tokens, topk mode:
 * sink masking :788-803, torch.topk :825-840, sink merge and 128-alignment :902-945).
 * For each of `rows` score rows of length L (a row = one query group of one head) writes, in
 * ascending order, the n_sink sink indices plus the (k_total - n_sink) non-sink indices with the
 * highest fp32 score; ties go to the lowest index.  Requirements: n_sink <= 64, sinks distinct
 * and in [0, L), n_sink <= k_total <= L.  The result is a pure function of the fp32 scores.
 */
int mcs_topk_select(const float* scores, int32_t* out, const int32_t* sinks, int32_t n_sink,
                    int64_t rows, int32_t L, int32_t k_total, void* stream);

/*
 * Packed form of an index tensor for sequences of up to 131,072 keys: n entries (a multiple of 128) become n 16-bit
 * values and n / 32 words holding bit 16 of 32 consecutive entries each: 272 instead of 512 bytes per tile of 128.
 * The attention entry points read this form directly (args->gi16 / gi_hi).  mcs_index_unpack17 is the inverse.
 * No counterpart in the reference, which keeps int32 indices (639 MB per layer at its production shape,
 * mcsparse/h3/token_sparse_dispatch.py:866-872) and moves them to host memory instead.
 */
int mcs_index_pack17(const int32_t* gi, int64_t n, uint16_t* lo, uint32_t* hi, void* stream);
int mcs_index_unpack17(const uint16_t* lo, const uint32_t* hi, int64_t n, int32_t* gi, void* stream);

/*
 * The same selection with a budget of its own for every row: row r gets the sinks plus its (k_rows[r] - n_sink)
 * best other tokens, ascending, in out[r * k_max ...]; the entries from k_rows[r] up to k_max are set to 0 (the
 * attention kernel never reads them: the caller passes ceil-free tile counts k_rows[r] / 128 as gather_kv_lengths).
 * k_rows is a device array of `rows` int32, each clamped to [n_sink, k_max].
 *
 * Replaces: the variable-length branches of mcsparse/kernels/flash_mcsa/token_sparse.py:755-945 (per-head budgets
 * :825-835, top-p :842-852, top-k-or-top-p :854-876, padding :924-934), where the reference sorts every row in full
 * and slices prefixes of different lengths.
 */
int mcs_topk_select_var(const float* scores, int32_t* out, const int32_t* sinks, int32_t n_sink, int64_t rows,
                        int32_t L, int32_t k_max, const int32_t* k_rows, void* stream);

/*
 * Top-p budgets: counts[r] = number of leading tokens of row r, in descending order of score, whose scores summed
 * BEFORE each of them stay below topp (at least 1, everything if the row's total stays below topp); sink tokens are
 * left out of the ranking and of the count.  scores: (rows, L) fp32 normalised masses; 0 < topp <= 1.
 *
 * Replaces: the sort + cumulative sum + mask count of mcsparse/kernels/flash_mcsa/token_sparse.py:842-852 and
 * :862-866 (topp / topk_topp modes); the tile alignment and the lower bound of topk_topp stay on the host.
 */
int mcs_topp_count(const float* scores, const int32_t* sinks, int32_t n_sink, int64_t rows, int32_t L, float topp,
                   int32_t* counts, void* stream);

/*
 * Fast PDDP query grouping: per (batch*head) permutation that puts similar rows into aligned
 * blocks of C rows by recursive principal-direction bisection.
 *
 * Replaces: mcsparse/kernels/flash_mcsa/pca_group.py:141-243 (pca_group_perm), as called from
 * mcsparse/kernels/flash_mcsa/token_sparse.py:254-293 (TokenSparseCache.get_or_make_perm).
 * x: (BH, N, D) bf16/fp16, element strides x_stride_bh / x_stride_row, rows contiguous,
 * D in {64, 128}.  perm_out: (BH, N) int64, x[b, perm[b, i]] is the i-th reordered row.
 * start_vectors: the power-iteration start vectors, level-major: for level l a
 * (BH * nodes_l, D) fp32 block (row b * nodes_l + node), mcs_pddp_start_vector_rows() rows in
 * total.  The reference draws them from a generator on the tensor's device (:184-185, :224); host
 * and device generators differ, so they are an input here.
 * Optional dumps for checking: proj_levels (levels, BH, N) fp32 = projection of the row at every
 * position of the order entering the level; perm_levels (levels + 1, BH, N) int32 = the order
 * entering every level and the final one.  Given the fp32 projections the new order is their
 * stable ascending sort inside every node: a pure function of those values.
 * workspace: mcs_pddp_workspace_bytes(BH, N, C) bytes of device memory (0 = unsupported shape).
 */
typedef struct mcs_pddp_args {
  const void* x;
  const float* start_vectors;
  int64_t* perm_out;
  float* proj_levels;    /* or NULL */
  int32_t* perm_levels;  /* or NULL */
  void* workspace;
  int32_t* status;
  int64_t x_stride_bh, x_stride_row;
  int64_t workspace_bytes;
  int32_t BH, N, D, C, pow_iters;   /* D: a multiple of 8 up to 256 (64 and 128 through the tensor-core Gram matrix) */
  int32_t dtype;         /* MCS_DTYPE_BF16 or MCS_DTYPE_FP16 */
} mcs_pddp_args;

int64_t mcs_pddp_workspace_bytes(int32_t BH, int32_t N, int32_t C);
int64_t mcs_pddp_start_vector_rows(int32_t BH, int32_t N, int32_t C);
int32_t mcs_pddp_levels(int32_t N, int32_t C);
int mcs_pddp_perm(const mcs_pddp_args* args, void* stream);

/*
 * Fast PDDP grouping without a caller-provided workspace.  No counterpart in the reference: this
 * entry point exists for callers that are not allowed to allocate device memory (a server whose
 * memory pool owns the whole GPU, a latency path where cudaMalloc is forbidden because it
 * synchronises the device).  Same arguments and results as mcs_pddp_perm, except that
 * `workspace` / `workspace_bytes` are ignored: the scratch is a fixed array inside the library's
 * device image, mcs_pddp_static_scratch_bytes() (32 MiB) large, held by every GPU that loads the
 * library until the process exits.  Shapes whose mcs_pddp_workspace_bytes() exceeds that size are
 * rejected with MCS_ERR_TOO_LARGE.  It calls no allocation routine of any kind.
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call outside any stream capture.  All calls on a device share the one array and
 * find the previous call's contents in it (nothing in it needs to start at zero: every region is
 * written before it is read); two calls that overlap on the GPU, e.g. on different streams, race.
 */
int64_t mcs_pddp_static_scratch_bytes(void);
int mcs_pddp_perm_static(const mcs_pddp_args* args, void* stream);

/*
 * Row permutation of a (BH, L, D) tensor, 16-byte aligned rows of row_bytes bytes, byte strides.
 * apply : out[b, i] = x[b, perm[b, i]]   replaces mcsparse/kernels/flash_mcsa/pca_group.py:40-42, 52-55
 * invert: out[b, perm[b, i]] = x[b, i]   replaces pca_group.py:45-49, 58-61 (no argsort needed)
 */
int mcs_perm_apply(const void* x, void* out, const int64_t* perm, int32_t BH, int32_t L, int32_t row_bytes,
                   int64_t x_bh_bytes, int64_t x_row_bytes, int64_t o_bh_bytes, int64_t o_row_bytes, void* stream);
int mcs_perm_invert(const void* x, void* out, const int64_t* perm, int32_t BH, int32_t L, int32_t row_bytes,
                    int64_t x_bh_bytes, int64_t x_row_bytes, int64_t o_bh_bytes, int64_t o_row_bytes, void* stream);

/*
 * Gather-rate probe (no reference counterpart; measurement aid).  Takes the argument block of
 * mcs_gather_attn_fwd (int32 index list, head dimension 64 or 128) and launches only the K/V row gather of
 * that call: same grid, same walk over the query groups, same four copying warps per CTA and the same 16-byte
 * copies into swizzled shared-memory tiles, which nothing reads.  Its duration is the time the selected rows of
 * one attention launch need to come out of L2 when no other role of the kernel competes - a floor for the
 * attention launch that its softmax and tensor-core schedule cannot lower.  q, out, residual are not touched.
 */
int mcs_gather_rate_probe(const mcs_gather_attn_args* a, void* stream);

/*
 * SM clock probe (no reference counterpart; measurement aid).  Launches one CTA that spins for about
 * 40,000 SM cycles and writes {SM cycles, nanoseconds} it observed to out2[0..1] (device memory, two
 * int64): cycles * 1000 / nanoseconds is the SM clock in MHz at that moment.  Launched right behind a
 * timed region on the same stream it reports the clock the GPU was running at under that load, which
 * a 100 ms nvidia-smi poll cannot resolve for regions of a few milliseconds.
 */
int mcs_sm_clock_probe(int64_t* out2, void* stream);

/*
 * Clock telemetry of the attention kernel (no reference counterpart; measurement aid).  After this call
 * every attention launch of this process writes {SM cycles, nanoseconds, KV tiles} of its first CTA's tile
 * loop to buf3[0..2] (device memory, three int64; pass NULL to switch it off): cycles * 1000 / nanoseconds
 * is the SM clock in MHz under the kernel's own load.  Process-wide and not thread-safe, like the
 * reference's module-global statistics.
 */
void mcs_set_clock_buffer(int64_t* buf3);

#ifdef __cplusplus
}
#endif
#endif /* MCSPARSE_B200_H_ */
