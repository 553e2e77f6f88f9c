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
  int32_t B, Sq, Sk, H, D;
  int32_t gather_len;   /* multiple of 128 */
  int32_t group_rows;   /* query rows per group, 1..128 (reference: 128) */
  int32_t dtype;        /* MCS_DTYPE_* */
  float softmax_scale;  /* > 0; ignored for e4m3 (scale_qk_log2 carries it) */
} mcs_gather_attn_args;

int mcs_gather_attn_fwd(const mcs_gather_attn_args* args, void* stream);

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
  int32_t B, H, Lq, Lk, D;
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

#ifdef __cplusplus
}
#endif
#endif /* MCSPARSE_B200_H_ */
