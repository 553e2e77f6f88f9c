"""Anchor-step token scoring and selection, and the host-side state of token-sparse attention.

Host mirror of the parts of the reference's ``mcsparse/kernels/flash_mcsa/token_sparse.py``
that sit on the accelerated path; the compute runs in the CUDA library through the C ABI.

* ``group_mass`` / ``_compute_token_probs``: token_sparse.py:590-595 -> block_probs.py:92-117
* ``select_topk_with_sinks`` / ``_select_topk_tokens``: token_sparse.py:755-945 (topk mode)
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from mcsparse_b200 import _lib


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.MCS_DTYPE_BF16
    if t.dtype == torch.float16:
        return _lib.MCS_DTYPE_FP16
    raise TypeError(f"q/k must be bf16 or fp16, got {t.dtype}")


def group_mass(q: torch.Tensor, k: torch.Tensor, lse: torch.Tensor, group_rows: int = 128,
               scale: Optional[float] = None, perm: Optional[torch.Tensor] = None,
               normalize: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 attention mass of every query group on every key token.

    ``mass[b,h,m,j] = sum_{i in group m} exp(scale * q_i . k_j - lse_i)`` (divided by the number of
    rows in the group if ``normalize``).  q: (B,H,Lq,D), k: (B,H,Lk,D) bf16/fp16 with contiguous
    rows; lse: (B,H,Lq) fp32, natural log, scale included, indexed by position in the query order
    given by ``perm`` ((B*H, Lq) int64, identity if None).  Returns (B,H,M,Lk) fp32.
    """
    if q.ndim != 4 or k.ndim != 4:
        raise ValueError("q and k must be (B, H, L, D)")
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    if k.shape[0] != B or k.shape[1] != H or k.shape[3] != D:
        raise ValueError("q and k must agree in batch, heads and head_dim")
    if not (q.is_cuda and k.is_cuda and lse.is_cuda):
        raise RuntimeError("q, k and lse must be CUDA tensors")
    if q.dtype != k.dtype:
        raise TypeError("q and k must have the same dtype")
    if tuple(lse.shape) != (B, H, Lq):
        raise ValueError(f"lse must have shape {(B, H, Lq)}, got {tuple(lse.shape)}")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    q = q if q.stride(-1) == 1 else q.contiguous()
    k = k if k.stride(-1) == 1 else k.contiguous()
    lse = lse.to(torch.float32).contiguous()
    M = math.ceil(Lq / group_rows)
    if out is None:
        out = torch.empty(B, H, M, Lk, dtype=torch.float32, device=q.device)
    elif tuple(out.shape) != (B, H, M, Lk) or out.dtype != torch.float32 or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous fp32 tensor of shape {(B, H, M, Lk)}")
    if perm is not None:
        if perm.dtype != torch.int64 or tuple(perm.shape) != (B * H, Lq):
            raise ValueError(f"perm must be int64 of shape {(B * H, Lq)}")
        perm = perm.contiguous()
    a = _lib.GroupMassArgs()
    a.q, a.k, a.lse, a.mass = q.data_ptr(), k.data_ptr(), lse.data_ptr(), out.data_ptr()
    a.perm = None if perm is None else perm.data_ptr()
    a.status = _lib.status_word(q.device).data_ptr()
    # C ABI stride order is (batch, sequence, head); the tensors here are (B, H, L, D)
    a.q_stride[0], a.q_stride[1], a.q_stride[2] = q.stride(0), q.stride(2), q.stride(1)
    a.k_stride[0], a.k_stride[1], a.k_stride[2] = k.stride(0), k.stride(2), k.stride(1)
    a.B, a.H, a.Lq, a.Lk, a.D = B, H, Lq, Lk, D
    a.group_rows, a.dtype, a.normalize = int(group_rows), _dtype_code(q), int(bool(normalize))
    a.softmax_scale = float(scale)
    _lib.launch("mcs_group_mass", a, q.device, "group_mass")
    return out


def _compute_token_probs(q, k, lse, BLKQ, scale):
    """Reference-compatible wrapper (token_sparse.py:590-595): mean over the block's rows, in q.dtype."""
    return group_mass(q, k, lse, group_rows=BLKQ, scale=scale, normalize=True).to(q.dtype)


def _sink_indices(sink_ranges, L_K: int):
    """Sorted distinct key positions covered by half-open ``sink_ranges`` (token_sparse.py:788-798)."""
    idx = set()
    for start, end in (sink_ranges or []):
        idx.update(range(max(0, int(start)), min(int(end), L_K)))
    return sorted(idx)


def select_topk_with_sinks(scores: torch.Tensor, k_total: int, sink_ranges=None,
                           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact selection: the sink tokens plus the ``k_total - n_sink`` highest-scoring other tokens.

    scores: (..., L) fp32 CUDA tensor (one row per query group).  Ties go to the lowest index and the
    result is ascending int32 of shape (..., k_total): a pure function of the fp32 scores.
    """
    if scores.dtype != torch.float32:
        raise TypeError("scores must be float32 (rank on the fp32 mass, not on a rounded copy)")
    if not scores.is_cuda:
        raise RuntimeError("scores must be a CUDA tensor")
    L = scores.shape[-1]
    sinks = _sink_indices(sink_ranges, L)
    if len(sinks) > 64:
        raise ValueError("at most 64 sink tokens are supported")
    if not (len(sinks) <= k_total <= L):
        raise ValueError(f"k_total must be in [n_sink={len(sinks)}, L={L}], got {k_total}")
    scores = scores.contiguous()
    rows = scores.numel() // L
    shape = tuple(scores.shape[:-1]) + (k_total,)
    if out is None:
        out = torch.empty(shape, dtype=torch.int32, device=scores.device)
    elif tuple(out.shape) != shape or out.dtype != torch.int32 or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous int32 tensor of shape {shape}")
    sink_t = torch.tensor(sinks, dtype=torch.int32, device=scores.device) if sinks else None
    stream = torch.cuda.current_stream(scores.device).cuda_stream
    rc = _lib.lib().mcs_topk_select(scores.data_ptr(), out.data_ptr(),
                                    None if sink_t is None else sink_t.data_ptr(), len(sinks), rows, L,
                                    int(k_total), stream)
    if rc != 0:
        raise RuntimeError(f"select_topk_with_sinks: {_lib.error_string(rc)} (code {rc})")
    if _lib.check_enabled():
        _lib.check_status(scores.device, "select_topk_with_sinks")
    return out


def _select_topk_tokens(token_probs, topk_ratio, tile_n=128, ds_k=1, orig_L_K=None,
                        selection_mode='topk', topp=None, sink_ranges=None):
    """Reference-shaped selection (token_sparse.py:755-945), ``topk`` mode, scalar ratio, ds_k == 1.

    Budget arithmetic as in the reference: ``k_sel = min(L_K, align_up(max(1, int(ratio * L_K)), tile_n))``;
    with sinks the list ``[sinks, top-k_sel]`` is cut to a whole number of tiles and tile counts are
    returned, without sinks the counts are None.  Where the reference drops an arbitrary subset of an
    unsorted top-k, this drops the lowest-ranked entries, and indices come back ascending.
    Returns ``(gather_indices (B,H,M,gather_len) int32, gather_kv_lengths (B,H,M) int32 | None)``.
    """
    if selection_mode != 'topk':
        raise NotImplementedError(f"selection_mode={selection_mode!r}: only 'topk' runs on this path")
    if ds_k != 1:
        raise NotImplementedError("key downsampling (ds_k > 1) is not part of this path")
    if isinstance(topk_ratio, torch.Tensor):
        raise NotImplementedError("adaptive per-head budgets are not part of this path")
    B, H, M, L_K = token_probs.shape
    n = max(1, int(topk_ratio * L_K))
    k_sel = min(((n + tile_n - 1) // tile_n) * tile_n, L_K)
    sinks = _sink_indices(sink_ranges, L_K)
    scores = token_probs.float()
    if not sinks:
        gl = k_sel if k_sel % tile_n == 0 else max(tile_n, (k_sel // tile_n) * tile_n)
        return select_topk_with_sinks(scores, min(gl, L_K)), None
    total = k_sel + len(sinks)
    cap = max(tile_n, min(((L_K + tile_n - 1) // tile_n) * tile_n, (total // tile_n) * tile_n))
    count = min(max(min(((total + tile_n - 1) // tile_n) * tile_n, total), tile_n), cap)
    count = min(count, L_K)
    gi = select_topk_with_sinks(scores, count, sink_ranges)
    lengths = torch.full((B, H, M), count // tile_n, dtype=torch.int32, device=token_probs.device)
    return gi, lengths


# =============================================================================================
# Host-side state of token-sparse attention: configuration, per-layer cache, step modes.
# Mirrors TokenSparseConfig (token_sparse.py:104-198), TokenSparseCache (:200-547, mode :233-247),
# TokenSparseBackend (:1013-1459) and TokenSparseContext (:1461-1845) for the options that lie on
# the accelerated path.  What the reference implements with a chain of torch ops and copies is one
# kernel call here: Q is read through the permutation, the residual is added in the epilogue and
# the output is written back in the original order.
# =============================================================================================
from dataclasses import dataclass, field
from typing import List, Tuple, Union


@dataclass
class TokenSparseConfig:
    """Token-level sparse attention settings (same names and defaults as the reference's)."""
    topk: float = 0.1
    topp: Optional[float] = None
    selection_mode: str = 'topk'
    BLKQ: int = 128
    tile_n: int = 128
    sink_ranges: Optional[List[Tuple[int, int]]] = None
    calibrate_steps: Optional[List[int]] = None
    update_steps: Optional[List[int]] = None
    full_steps: Optional[List[int]] = None
    full_layers: List[int] = field(default_factory=list)
    share_lse: bool = False
    cal_downsample: Union[int, Tuple[int, int]] = 1
    bias_correction: bool = False
    pca_reorder: bool = False
    pca_pow_iters: int = 4
    pca_seed: int = 0

    def __post_init__(self):
        assert 0 < self.topk <= 1.0
        assert self.selection_mode in ('topk', 'topp', 'topk_topp'), \
            f"selection_mode must be 'topk', 'topp', or 'topk_topp', got '{self.selection_mode}'"
        if self.selection_mode != 'topk':
            raise NotImplementedError("only selection_mode='topk' runs on the accelerated path")
        assert self.BLKQ == 128
        assert self.tile_n == 128
        if isinstance(self.cal_downsample, (list, tuple)):
            ds = (int(self.cal_downsample[0]), int(self.cal_downsample[1]))
        else:
            ds = (int(self.cal_downsample),) * 2
        if ds != (1, 1):
            raise NotImplementedError("cal_downsample > 1 is not part of the accelerated path")
        self._cal_ds_q, self._cal_ds_k = ds
        self._calibrate_set = set(self.calibrate_steps) if self.calibrate_steps else None
        self._update_set = set(self.update_steps) if self.update_steps else None
        self._full_set = set(self.full_steps) if self.full_steps else None
        if self.sink_ranges:
            for start, end in self.sink_ranges:
                assert 0 <= start < end, f"Invalid sink_ranges interval: ({start}, {end})"
        if self.pca_reorder:
            assert not self.share_lse, "pca_reorder is incompatible with share_lse"


class TokenSparseCache:
    """Per-layer state carried between denoising steps: permutation, indices, LSE, residual."""

    def __init__(self, config: TokenSparseConfig):
        self.config = config
        self._step_count = 0
        self._cached_lse = None
        self._cached_indices = None
        self._cached_lengths = None
        self._cached_perm = None
        self._cached_residual = None
        self._perm_generation = 0          # advances on every permutation refresh
        self._residual_perm_gen = None     # generation the residual was computed under
        self._cached_len = None

    @property
    def has_cache(self) -> bool:
        return self._cached_indices is not None

    @property
    def mode(self) -> str:
        """Mode of the current step (token_sparse.py:233-247)."""
        s, c = self._step_count, self.config
        if c._full_set and s in c._full_set:
            if c._calibrate_set and s in c._calibrate_set:
                return 'full_calibrate'
            return 'full'
        if c._calibrate_set and s in c._calibrate_set:
            return 'calibrate'
        if c._update_set and s in c._update_set:
            return 'update'
        if not self.has_cache:
            return 'calibrate'
        return 'reuse'

    def step(self) -> None:
        self._step_count += 1

    def reset(self) -> None:
        self.__init__(self.config)

    def residual_if_valid(self):
        """The cached residual, unless it belongs to an older permutation (token_sparse.py:505-521)."""
        if self._cached_residual is None:
            return None
        if self.config.pca_reorder and self._residual_perm_gen != self._perm_generation:
            self._cached_residual = None
            return None
        return self._cached_residual


def dense_attention_with_lse(q, k, v, scale):
    """Dense attention output and natural-log LSE on (B,H,L,D) tensors: the input of the anchor step.

    The reference calls FA3 here (ops/full_attn.py:88-121); this is the package's own attention kernel in
    dense mode, on strided views of the (B,H,L,D) tensors (no layout copies).
    """
    from mcsparse_b200.kernels.flash_mcsa.ops.full_attn import full_attention_with_lse
    return full_attention_with_lse(q, k, v, scale)


class TokenSparseBackend:
    """One attention call of one layer, on (B, H, L, D) tensors, by the mode of the layer's cache."""

    def __init__(self, config: TokenSparseConfig):
        self.config = config

    def _sparse(self, q, k, v, gi, gl, scale, residual, perm, subtract: bool = False):
        from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute.interface import flash_attn_gather_kv_func
        # (B,H,L,D) storage viewed as (B,L,H,D): no copies, the kernel takes the strides
        out = torch.empty_like(q)
        flash_attn_gather_kv_func(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gi, softmax_scale=scale,
                                  gather_kv_lengths=gl, out=out.transpose(1, 2), residual=residual, perm=perm,
                                  residual_minus_attention=subtract)
        return out

    def forward(self, cache: TokenSparseCache, q, k, v, scale: Optional[float] = None):
        from mcsparse_b200.kernels.flash_mcsa.pca_group import apply_perm_bhld, pca_group_perm
        cfg = self.config
        B, H, L, D = q.shape
        if scale is None:
            scale = 1.0 / math.sqrt(D)
        if cache._cached_len is not None and cache._cached_len != (L, k.shape[2]):
            cache.reset()                                           # length change forces a new anchor step
        mode = cache.mode
        if mode == 'full':
            return dense_attention_with_lse(q, k, v, scale)[0]
        if mode in ('calibrate', 'full_calibrate'):
            perm = None
            if cfg.pca_reorder:
                perm = pca_group_perm(q.reshape(B * H, L, D), C=cfg.BLKQ, pow_iters=cfg.pca_pow_iters, seed=cfg.pca_seed)
                cache._perm_generation += 1
            cache._cached_perm = perm
            q_grp = q if perm is None else apply_perm_bhld(q, perm)
            dense_grp, lse = dense_attention_with_lse(q_grp, k, v, scale)        # group (permuted) order
            cache._cached_lse = lse
            mass = group_mass(q_grp, k, lse, group_rows=cfg.BLKQ, scale=scale)
            gi, gl = _select_topk_tokens(mass, cfg.topk, tile_n=cfg.tile_n, sink_ranges=cfg.sink_ranges)
            cache._cached_indices, cache._cached_lengths, cache._cached_len = gi, gl, (L, k.shape[2])
            if cfg.bias_correction:
                # residual = dense - sparse in one kernel pass (the reference runs the sparse kernel and then an
                # elementwise subtraction, token_sparse.py:1209-1216); permuted-query order
                cache._cached_residual = self._sparse(q_grp, k, v, gi, gl, scale, dense_grp, None, subtract=True)
                cache._residual_perm_gen = cache._perm_generation
            if perm is None:
                return dense_grp
            from mcsparse_b200.kernels.flash_mcsa.pca_group import invert_perm_bhld
            return invert_perm_bhld(dense_grp, perm)
        if mode == 'update':
            perm = cache._cached_perm
            q_grp = q if perm is None else apply_perm_bhld(q, perm)
            mass = group_mass(q_grp, k, cache._cached_lse, group_rows=cfg.BLKQ, scale=scale)
            cache._cached_indices, cache._cached_lengths = _select_topk_tokens(
                mass, cfg.topk, tile_n=cfg.tile_n, sink_ranges=cfg.sink_ranges)
        # reuse (and the attention of an update step): one fused kernel call
        residual = cache.residual_if_valid() if cfg.bias_correction else None
        return self._sparse(q, k, v, cache._cached_indices, cache._cached_lengths, scale, residual, cache._cached_perm)


class TokenSparseContext:
    """All layers of a model: one cache per layer, one step clock (token_sparse.py:1461-1845)."""

    def __init__(self, config: TokenSparseConfig, num_layers: int):
        self.config = config
        self.backend = TokenSparseBackend(config)
        self.caches = [TokenSparseCache(config) for _ in range(num_layers)]

    def forward(self, li: int, q, k, v, scale: Optional[float] = None):
        if li in self.config.full_layers:
            return dense_attention_with_lse(q, k, v, scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))[0]
        return self.backend.forward(self.caches[li], q, k, v, scale)

    def step(self) -> None:
        for c in self.caches:
            c.step()

    def reset(self) -> None:
        for c in self.caches:
            c.reset()
