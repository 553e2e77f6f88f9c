"""Anchor-step token scoring and selection, and the host-side state of token-sparse attention.

Host mirror of the parts of the reference's ``mcsparse/kernels/flash_mcsa/token_sparse.py``
that sit on the accelerated path; the compute runs in the CUDA library through the C ABI.

* ``group_mass`` / ``_compute_token_probs``: token_sparse.py:590-595 -> block_probs.py:92-117
* ``select_topk_with_sinks`` / ``_select_topk_tokens``: token_sparse.py:755-945 (topk mode)
"""

from __future__ import annotations

import contextlib
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
    _lib.raise_on_error(rc, f"select_topk_with_sinks")
    if _lib.check_enabled():
        _lib.check_status(scores.device, "select_topk_with_sinks")
    return out


def topp_count(scores: torch.Tensor, topp: float, sink_ranges=None) -> torch.Tensor:
    """Per row of normalised fp32 masses (..., L): how many tokens, taken in descending order of mass, are needed
    before the mass in front of the next one reaches ``topp`` (at least 1; sinks are not ranked or counted).
    Returns int32 (...)."""
    if scores.dtype != torch.float32 or not scores.is_cuda:
        raise TypeError("scores must be a float32 CUDA tensor")
    L = scores.shape[-1]
    sinks = _sink_indices(sink_ranges, L)
    if len(sinks) > 64:
        raise ValueError("at most 64 sink tokens are supported")
    scores = scores.contiguous()
    rows = scores.numel() // L
    out = torch.empty(scores.shape[:-1], dtype=torch.int32, device=scores.device)
    sink_t = torch.tensor(sinks, dtype=torch.int32, device=scores.device) if sinks else None
    stream = torch.cuda.current_stream(scores.device).cuda_stream
    rc = _lib.lib().mcs_topp_count(scores.data_ptr(), None if sink_t is None else sink_t.data_ptr(), len(sinks), rows, L,
                                   float(topp), out.data_ptr(), stream)
    _lib.raise_on_error(rc, "topp_count")
    if _lib.check_enabled():
        _lib.check_status(scores.device, "topp_count")
    return out


def select_topk_var(scores: torch.Tensor, k_rows: torch.Tensor, k_max: int, sink_ranges=None) -> torch.Tensor:
    """Selection with a budget per row: row r gets the sinks plus its ``k_rows[r] - n_sink`` best other tokens,
    ascending, padded with zeros to ``k_max``.  scores (..., L) fp32, k_rows (...) int32.  Returns (..., k_max) int32."""
    if scores.dtype != torch.float32 or not scores.is_cuda:
        raise TypeError("scores must be a float32 CUDA tensor")
    L = scores.shape[-1]
    sinks = _sink_indices(sink_ranges, L)
    if len(sinks) > 64:
        raise ValueError("at most 64 sink tokens are supported")
    if tuple(k_rows.shape) != tuple(scores.shape[:-1]):
        raise ValueError("one budget per score row")
    if not (len(sinks) <= k_max <= L):
        raise ValueError(f"k_max must be in [n_sink={len(sinks)}, L={L}], got {k_max}")
    scores = scores.contiguous()
    k_rows = k_rows.to(torch.int32).contiguous()
    rows = scores.numel() // L
    out = torch.empty(tuple(scores.shape[:-1]) + (k_max,), dtype=torch.int32, device=scores.device)
    sink_t = torch.tensor(sinks, dtype=torch.int32, device=scores.device) if sinks else None
    stream = torch.cuda.current_stream(scores.device).cuda_stream
    rc = _lib.lib().mcs_topk_select_var(scores.data_ptr(), out.data_ptr(), None if sink_t is None else sink_t.data_ptr(),
                                        len(sinks), rows, L, int(k_max), k_rows.data_ptr(), stream)
    _lib.raise_on_error(rc, "select_topk_var")
    if _lib.check_enabled():
        _lib.check_status(scores.device, "select_topk_var")
    return out


def selection_counts(L_K: int, n_sink: int, tile_n: int, base_counts: torch.Tensor) -> torch.Tensor:
    """Budget arithmetic of the variable-length modes (token_sparse.py:811-823, :902-923): the per-row number of
    ranked tokens is rounded up to whole tiles (never beyond L_K), the sinks are added, the total is rounded up to whole
    tiles again as long as ranked tokens are left to fill it, else down, and it is at least one tile."""
    c = base_counts.long().clamp(min=1)
    c = (((c + tile_n - 1) // tile_n) * tile_n).clamp(max=L_K)
    avail = int(c.max().item()) + n_sink                      # length of [sinks, ranked prefix] in the reference
    if n_sink:
        c = (((c + n_sink + tile_n - 1) // tile_n) * tile_n).clamp(max=avail)
    cap = max(tile_n, min(((L_K + tile_n - 1) // tile_n) * tile_n, (avail // tile_n) * tile_n))
    c = c.clamp(min=tile_n, max=cap)
    return ((c // tile_n) * tile_n).clamp(max=L_K)


def _select_topk_tokens(token_probs, topk_ratio, tile_n=128, ds_k=1, orig_L_K=None,
                        selection_mode='topk', topp=None, sink_ranges=None):
    """Reference-shaped selection (token_sparse.py:755-945), ds_k == 1.

    ``topk`` with a scalar ratio: ``k_sel = min(L_K, align_up(max(1, int(ratio * L_K)), tile_n))``; with sinks the list
    ``[sinks, top-k_sel]`` is cut to a whole number of tiles and tile counts are returned, without sinks the counts are
    None.  ``topk`` with a (B, H) ratio tensor (adaptive heads), ``topp`` (shortest prefix of the descending order
    that reaches mass ``topp``) and ``topk_topp`` (the same with the top-k budget as lower bound) give every row its
    own budget: rounded up to whole tiles with real tokens, tile counts returned, rows padded with zeros beyond them.
    Where the reference keeps an arbitrary subset of an unsorted top-k or a descending prefix, this keeps the
    best-ranked tokens (ties to the lowest index) and returns them ascending.
    Returns ``(gather_indices (B,H,M,gather_len) int32, gather_kv_lengths (B,H,M) int32 | None)``.
    """
    if selection_mode not in ('topk', 'topp', 'topk_topp'):
        raise ValueError(f"Unknown selection_mode: {selection_mode}")
    if ds_k != 1:
        raise NotImplementedError("key downsampling (ds_k > 1) is not part of this path")
    B, H, M, L_K = token_probs.shape
    sinks = _sink_indices(sink_ranges, L_K)
    scores = token_probs.float()
    adaptive = isinstance(topk_ratio, torch.Tensor)
    if selection_mode == 'topk' and not adaptive:
        n = max(1, int(topk_ratio * L_K))
        k_sel = min(((n + tile_n - 1) // tile_n) * tile_n, L_K)
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
    # ---- every row with a budget of its own
    if selection_mode == 'topk':
        base = (topk_ratio.to(scores.device).float() * L_K).long().view(B, H, 1).expand(B, H, M)
    else:
        if topp is None:
            raise AssertionError(f"{selection_mode} mode requires topp")
        base = topp_count(scores, topp, sink_ranges).long()
        if selection_mode == 'topk_topp':
            if adaptive:
                floor_k = (topk_ratio.to(scores.device).float() * L_K).clamp(min=1, max=L_K).long().view(B, H, 1).expand(B, H, M)
            else:
                floor_k = torch.full_like(base, min(max(1, int(topk_ratio * L_K)), L_K))
            base = torch.maximum(base, floor_k)
    counts = selection_counts(L_K, len(sinks), tile_n, base)
    k_max = int(counts.max().item())
    gi = select_topk_var(scores, counts.to(torch.int32), k_max, sink_ranges)
    return gi, (counts // tile_n).to(torch.int32).contiguous()


def _compute_adaptive_topk_token(token_probs, base_topk, layer_t=None):
    """Per-head budgets from the retained mass (token_sparse.py:695-738): heads whose top-k already holds more of
    the mass get less budget.  Returns (B, H) fractions."""
    B, H, M, L_K = token_probs.shape
    k = min(max(1, int(base_topk * L_K)), L_K)
    scores = token_probs.float()
    gi = select_topk_with_sinks(scores, k)                                   # (B,H,M,k) ascending indices
    kept = scores.gather(-1, gi.long()).sum(-1)
    recall = (kept / scores.sum(-1).clamp(min=1e-8)).mean(-1)                # (B, H)
    order = recall.argsort(dim=-1)
    ranks = torch.zeros_like(order)
    ranks.scatter_(-1, order, torch.arange(H, device=scores.device).expand(B, H))
    t = ranks.float() / max(H - 1, 1)
    per_head = base_topk * ((1.0 + 0.5 * layer_t - 0.5 * t) if layer_t is not None else (1.5 - t))
    return per_head.clamp(min=1.0 / L_K, max=1.0)


def _chunked_online_topk(q, k, lse, BLKQ, scale, topk_k, tile_n=128, chunk_size=None, perm=None):
    """Selection without the full (B,H,M,L_K) score tensor in memory (token_sparse.py:602-687).

    The reference walks the keys in chunks and keeps a running top-k of bf16-rounded scores.  Here the
    mass kernel writes fp32 scores for a few heads at a time (the bound on memory is the same idea,
    cut along heads instead of keys: at most about ``chunk_size * 2^16`` scores at once) and the exact selection
    kernel picks the top ``topk_k`` of each row, ascending.  Returns (B,H,M,topk_k) int32."""
    B, H, Lq, D = q.shape
    L_K = k.shape[2]
    M = math.ceil(Lq / BLKQ)
    k_sel = min(((topk_k + tile_n - 1) // tile_n) * tile_n, L_K)
    budget = int(chunk_size or 16384) << 16
    hc = max(1, min(H, budget // max(1, M * L_K)))
    gi = torch.empty(B, H, M, k_sel, dtype=torch.int32, device=q.device)
    for h0 in range(0, H, hc):
        h1 = min(H, h0 + hc)
        pm = None if perm is None else perm.view(B, H, Lq)[:, h0:h1].reshape(-1, Lq)
        mass = group_mass(q[:, h0:h1], k[:, h0:h1], lse[:, h0:h1], group_rows=BLKQ, scale=scale, perm=pm)
        gi[:, h0:h1] = select_topk_with_sinks(mass, k_sel)
        del mass
    return gi


def _approx_select(q, k, cfg, perm=None):
    """Selection of an ``approx`` step (token_sparse.py:1344-1406): score every key against the mean query of
    each group (no LSE needed), keep the top budget, ascending.  The (M x D) x (D x L_K) product per head is a
    plain library GEMM; the selection is this package's kernel on the fp32 scores."""
    from mcsparse_b200.kernels.flash_mcsa.pca_group import apply_perm_bhld
    B, H, L, D = q.shape
    L_K = k.shape[2]
    M = math.ceil(L / cfg.BLKQ)
    q_grp = q if perm is None else apply_perm_bhld(q, perm)
    if M * cfg.BLKQ > L:
        q_grp = torch.nn.functional.pad(q_grp, (0, 0, 0, M * cfg.BLKQ - L))
    q_mean = q_grp.reshape(B, H, M, cfg.BLKQ, D).float().mean(dim=3).to(q.dtype)
    n = max(1, int(cfg.topk * L_K))
    k_sel = min(((n + cfg.tile_n - 1) // cfg.tile_n) * cfg.tile_n, L_K)
    gi = torch.empty(B, H, M, k_sel, dtype=torch.int32, device=q.device)
    for h in range(H):                                   # one head at a time bounds the score tensor
        scores = torch.matmul(q_mean[:, h], k[:, h].transpose(-1, -2)).float()
        gi[:, h] = select_topk_with_sinks(scores.contiguous(), k_sel)
    return gi


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
    adaptive_heads: bool = False
    adaptive_layers: bool = False
    use_chunk_selector: bool = False
    chunk_selector_size: int = 16384
    offload_indices: bool = False          # keep the indices in pinned host memory between uses
    approx_steps: Optional[List[int]] = None
    bias_correction: bool = False
    cache_offload: str = 'none'            # 'residual': the same for the bias-correction residual
    full_attn_impl: str = 'sdpa'           # accepted for call compatibility: there is one dense implementation here
    pca_reorder: bool = False
    pca_pow_iters: int = 4
    pca_proj_dim: Optional[int] = None
    pca_whiten: bool = False
    # additions of this package (after the reference's fields, so positional construction keeps its meaning)
    pca_seed: int = 0
    offload_prefetch_ahead: int = 1        # layers ahead of its use at which an offloaded tensor starts to come back
    compact_indices: bool = False          # keep the cached indices in the packed 17-bit form (sequences up to 131,072 keys)

    def __post_init__(self):
        assert 0 < self.topk <= 1.0
        assert self.selection_mode in ('topk', 'topp', 'topk_topp'), \
            f"selection_mode must be 'topk', 'topp', or 'topk_topp', got '{self.selection_mode}'"
        if self.selection_mode in ('topp', 'topk_topp'):
            assert self.topp is not None and 0 < self.topp <= 1.0, f"selection_mode='{self.selection_mode}' requires topp"
        assert self.BLKQ == 128
        assert self.tile_n == 128
        if isinstance(self.cal_downsample, (list, tuple)):
            ds = (int(self.cal_downsample[0]), int(self.cal_downsample[1]))
        else:
            ds = (int(self.cal_downsample),) * 2
        if ds != (1, 1):
            raise NotImplementedError("cal_downsample > 1 is not part of the accelerated path")
        if self.pca_proj_dim is not None or self.pca_whiten:
            raise NotImplementedError("pca_proj_dim / pca_whiten are not part of the accelerated path")
        self._cal_ds_q, self._cal_ds_k = ds
        self._calibrate_set = set(self.calibrate_steps) if self.calibrate_steps else None
        self._update_set = set(self.update_steps) if self.update_steps else None
        self._approx_set = set(self.approx_steps) if self.approx_steps else None
        self._full_set = set(self.full_steps) if self.full_steps else None
        if self.sink_ranges:
            for start, end in self.sink_ranges:
                assert 0 <= start < end, f"Invalid sink_ranges interval: ({start}, {end})"
        if self.pca_reorder:
            assert not self.share_lse, "pca_reorder is incompatible with share_lse"
        assert self.chunk_selector_size > 0 and self.chunk_selector_size % self.tile_n == 0
        assert self.cache_offload in ('none', 'residual'), f"cache_offload must be 'none' or 'residual', got {self.cache_offload!r}"
        assert self.offload_prefetch_ahead in (0, 1), "offload_prefetch_ahead only supports 0 or 1"
        if self.cache_offload == 'residual':
            assert self.bias_correction, "cache_offload='residual' requires bias_correction=True"
        assert not (self.compact_indices and self.offload_indices), "compact_indices keeps the indices in HBM; choose one of the two"
        if self.share_lse:
            raise NotImplementedError("share_lse (one layer's LSE reused by the others) is not part of the accelerated path: "
                                      "every layer computes its own")


# modes in which the permutation is renewed together with the selection (token_sparse.py:984); an update
# step keeps it because the cached per-query LSE is in the order of the anchor step
_SELECTION_RECOMPUTE_MODES = ('calibrate', 'full_calibrate', 'approx')


class TokenSparseCache:
    """Per-layer state carried between denoising steps: permutation, indices, LSE, residual."""

    def __init__(self, config: TokenSparseConfig, layer_idx: int = 0, layer_t: Optional[float] = None):
        self.config = config
        self._layer_idx = layer_idx
        self.layer_t = layer_t             # normalised depth in [0, 1] for adaptive_layers, else None
        self._step_count = 0
        self._cached_lse = None
        # indices, tile counts and residual live in slots that can park them in pinned host memory (residency.py)
        from mcsparse_b200.kernels.flash_mcsa.residency import OffloadSlot
        old = getattr(self, "_slots", None)
        if old is not None:
            for sl in old:
                sl.clear()
        self._idx, self._len, self._res = old if old is not None else (OffloadSlot(), OffloadSlot(), OffloadSlot())
        self._slots = (self._idx, self._len, self._res)
        self._cached_perm = None
        self._perm_generation = 0          # advances on every permutation refresh
        self._residual_perm_gen = None     # generation the residual was computed under
        self._cached_len = None

    # the three cached tensors as plain attributes: reading one makes it available on the current stream
    @property
    def _cached_indices(self):
        return self._idx.get()

    @_cached_indices.setter
    def _cached_indices(self, t):
        if self.config.compact_indices and isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.int32 \
                and self._cached_len is not None and self._cached_len[1] <= (1 << 17):
            from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute.interface import PackedIndices
            t = PackedIndices.pack(t)              # 272 instead of 512 bytes per tile; the attention kernel reads it as it is
        self._idx.store(t, offload=self.config.offload_indices)

    @property
    def _cached_lengths(self):
        return self._len.get()

    @_cached_lengths.setter
    def _cached_lengths(self, t):
        self._len.store(t, offload=self.config.offload_indices)

    @property
    def _cached_residual(self):
        return self._res.get()

    @_cached_residual.setter
    def _cached_residual(self, t):
        self._res.store(t, offload=self.config.cache_offload == 'residual')

    @property
    def has_cache(self) -> bool:
        return self._idx.present

    def prefetch(self) -> None:
        """Start bringing offloaded tensors back if the coming use is a reuse step (token_sparse.py:340-361, :425-452)."""
        if self.mode != 'reuse':
            return
        self._idx.prefetch()
        self._len.prefetch()
        if self.config.bias_correction and self._residual_perm_gen == self._perm_generation:
            self._res.prefetch()

    def offload_stats(self) -> dict:
        return {"idx_prefetch_hit": self._idx.hits, "idx_prefetch_miss": self._idx.misses,
                "res_prefetch_hit": self._res.hits, "res_prefetch_miss": self._res.misses}

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
        if c._approx_set and s in c._approx_set:
            return 'approx'
        if c._update_set and s in c._update_set:
            return 'update'
        if not self.has_cache:
            return 'calibrate'
        return 'reuse'

    def step(self) -> None:
        self._step_count += 1

    def reset(self) -> None:
        self.__init__(self.config, self._layer_idx, self.layer_t)

    def residual_if_valid(self):
        """The cached residual, unless it belongs to an older permutation (token_sparse.py:505-521)."""
        if not self._res.present:
            return None
        if self.config.pca_reorder and self._residual_perm_gen != self._perm_generation:
            self._cached_residual = None
            return None
        return self._cached_residual


def dense_attention_with_lse(q, k, v, scale, perm=None, group_order: bool = False):
    """Dense attention output and natural-log LSE on (B,H,L,D) tensors: the input of the anchor step.

    The reference calls FA3 here (ops/full_attn.py:88-121); this is the package's own attention kernel in
    dense mode, on strided views of the (B,H,L,D) tensors (no layout copies).  With ``perm`` and
    ``group_order`` the queries are read through the permutation and output and LSE come back in the
    permuted (group) order, which replaces the gathered copy of Q in front of the dense pass.
    """
    from mcsparse_b200.kernels.flash_mcsa.ops.full_attn import full_attention_with_lse
    return full_attention_with_lse(q, k, v, scale, perm=perm, group_order=group_order)


class TokenSparseBackend:
    """One attention call of one layer, on (B, H, L, D) tensors, by the mode of the layer's cache."""

    def __init__(self, config: TokenSparseConfig):
        self.config = config

    def _sparse(self, q, k, v, gi, gl, scale, residual, perm, subtract: bool = False, out_peers=None,
                group_order: bool = False):
        from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute.interface import flash_attn_gather_kv_func
        # (B,H,L,D) storage viewed as (B,L,H,D): no copies, the kernel takes the strides
        out = None if out_peers is not None else torch.empty_like(q)
        flash_attn_gather_kv_func(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gi, softmax_scale=scale,
                                  gather_kv_lengths=gl, out=None if out is None else out.transpose(1, 2),
                                  residual=residual, perm=perm, residual_minus_attention=subtract, out_peers=out_peers,
                                  out_group_order=group_order)
        return out

    def _resolve_topk(self, tp, cache: TokenSparseCache):
        """Scalar or (B, H) budget from head / layer adaptation (token_sparse.py:1246-1258)."""
        cfg = self.config
        has_layer = cfg.adaptive_layers and cache.layer_t is not None
        if cfg.adaptive_heads and tp.shape[1] > 1:
            return _compute_adaptive_topk_token(tp, cfg.topk, layer_t=cache.layer_t if has_layer else None)
        if has_layer:
            return cfg.topk * (0.5 + cache.layer_t)
        return cfg.topk

    def _select(self, cache: TokenSparseCache, q_grp, k, lse, scale, perm=None):
        """Group mass + selection of the anchor / update step.  ``q_grp`` is q itself when ``perm`` carries the
        grouping (the mass kernel reads Q through it), else the queries in group order."""
        cfg = self.config
        if cfg.use_chunk_selector:
            # the chunked selector of the reference exists to avoid the (B,H,M,L_K) score tensor; its result is
            # the plain top-k of a fixed budget without sinks, lengths or head adaptation (token_sparse.py:1171-1178)
            L_K = k.shape[2]
            n = max(1, int(cfg.topk * L_K))
            k_sel = min(((n + cfg.tile_n - 1) // cfg.tile_n) * cfg.tile_n, L_K)
            gi = _chunked_online_topk(q_grp, k, lse, cfg.BLKQ, scale, k_sel, tile_n=cfg.tile_n,
                                      chunk_size=cfg.chunk_selector_size, perm=perm)
            return gi, None
        mass = group_mass(q_grp, k, lse, group_rows=cfg.BLKQ, scale=scale, perm=perm, normalize=True)
        return _select_topk_tokens(mass, self._resolve_topk(mass, cache), tile_n=cfg.tile_n,
                                   selection_mode=cfg.selection_mode, topp=cfg.topp, sink_ranges=cfg.sink_ranges)

    def forward(self, cache: TokenSparseCache, q, k, v, scale: Optional[float] = None, out_peers=None):
        """Returns the (B,H,L,D) output, or None when ``out_peers`` was given and the call ended in the sparse
        kernel (reuse step), whose epilogue then stored the rows into the owners' sequence shards."""
        from mcsparse_b200.kernels.flash_mcsa.pca_group import invert_perm_bhld, pca_group_perm
        cfg = self.config
        B, H, L, D = q.shape
        if scale is None:
            scale = 1.0 / math.sqrt(D)
        if cache._cached_len is not None and cache._cached_len != (L, k.shape[2]):
            cache.reset()                                           # length change forces a new anchor step
        mode = cache.mode
        if mode == 'full':
            return dense_attention_with_lse(q, k, v, scale)[0]
        perm = cache._cached_perm
        if cfg.pca_reorder and (mode in _SELECTION_RECOMPUTE_MODES or perm is None):
            perm = pca_group_perm(q.reshape(B * H, L, D) if q.is_contiguous() else q.flatten(0, 1), C=cfg.BLKQ,
                                  pow_iters=cfg.pca_pow_iters, seed=cfg.pca_seed)
            cache._perm_generation += 1
            cache._cached_perm = perm
        if not cfg.pca_reorder:
            perm = None
        if mode in ('calibrate', 'full_calibrate'):
            cache._cached_len = (L, k.shape[2])
            # dense pass on the regrouped queries, read through the permutation; output and LSE in group order
            dense_grp, lse = dense_attention_with_lse(q, k, v, scale, perm=perm, group_order=perm is not None)
            cache._cached_lse = lse
            gi, gl = self._select(cache, q, k, lse, scale, perm=perm)
            cache._cached_indices, cache._cached_lengths = gi, gl
            if cfg.bias_correction:
                # residual = dense - sparse in one kernel pass (the reference runs the sparse kernel and then an
                # elementwise subtraction, token_sparse.py:1209-1216); both operands and the result in group order
                cache._cached_residual = self._sparse(q, k, v, gi, gl, scale, dense_grp, perm, subtract=True,
                                                      group_order=perm is not None)
                cache._residual_perm_gen = cache._perm_generation
            elif mode == 'calibrate':
                # without bias correction a plain anchor step returns the sparse result (token_sparse.py:1290)
                return self._sparse(q, k, v, gi, gl, scale, None, perm)
            return dense_grp if perm is None else invert_perm_bhld(dense_grp, perm)
        if mode == 'approx':
            cache._cached_len = (L, k.shape[2])
            gi = _approx_select(q, k, cfg, perm)
            cache._cached_indices, cache._cached_lengths = gi, None
            return self._sparse(q, k, v, gi, None, scale, None, perm)
        if mode == 'update':
            # new selection from the cached LSE (group order of the anchor step's permutation)
            gi, gl = self._select(cache, q, k, cache._cached_lse, scale, perm=perm)
            cache._cached_indices, cache._cached_lengths = gi, gl
            if cfg.bias_correction:
                # the residual belongs to the selection: renew it against a fresh dense pass and return the dense
                # output (token_sparse.py:1333-1341)
                dense_grp, _ = dense_attention_with_lse(q, k, v, scale, perm=perm, group_order=perm is not None)
                cache._cached_residual = self._sparse(q, k, v, gi, gl, scale, dense_grp, perm, subtract=True,
                                                      group_order=perm is not None)
                cache._residual_perm_gen = cache._perm_generation
                return dense_grp if perm is None else invert_perm_bhld(dense_grp, perm)
            return self._sparse(q, k, v, gi, gl, scale, None, perm)
        # reuse: one fused kernel call
        residual = cache.residual_if_valid() if cfg.bias_correction else None
        return self._sparse(q, k, v, cache._cached_indices, cache._cached_lengths, scale, residual, perm,
                            out_peers=out_peers)


class TokenSparseContext:
    """All layers of a model: one cache per layer, one step clock (token_sparse.py:1461-1845).  Without
    ``num_layers`` the caches are created as layers show up (``cache(li)``).

    Named cache slots (``cache_context`` / ``use_slot``, token_sparse.py:1581-1612) keep separate per-layer caches
    for forwards that alternate within one denoising step (serial classifier-free guidance: a conditional and an
    unconditional pass), so that one pass's anchor step does not overwrite the other's selection; all slots share
    the step clock."""

    def __init__(self, config: TokenSparseConfig, num_layers: Optional[int] = None):
        self.config = config
        self.backend = TokenSparseBackend(config)
        self._nl = num_layers
        self._sc = 0
        self.caches: List[TokenSparseCache] = []
        self._cache_slots = {"_default": self.caches}
        self._active_slot = "_default"
        for i in range(num_layers or 0):
            self.cache(i)

    def cache(self, li: int) -> TokenSparseCache:
        while len(self.caches) <= li:
            i = len(self.caches)
            t = i / max(self._nl - 1, 1) if (self._nl and self.config.adaptive_layers) else None
            c = TokenSparseCache(self.config, i, t)
            c._step_count = self._sc                    # a cache that shows up later joins the common clock
            self.caches.append(c)
        return self.caches[li]

    def use_slot(self, name: str) -> None:
        """Make ``name`` the active cache slot (created empty on first use)."""
        if name not in self._cache_slots:
            self._cache_slots[name] = []
        self._active_slot = name
        self.caches = self._cache_slots[name]
        for i in range(self._nl or 0):
            self.cache(i)

    @contextlib.contextmanager
    def cache_context(self, name: str):
        """Activate a named cache slot for the duration of one forward and restore the previous one afterwards."""
        prev = self._active_slot
        self.use_slot(name)
        try:
            yield
        finally:
            self.use_slot(prev)

    def forward(self, li: int, q, k, v, scale: Optional[float] = None, out_peers=None):
        if self.config.offload_prefetch_ahead and li + 1 < len(self.caches):
            self.caches[li + 1].prefetch()              # comes back under this layer's kernels
        if li in self.config.full_layers:
            return dense_attention_with_lse(q, k, v, scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))[0]
        return self.backend.forward(self.cache(li), q, k, v, scale, out_peers=out_peers)

    def _all_caches(self):
        for slot in self._cache_slots.values():
            yield from slot

    def step(self) -> None:
        self._sc += 1
        for c in self._all_caches():
            c.step()
        if self.caches and self.config.offload_prefetch_ahead:
            self.caches[0].prefetch()                   # the first layer of the next step has no layer in front of it
        # once per denoising step, without synchronising: did any kernel report an expired wait?
        if self.caches and torch.cuda.is_available():
            _lib.poll_status(torch.cuda.current_device(), "TokenSparseContext.step")

    def reset(self) -> None:
        self._sc = 0
        for c in self._all_caches():
            c.reset()
        self.caches = self._cache_slots["_default"]
        self._active_slot = "_default"

    def offload_stats(self) -> dict:
        """Prefetch hits and misses over all layers: a miss is a use that had to copy on its own stream."""
        out = {"idx_prefetch_hit": 0, "idx_prefetch_miss": 0, "res_prefetch_hit": 0, "res_prefetch_miss": 0}
        for c in self._all_caches():
            for k, v in c.offload_stats().items():
                out[k] += v
        return out
