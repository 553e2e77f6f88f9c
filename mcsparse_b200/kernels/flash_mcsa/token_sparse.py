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
