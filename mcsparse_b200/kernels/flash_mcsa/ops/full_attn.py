"""Dense attention for full steps and for the anchor (calibrate) step, on (B, H, L, D) tensors.

Mirrors the reference's ``mcsparse/kernels/flash_mcsa/ops/full_attn.py`` (``full_attention`` :65-86,
``full_attention_with_lse`` :88-121).  The reference calls FlashAttention-3 (a Hopper build) and needs three
layout copies in and one out; here both functions run this package's own attention kernel in dense mode
(``mcs_dense_attn_fwd``: every query group attends to all keys) on strided views, so there is no copy, no
external library and no backend to resolve.  The LSE is the natural logarithm of the row sums of
``exp(scale * q . k)``, i.e. it includes the attention scale, as the token-probability kernel expects.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor

from mcsparse_b200 import _lib


def resolve_impl(requested: str = "auto") -> str:
    """The reference chooses between FA3 and SDPA here; this package has one implementation."""
    if requested not in ("auto", "native", "fa3", "sdpa"):
        raise ValueError(f"unknown full-attention implementation {requested!r}")
    return "native"


def describe(resolved: str) -> str:
    return "full attention = mcsparse_b200 dense mode of the gather-KV kernel (sm_100a)"


def _dense(q: Tensor, k: Tensor, v: Tensor, scale: Optional[float], want_lse: bool,
           residual: Optional[Tensor] = None, perm: Optional[Tensor] = None,
           group_order: bool = False) -> Tuple[Tensor, Optional[Tensor]]:
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import interface as itf
    if q.dim() != 4 or k.shape != v.shape or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3]:
        raise ValueError(f"expected (B, H, L, D) tensors, got q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("dense attention needs bf16 or fp16 q, k, v of one dtype")
    if not q.is_cuda:
        raise RuntimeError("dense attention runs on a CUDA device only; there is no CPU path")
    B, H, Lq, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    lse = torch.empty(B, H, Lq, dtype=torch.float32, device=q.device) if want_lse else None
    qv, kv, vv, ov = (itf.maybe_contiguous(t).transpose(1, 2) for t in (q, k, v, out))   # (B, L, H, D) views
    residual, perm = itf._extras_checks(residual, perm, qv, q.dtype, B, H, Lq, D)
    dtype_code = _lib.MCS_DTYPE_BF16 if q.dtype == torch.bfloat16 else _lib.MCS_DTYPE_FP16
    gi_dummy = torch.empty(0, dtype=torch.int32, device=q.device)
    args = itf._fill_args(qv.detach(), kv.detach(), vv.detach(), ov, lse, gi_dummy, None, residual, perm, 128, 128,
                          dtype_code, scale)
    args.gi = None
    if group_order and perm is not None:
        args.flags = _lib.MCS_ATTN_OUT_GROUP_ORDER
    stream = torch.cuda.current_stream(q.device).cuda_stream
    rc = _lib.lib().mcs_dense_attn_fwd(args, stream)
    _lib.raise_on_error(rc, f"mcs_dense_attn_fwd")
    if _lib.check_enabled():
        _lib.check_status(q.device, "full_attention")
    return out, lse


def full_attention(q: Tensor, k: Tensor, v: Tensor, resolved: str = "native", scale: Optional[float] = None) -> Tensor:
    """Exact softmax attention in BHLD layout; query and key lengths may differ."""
    return _dense(q, k, v, scale, want_lse=False)[0]


def full_attention_with_lse(q: Tensor, k: Tensor, v: Tensor, scale: Optional[float] = None, *,
                            perm: Optional[Tensor] = None, group_order: bool = False) -> Tuple[Tensor, Tensor]:
    """Dense attention output (B, H, L_q, D) in q's dtype and its LSE (B, H, L_q) fp32 from one kernel launch.

    ``perm`` ((B*H, L_q) int64, an addition to the reference signature) makes the kernel read query row i from
    ``q[perm[i]]``; output and LSE row i then go back to position ``perm[i]``, or stay at position i (the
    permuted, "group" order the anchor step works in) with ``group_order``."""
    out, lse = _dense(q, k, v, scale, want_lse=True, perm=perm, group_order=group_order)
    return out, lse
