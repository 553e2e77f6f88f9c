"""Oracle: gather-KV sparse attention (+ residual, + permutation, + LSE) on CPU.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Parity against reference
outputs is unpinned: the reference ships no CPU path and no golden vectors for this
operator.  The function restates the operator contract:

* group of query row i is ``i // group_rows``; its key multiset is
  ``gi[b,h,m, 0:T*128]`` with ``T = gl[b,h,m]`` or ``gather_len/128``
  (interface.py:121-136, flash_fwd_sm90.py:826-829);
* indices address rows of the ORIGINAL K/V of that head (topk_gather_kv.py:351-360,
  flash_fwd_sm90.py:762-768); duplicates are separate softmax columns;
* ``O = softmax(scale * Q K_J^T) V_J``; ``lse = max*scale + ln(sum)`` natural log
  (softmax.py:192-227);
* reuse step adds the cached residual in permuted-query (B,H,L,D) order
  (token_sparse.py:1095-1112); with a permutation only Q rows are permuted and
  the output is un-permuted afterwards (token_sparse.py:1056-1060, pca_group.py:40-61).
"""

from __future__ import annotations

import math
from typing import Optional

import torch


def gather_attn_ref(
    q: torch.Tensor,            # (B, Sq, H, D)
    k: torch.Tensor,            # (B, Sk, H, D)
    v: torch.Tensor,            # (B, Sk, H, D)
    gi: torch.Tensor,           # (B, H, M, gather_len) int
    softmax_scale: Optional[float] = None,
    gl: Optional[torch.Tensor] = None,        # (B, H, M) tile counts
    residual: Optional[torch.Tensor] = None,  # (B, H, Sq, D), permuted query order
    perm: Optional[torch.Tensor] = None,      # (B*H, Sq) int64
    group_rows: int = 128,
    dtype: torch.dtype = torch.float32,
):
    """Returns ``(out (B,Sq,H,D), lse (B,H,Sq))`` in ``dtype`` (fp32 or fp64), original token order."""
    B, Sq, H, D = q.shape
    M = math.ceil(Sq / group_rows)
    gather_len = gi.shape[-1]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    out = torch.zeros(B, Sq, H, D, dtype=dtype)
    lse = torch.zeros(B, H, Sq, dtype=dtype)
    for b in range(B):
        for h in range(H):
            kh, vh = kf[b, :, h], vf[b, :, h]
            p = perm[b * H + h].long() if perm is not None else None
            for m in range(M):
                lo, hi = m * group_rows, min((m + 1) * group_rows, Sq)
                n = gather_len if gl is None else int(gl[b, h, m]) * 128
                idx = gi[b, h, m, :n].long()
                rows = torch.arange(lo, hi)
                src = p[rows] if p is not None else rows
                s = (qf[b, src, h] @ kh[idx].T) * softmax_scale
                l = torch.logsumexp(s, dim=-1)
                o = torch.softmax(s, dim=-1) @ vh[idx]
                if residual is not None:
                    o = o + residual[b, h, lo:hi].to(dtype)
                out[b, src, h] = o
                lse[b, h, src] = l
    return out, lse


def dense_attn_ref(q, k, v, softmax_scale=None, dtype=torch.float32):
    """Plain dense attention on (B,S,H,D) tensors: ``(out, lse)``; used to validate the oracle itself."""
    B, Sq, H, D = q.shape
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    qf, kf, vf = (t.to(dtype).permute(0, 2, 1, 3) for t in (q, k, v))
    s = (qf @ kf.transpose(-1, -2)) * softmax_scale
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ vf
    return o.permute(0, 2, 1, 3).contiguous(), lse


def error_metrics(out: torch.Tensor, ref: torch.Tensor):
    """(max-abs, mean-rel) as used for the stated tolerances: mean|d| / mean|ref|."""
    d = (out.double() - ref.double()).abs()
    return float(d.max()), float(d.mean() / ref.double().abs().mean().clamp_min(1e-30))


def gather_attn_fp8_ref(q8, k8, v8, gi, scale_qk_log2, scale_v, gl=None, residual=None, perm=None,
                        dtype=torch.float32):
    """FP8 entry point contract (interface.py:358-373, flash_fwd_sm90_fp8.py:19-23, 145-241):
    logits in the log2 domain are ``(q8 . k8) * scale_qk_log2[b,h,m]``; the output is
    ``softmax(...) @ v8 * scale_v[b,h]``.  The kernel's internal P quantisation and 2^k offsets are
    implementation details covered by the tolerance.  q8/k8/v8: float8_e4m3fn (B,S,H,D)."""
    B, Sq, H, D = q8.shape
    M = gi.shape[2]
    qf, kf, vf = q8.to(dtype), k8.to(dtype), v8.to(dtype)
    out = torch.zeros(B, Sq, H, D, dtype=dtype)
    lse = torch.zeros(B, H, Sq, dtype=dtype)
    ln2 = math.log(2.0)
    for b in range(B):
        for h in range(H):
            p = perm[b * H + h].long() if perm is not None else None
            for m in range(M):
                lo, hi = m * 128, min((m + 1) * 128, Sq)
                n = gi.shape[-1] if gl is None else int(gl[b, h, m]) * 128
                idx = gi[b, h, m, :n].long()
                rows = torch.arange(lo, hi)
                src = p[rows] if p is not None else rows
                s = (qf[b, src, h] @ kf[b, idx, h].T) * float(scale_qk_log2[b, h, m]) * ln2
                o = torch.softmax(s, dim=-1) @ vf[b, idx, h] * float(scale_v[b, h])
                if residual is not None:
                    o = o + residual[b, h, lo:hi].to(dtype)
                out[b, src, h] = o
                lse[b, h, src] = torch.logsumexp(s, dim=-1)
    return out, lse
