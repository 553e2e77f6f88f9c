"""Oracle: the context-parallel DiT attention layer of the multi-GPU benchmark configuration, unsharded, on CPU
in fp32.  TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

The reference contains the attention call of this layer only (``forward_op``, mcsparse/h3/context_parallel.py:
165-176); projections, q/k normalisation and rotary embedding belong to the host model, which is not part of the
reference tree.  PARITY UNPINNED against reference outputs: the definitions below are the ones stated in
``mcsparse_b200/h3/ulysses_layer.py`` (RMSNorm over the head dimension, interleaved rotary pairs split over frame /
row / column, theta 10000), restated with plain torch operations; the attention in the middle is
``oracle.gather_attn.gather_attn_ref``.
"""

from __future__ import annotations

import torch

from oracle.gather_attn import gather_attn_ref


def rope_angles(grid, head_dim: int, theta: float = 10000.0) -> torch.Tensor:
    """(L, D/2) rotation angle of every token (frame-major flattening) and rotation pair."""
    F, Hh, W = grid
    per = head_dim // 6
    n_t, n_h, n_w = head_dim // 2 - 2 * per, per, per
    f = torch.arange(F).view(F, 1, 1).expand(F, Hh, W).reshape(-1).double()
    y = torch.arange(Hh).view(1, Hh, 1).expand(F, Hh, W).reshape(-1).double()
    x = torch.arange(W).view(1, 1, W).expand(F, Hh, W).reshape(-1).double()
    parts = []
    for pos, n in ((f, n_t), (y, n_h), (x, n_w)):
        freq = theta ** (-torch.arange(n, dtype=torch.float64) / max(n, 1))
        parts.append(pos[:, None] * freq[None, :])
    return torch.cat(parts, dim=1)


def norm_rope_ref(t: torch.Tensor, gamma: torch.Tensor, angles: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """t: (L, H, D) fp32.  RMSNorm over D with weight gamma, then rotation of pairs (2p, 2p+1) by angles[l, p]."""
    t = t.double()
    t = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * gamma.double()
    a, b = t[..., 0::2], t[..., 1::2]
    c, s = torch.cos(angles)[:, None, :], torch.sin(angles)[:, None, :]
    out = torch.empty_like(t)
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = a * s + b * c
    return out.float()


def layer_ref(x, w, grid, heads: int, head_dim: int, gi, residual=None, perm=None, eps: float = 1e-6, round_to=None):
    """x: (L, hidden).  Returns (out (L, hidden), q, k, v (1, L, H, D)) in fp32.  ``round_to`` (a 16-bit dtype)
    rounds the projection outputs, q/k/v and the attention output where the GPU layer stores 16-bit tensors, which
    makes the comparison of the final output independent of those roundings."""
    rd = (lambda t: t.to(round_to).float()) if round_to is not None else (lambda t: t)
    L = x.shape[0]
    xf = x.float()
    ang = rope_angles(grid, head_dim)
    q = rd(xf @ w["wq"].float().t()).view(L, heads, head_dim)
    k = rd(xf @ w["wk"].float().t()).view(L, heads, head_dim)
    v = rd(xf @ w["wv"].float().t()).view(L, heads, head_dim)
    q = rd(norm_rope_ref(q, w["gq"].float(), ang, eps)).unsqueeze(0)
    k = rd(norm_rope_ref(k, w["gk"].float(), ang, eps)).unsqueeze(0)
    v = v.unsqueeze(0)
    o, _ = gather_attn_ref(q, k, v, gi, residual=residual, perm=perm)
    o = rd(o)
    out = o.reshape(L, heads * head_dim) @ w["wo"].float().t()
    return out, q, k, v
