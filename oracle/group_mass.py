"""Oracle: group attention mass on CPU.  TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Restates mcsparse/kernels/flash_mcsa/ops/triton/block_probs.py:27-89: per (head, query block m,
key j) ``(1/n_m) * sum_{i in block m} exp(scale * q_i . k_j - lse_i)``, rows past L_Q contribute 0
(:77) and the divisor is the number of real rows in the block (:79-80).  ``normalize=False`` gives
the plain sum.  Pinned: ``tests/test_oracle.py`` compares it with outputs of the reference kernel
itself (run through Triton's CPU interpreter by ``tests/golden/make_golden.py``); the identity
``sum_j mass = n_m`` for an exact lse is checked as well.
"""

from __future__ import annotations

import math

import torch


def group_mass_ref(q, k, lse, group_rows=128, scale=None, perm=None, normalize=False, dtype=torch.float64):
    """q: (B,H,Lq,D), k: (B,H,Lk,D), lse: (B,H,Lq) in group order. Returns (B,H,M,Lk) in ``dtype``."""
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    M = math.ceil(Lq / group_rows)
    out = torch.zeros(B, H, M, Lk, dtype=dtype)
    for b in range(B):
        for h in range(H):
            qh = q[b, h].to(dtype)
            if perm is not None:
                qh = qh[perm[b * H + h].long()]
            s = qh @ k[b, h].to(dtype).T * scale - lse[b, h].to(dtype)[:, None]
            pr = torch.exp(s)
            for m in range(M):
                blk = pr[m * group_rows:(m + 1) * group_rows]
                out[b, h, m] = blk.sum(0) / (blk.shape[0] if normalize else 1)
    return out


def dense_lse_ref(q, k, scale=None, dtype=torch.float64):
    """Natural-log LSE of scaled logits, (B,H,Lq); q,k: (B,H,L,D)."""
    D = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    s = q.to(dtype) @ k.to(dtype).transpose(-1, -2) * scale
    return torch.logsumexp(s, dim=-1)
