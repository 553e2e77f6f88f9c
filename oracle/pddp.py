"""Oracle: Fast PDDP query grouping on CPU.  TEST INFRASTRUCTURE ONLY.

Restates mcsparse/kernels/flash_mcsa/pca_group.py:141-243 node by node:
block intervals [lo, hi) of C tokens, every interval processed at every level (:187-188);
per node Gram ``X^T X - s s^T / n`` in fp32 (:216-221), one start vector per node drawn level by
level from a single seeded generator (:184-185, :224), ``pow_iters`` normalised mat-vecs with the
norm clamped at 1e-12 (:225-228), projection ``a = X v`` (:232), sort, write back (:234-239), split
at the block midpoint ``lo + (hi - lo) // 2`` (:112).

Deterministic contract of this oracle (what the CUDA path is compared with bit for bit, given the
same fp32 projections): projections in fp32, STABLE ascending sort, ties keep the current order.
Pinned against the reference's own ``pca_group_perm`` on CPU with fp32 inputs
(``tests/test_oracle.py`` when the reference tree is present, and ``tests/golden/pddp_*.pt``).
"""

from __future__ import annotations

import torch


def level_ranges(N: int, C: int):
    """List of levels; each level is a list of (token_start, token_end) of its nodes."""
    K = (N + C - 1) // C
    ranges = [(0, K)]
    levels = []
    while any(hi - lo > 1 for lo, hi in ranges):
        levels.append([(lo * C, min(hi * C, N)) for lo, hi in ranges])
        nxt = []
        for lo, hi in ranges:
            if hi - lo <= 1:
                nxt.append((lo, hi))
            else:
                mid = lo + (hi - lo) // 2
                nxt += [(lo, mid), (mid, hi)]
        ranges = nxt
    return levels


def start_vectors(BH: int, N: int, C: int, D: int, seed: int = 0):
    """Per level a (BH * nodes, D) fp32 tensor: the reference's draws on a CPU generator (row bh*nodes+node)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    return [torch.randn(BH * len(lv), D, generator=gen) for lv in level_ranges(N, C)]


def pddp_perm_ref(x: torch.Tensor, C: int = 128, pow_iters: int = 4, seed: int = 0, v0=None,
                  return_projections: bool = False):
    """x: (BH, N, D). Returns perm (BH, N) int64 [, list of per-level fp32 projections (BH, N) by position]."""
    BH, N, D = x.shape
    perm = torch.arange(N).unsqueeze(0).expand(BH, N).clone()
    if N <= C:
        return (perm, []) if return_projections else perm
    xf = x.float()
    levels = level_ranges(N, C)
    if v0 is None:
        v0 = start_vectors(BH, N, C, D, seed)
    projs = []
    for li, nodes in enumerate(levels):
        proj = torch.zeros(BH, N)
        new_perm = perm.clone()
        for b in range(BH):
            for ni, (s, e) in enumerate(nodes):
                ids = perm[b, s:e]
                X = xf[b, ids]                                   # (n, D)
                n = e - s
                ssum = X.sum(0)
                G = X.T @ X - torch.outer(ssum, ssum) / n
                v = v0[li][b * len(nodes) + ni].clone()
                v = v / v.norm().clamp(min=1e-12)
                for _ in range(pow_iters):
                    v = G @ v
                    v = v / v.norm().clamp(min=1e-12)
                a = X @ v
                proj[b, s:e] = a
                order = torch.sort(a, stable=True).indices
                new_perm[b, s:e] = ids[order]
        perm = new_perm
        projs.append(proj)
    return (perm, projs) if return_projections else perm


def resort_from_projections(perm_before: torch.Tensor, proj: torch.Tensor, nodes):
    """Second stage of the two-stage contract: given the perm entering a level and the fp32 projections
    of every position, the stable ascending sort inside each node."""
    out = perm_before.clone()
    for b in range(perm_before.shape[0]):
        for s, e in nodes:
            order = torch.sort(proj[b, s:e], stable=True).indices
            out[b, s:e] = perm_before[b, s:e][order]
    return out
