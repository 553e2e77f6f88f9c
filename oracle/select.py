"""Oracle: exact top-k selection with forced sinks on CPU.  TEST INFRASTRUCTURE ONLY.

Definition (tightens mcsparse/kernels/flash_mcsa/token_sparse.py:755-945, topk mode): sinks are
removed from the ranking (:802-803) and forced in (:902-905); the other tokens are ranked by a
stable descending sort of the fp32 score, so ties go to the lowest index; the result is ascending.
Pinned against the reference's own ``_select_topk_tokens`` (run on CPU): on tie-free scores the
reference's selected SET must equal this one's after the reference's truncation is accounted for
(``tests/test_oracle.py``, golden vectors in ``tests/golden``).
"""

from __future__ import annotations

import torch


def select_topk_ref(scores: torch.Tensor, k_total: int, sinks=()) -> torch.Tensor:
    """scores (..., L) float; returns (..., k_total) int32 ascending."""
    L = scores.shape[-1]
    sinks = sorted(set(int(s) for s in sinks))
    flat = scores.reshape(-1, L).float()
    mask = torch.zeros(L, dtype=torch.bool)
    if sinks:
        mask[torch.tensor(sinks)] = True
    out = torch.empty(flat.shape[0], k_total, dtype=torch.int32)
    nonsink = (~mask).nonzero(as_tuple=True)[0]
    k = k_total - len(sinks)
    for r in range(flat.shape[0]):
        vals = flat[r, nonsink]
        order = torch.sort(vals, descending=True, stable=True).indices[:k]
        sel = torch.cat([torch.tensor(sinks, dtype=torch.long), nonsink[order]])
        out[r] = sel.sort().values.to(torch.int32)
    return out.reshape(*scores.shape[:-1], k_total)


def topp_count_ref(scores: torch.Tensor, topp: float, sinks=()) -> torch.Tensor:
    """Per row: number of tokens, in descending order of score, whose preceding mass is below ``topp``
    (token_sparse.py:842-852: sort, cumulative sum minus self, mask, count); sinks are not ranked.  fp64 sums."""
    L = scores.shape[-1]
    flat = scores.reshape(-1, L).double().clone()
    sinks = sorted(set(int(s) for s in sinks))
    keep = torch.ones(L, dtype=torch.bool)
    if sinks:
        keep[torch.tensor(sinks)] = False
    out = torch.empty(flat.shape[0], dtype=torch.int32)
    for r in range(flat.shape[0]):
        v = torch.sort(flat[r, keep], descending=True, stable=True).values
        before = torch.cumsum(v, 0) - v
        out[r] = max(1, int((before < topp).sum()))
    return out.reshape(scores.shape[:-1])


def selection_counts_ref(L_K: int, n_sink: int, tile_n: int, base_counts: torch.Tensor) -> torch.Tensor:
    """Budget arithmetic of the variable-length modes (token_sparse.py:811-823 _align_up, :902-913 sink
    re-alignment, :915-923 cap), per row, in tokens."""
    c = base_counts.long().clamp(min=1)
    c = (((c + tile_n - 1) // tile_n) * tile_n).clamp(max=L_K)
    actual = int(c.max()) + n_sink
    if n_sink:
        c = (((c + n_sink + tile_n - 1) // tile_n) * tile_n).clamp(max=actual)
    cap = max(tile_n, min(((L_K + tile_n - 1) // tile_n) * tile_n, (actual // tile_n) * tile_n))
    c = c.clamp(min=tile_n, max=cap)
    return (c // tile_n) * tile_n


def select_modes_ref(scores: torch.Tensor, ratio, mode: str, topp=None, sinks=(), tile_n: int = 128):
    """Variable-length selection (token_sparse.py:755-945: per-head budgets, topp, topk_topp) under this oracle's
    deterministic contract: every row keeps the sinks plus its best-ranked other tokens (stable descending sort),
    ascending, zero-padded to the longest row.  scores (B,H,M,L).  Returns (gi int32 (B,H,M,kmax), tile counts
    int32 (B,H,M))."""
    B, H, M, L = scores.shape
    sinks = sorted(set(int(s) for s in sinks))
    adaptive = isinstance(ratio, torch.Tensor)
    if mode == "topk":
        base = (ratio.float() * L).long().view(B, H, 1).expand(B, H, M)
    else:
        base = topp_count_ref(scores, topp, sinks).long()
        if mode == "topk_topp":
            if adaptive:
                floor_k = (ratio.float() * L).clamp(min=1, max=L).long().view(B, H, 1).expand(B, H, M)
            else:
                floor_k = torch.full_like(base, min(max(1, int(ratio * L)), L))
            base = torch.maximum(base, floor_k)
    counts = selection_counts_ref(L, len(sinks), tile_n, base).clamp(max=L)
    kmax = int(counts.max())
    gi = torch.zeros(B, H, M, kmax, dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            for m in range(M):
                c = int(counts[b, h, m])
                gi[b, h, m, :c] = select_topk_ref(scores[b, h, m].view(1, L), c, sinks)[0]
    return gi, (counts // tile_n).to(torch.int32)
