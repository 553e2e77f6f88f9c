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
