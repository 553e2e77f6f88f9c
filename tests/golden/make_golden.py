"""Generates the golden fixtures in this directory by running the REFERENCE's own CPU-runnable code
(Fast PDDP and token selection) on small seeded inputs.  Needs the reference tree on sys.path
(``PYTHONPATH=/path/to/mcsparse python tests/golden/make_golden.py``); the fixtures it writes are
committed, so the tests themselves never need the reference.
"""

import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def main():
    from mcsparse.kernels.flash_mcsa.pca_group import pca_group_perm
    from mcsparse.kernels.flash_mcsa.token_sparse import _select_topk_tokens

    # ---- Fast PDDP: fp32 clustered inputs, two shapes (power-of-two and ragged block counts)
    cases = []
    for (BH, N, D, C, iters, seed) in [(2, 1024, 32, 128, 4, 0), (2, 1500, 64, 128, 8, 3), (1, 700, 16, 64, 4, 5)]:
        g = torch.Generator().manual_seed(100 + seed)
        cent = torch.randn(BH, 8, D, generator=g)
        cid = torch.randint(0, 8, (N,), generator=g)
        x = cent[:, cid] + 0.3 * torch.randn(BH, N, D, generator=g)
        perm = pca_group_perm(x, C=C, pow_iters=iters, seed=seed)
        cases.append({"BH": BH, "N": N, "D": D, "C": C, "pow_iters": iters, "seed": seed, "gen_seed": 100 + seed,
                      "perm": perm.to(torch.int32)})
    torch.save(cases, HERE / "pddp_reference.pt")

    # ---- selection: tie-free scores, with and without sinks
    sel = []
    for (L, ratio, sinks, seed) in [(1024, 0.125, [(0, 4)], 1), (2000, 0.2, None, 2), (1536, 0.25, [(0, 4), (10, 12)], 3)]:
        g = torch.Generator().manual_seed(seed)
        tp = torch.rand(1, 2, 3, L, generator=g)
        gi, gl = _select_topk_tokens(tp, ratio, sink_ranges=sinks)
        sel.append({"L": L, "ratio": ratio, "sinks": sinks, "seed": seed, "gi": gi, "gl": gl})
    torch.save(sel, HERE / "select_reference.pt")
    print("wrote", HERE / "pddp_reference.pt", HERE / "select_reference.pt")


if __name__ == "__main__":
    main()
