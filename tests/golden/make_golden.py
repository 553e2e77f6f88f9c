"""Generates the golden fixtures in this directory by running the REFERENCE's own code on small seeded
inputs: Fast PDDP and token selection (plain torch, CPU) and the group-mass kernel
(``ops/triton/block_probs.py``, a Triton kernel, executed on the CPU by Triton's interpreter,
``TRITON_INTERPRET=1``).  Needs the reference tree on sys.path
(``PYTHONPATH=/path/to/mcsparse python tests/golden/make_golden.py``); the fixtures it writes are
committed, so the tests themselves never need the reference.
"""

import math
import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")     # must be set before triton is imported

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
from mass_cases import MASS_CASES, mass_inputs  # noqa: E402

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
    # ---- variable-length selection modes on normalised probabilities
    modes = []
    for (L, mode, ratio, topp, sinks, seed) in [(1536, "topp", 0.1, 0.6, None, 11), (2000, "topp", 0.1, 0.9, [(0, 4)], 12),
                                                (1536, "topk_topp", 0.25, 0.5, [(0, 4)], 13), (1024, "topk_topp", 0.05, 0.8, None, 14),
                                                (1536, "topk", "adaptive", None, [(0, 4)], 15), (2048, "topk_topp", "adaptive", 0.7, None, 16)]:
        g = torch.Generator().manual_seed(seed)
        # peaked rows: a softmax over scaled logits so that top-p prefixes have very different lengths
        tp = torch.softmax(torch.randn(1, 2, 3, L, generator=g) * torch.tensor([1.0, 3.0]).view(1, 2, 1, 1), dim=-1)
        r = torch.tensor([[0.08, 0.3]]) if ratio == "adaptive" else ratio
        gi, gl = _select_topk_tokens(tp, r, selection_mode=mode, topp=topp, sink_ranges=sinks)
        modes.append({"L": L, "mode": mode, "ratio": ratio, "topp": topp, "sinks": sinks, "seed": seed, "gi": gi, "gl": gl})
    # per-head budgets from retained mass (adaptive heads), with and without layer depth
    from mcsparse.kernels.flash_mcsa.token_sparse import _compute_adaptive_topk_token
    g = torch.Generator().manual_seed(21)
    tp = torch.softmax(torch.randn(2, 4, 3, 1024, generator=g) * torch.tensor([0.5, 1.0, 2.0, 4.0]).view(1, 4, 1, 1), dim=-1)
    modes.append({"mode": "adaptive_ratio", "seed": 21, "base": 0.1,
                  "ratio": _compute_adaptive_topk_token(tp, 0.1), "ratio_t": _compute_adaptive_topk_token(tp, 0.1, layer_t=0.25)})
    torch.save(modes, HERE / "select_modes_reference.pt")
    print("wrote", HERE / "select_modes_reference.pt")
    mass_golden()


def mass_golden():
    """Group mass by the reference's own Triton kernel (block_probs.py:27-117: mean over the block's rows,
    output in the input dtype)."""
    from mcsparse.kernels.flash_mcsa.ops.triton.block_probs import _compute_token_probs_bf16_triton
    out = []
    for case in MASS_CASES:
        q, k, lse, scale = mass_inputs(case)
        M = math.ceil(case["Lq"] / 128)
        tp = _compute_token_probs_bf16_triton(q, k, lse, 128, M, scale)
        assert torch.isfinite(tp.float()).all()
        out.append({**case, "token_probs": tp})
    torch.save(out, HERE / "mass_reference.pt")
    print("wrote", HERE / "mass_reference.pt")


if __name__ == "__main__":
    main()
