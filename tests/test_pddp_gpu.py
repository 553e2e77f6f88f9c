"""GPU parity: Fast PDDP kernels vs the CPU oracle, in the two stages of the determinism contract:
(1) the fp32 projections match the oracle's within tolerance, level by level, for the same order
entering the level; (2) the new order is bit-exactly the stable sort of the kernel's own fp32
projections; plus end-to-end agreement with the oracle's permutation."""

import pytest
import torch

from oracle.pddp import level_ranges, pddp_perm_ref, resort_from_projections, start_vectors

pytestmark = pytest.mark.gpu


def _clustered(BH, N, D, seed):
    g = torch.Generator().manual_seed(seed)
    cent = torch.randn(BH, 16, D, generator=g)
    cid = torch.randint(0, 16, (N,), generator=g)
    return (cent[:, cid] + 0.3 * torch.randn(BH, N, D, generator=g)).to(torch.bfloat16)


# (the head dimensions other than 64 and 128 run Gram-free power iterations; the contract is the same)
@pytest.mark.parametrize("BH,N,D,C,iters", [(2, 1000, 128, 128, 8), (2, 2048, 64, 128, 4), (1, 5000, 128, 128, 8),
                                            (1, 9000, 128, 64, 4), (2, 5000, 144, 128, 8), (1, 3000, 256, 128, 4),
                                            (2, 2500, 96, 128, 8), (1, 1000, 160, 64, 0)])
def test_two_stage_contract(cuda_device, BH, N, D, C, iters):
    from mcsparse_b200.kernels.flash_mcsa.pca_group import pca_group_perm, pddp_start_vectors
    x = _clustered(BH, N, D, N)
    sv = pddp_start_vectors(BH, N, C, D, seed=0)
    assert torch.equal(sv, torch.cat(start_vectors(BH, N, C, D, 0)))      # same draws as the oracle
    perm, proj, orders = pca_group_perm(x.to(cuda_device), C=C, pow_iters=iters, start_vectors=sv, return_debug=True)
    perm, proj, orders = perm.cpu(), proj.cpu(), orders.cpu().long()
    levels = level_ranges(N, C)
    assert proj.shape[0] == len(levels)
    assert torch.equal(orders[-1], perm)
    assert torch.equal(perm.sort(dim=1).values, torch.arange(N).expand(BH, N))    # a permutation
    xf = x.float()
    v0 = start_vectors(BH, N, C, D, 0)
    for li, nodes in enumerate(levels):
        before, after = orders[li], orders[li + 1]
        # stage 2: new order == stable ascending sort of the kernel's own projections, per node
        assert torch.equal(resort_from_projections(before, proj[li], nodes), after), f"level {li}"
        # stage 1: projections vs an fp32 recomputation from the same incoming order
        for b in range(BH):
            for ni, (s, e) in enumerate(nodes):
                X = xf[b, before[b, s:e]]
                ssum = X.sum(0)
                G = X.T @ X - torch.outer(ssum, ssum) / (e - s)
                v = v0[li][b * len(nodes) + ni].clone()
                v = v / v.norm().clamp(min=1e-12)
                for _ in range(iters):
                    v = G @ v
                    v = v / v.norm().clamp(min=1e-12)
                a = X @ v
                err = (a - proj[li][b, s:e]).abs().max() / a.abs().max().clamp(min=1e-6)
                assert err < 2e-3, (li, b, ni, float(err))


def test_end_to_end_matches_oracle_leaves(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.pca_group import leaf_inertia, pca_group_perm
    BH, N, D, C = 2, 4096, 128, 128
    x = _clustered(BH, N, D, 7)
    perm = pca_group_perm(x.to(cuda_device), C=C, pow_iters=8, seed=0).cpu()
    ref = pddp_perm_ref(x, C=C, pow_iters=8, seed=0)
    same_leaf = ((torch.argsort(ref, 1) // C) == (torch.argsort(perm, 1) // C)).float().mean().item()
    assert same_leaf > 0.98, same_leaf       # near-ties in fp32 projections may move single tokens
    ident = torch.arange(N).expand(BH, N)
    assert leaf_inertia(x, perm, C) < 0.5 * leaf_inertia(x, ident, C)


def test_apply_and_invert_perm(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.pca_group import apply_perm, apply_perm_bhld, invert_perm, invert_perm_bhld
    g = torch.Generator().manual_seed(1)
    x = torch.randn(3, 777, 128, generator=g).to(torch.bfloat16)
    perm = torch.stack([torch.randperm(777, generator=g) for _ in range(3)])
    xp = apply_perm(x.to(cuda_device), perm.to(cuda_device))
    assert torch.equal(xp.cpu(), x.gather(1, perm.unsqueeze(-1).expand(-1, -1, 128)))
    assert torch.equal(invert_perm(xp, perm.to(cuda_device)).cpu(), x)
    x4 = x.view(1, 3, 777, 128)
    assert torch.equal(invert_perm_bhld(apply_perm_bhld(x4.to(cuda_device), perm.to(cuda_device)), perm.to(cuda_device)).cpu(), x4)


def test_short_sequence_is_identity(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.pca_group import pca_group_perm
    x = torch.randn(2, 100, 128).to(torch.bfloat16).to(cuda_device)
    assert torch.equal(pca_group_perm(x, C=128).cpu(), torch.arange(100).expand(2, 100))


@pytest.mark.parametrize("N,C", [(8, 2), (4, 3), (37, 5), (64, 4)])
def test_tiny_groups(cuda_device, N, C):
    """Groups smaller than the projection kernel's row batch (8 slots): nodes of 1 to 7 tokens."""
    from mcsparse_b200.kernels.flash_mcsa.pca_group import pca_group_perm, pddp_start_vectors
    BH, D = 2, 64
    x = _clustered(BH, N, D, 100 + N)
    sv = pddp_start_vectors(BH, N, C, D, seed=0)
    perm, proj, orders = pca_group_perm(x.to(cuda_device), C=C, pow_iters=4, start_vectors=sv, return_debug=True)
    perm, proj, orders = perm.cpu(), proj.cpu(), orders.cpu().long()
    assert torch.equal(perm.sort(dim=1).values, torch.arange(N).expand(BH, N))
    for li, nodes in enumerate(level_ranges(N, C)):
        assert torch.equal(resort_from_projections(orders[li], proj[li], nodes), orders[li + 1]), f"level {li}"
    assert torch.equal(orders[-1], perm)
