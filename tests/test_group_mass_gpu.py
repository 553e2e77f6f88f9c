"""GPU parity: group-mass kernel vs the CPU oracle (through the C ABI)."""

import pytest
import torch

from oracle.group_mass import dense_lse_ref, group_mass_ref

pytestmark = pytest.mark.gpu


def _clustered(B, H, L, D, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    cent = torch.randn(H, 8, D, generator=g)
    cid = torch.randint(0, 8, (L,), generator=g)
    q = (cent[:, cid] + 0.3 * torch.randn(B, H, L, D, generator=g)).to(dtype)
    k = (cent[:, cid] + 0.3 * torch.randn(B, H, L, D, generator=g)).to(dtype)
    return q, k


@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (64, torch.bfloat16), (128, torch.float16)])
def test_mass_matches_oracle(cuda_device, D, dtype):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import group_mass
    B, H, L = 1, 2, 600          # ragged: last query group has 88 rows, last key tile 88 tokens
    q, k = _clustered(B, H, L, D, 1, dtype)
    lse = dense_lse_ref(q, k).float()
    ref = group_mass_ref(q, k, lse)
    out = group_mass(q.to(cuda_device), k.to(cuda_device), lse.to(cuda_device)).cpu().double()
    # ex2.approx and fp32 accumulation: relative to the row's total mass
    err = (out - ref).abs().max() / ref.abs().max()
    assert err < 2e-3, err
    # with an exact lse every query row contributes total mass 1
    M = ref.shape[2]
    rows = torch.tensor([min(128, L - 128 * m) for m in range(M)], dtype=torch.float64)
    assert torch.allclose(out.sum(-1), rows.expand(B, H, M), rtol=3e-3)


def test_mass_with_perm_and_normalize(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import _compute_token_probs, group_mass
    B, H, L, D = 1, 2, 384, 128
    q, k = _clustered(B, H, L, D, 2, torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    perm = torch.stack([torch.randperm(L, generator=g) for _ in range(B * H)])
    qp = torch.stack([q[0, h][perm[h]] for h in range(H)]).unsqueeze(0)
    lse_p = dense_lse_ref(qp, k).float()           # lse in permuted order, as the dense pass on q_perm gives it
    ref = group_mass_ref(q, k, lse_p, perm=perm, normalize=True)
    dev = cuda_device
    out = group_mass(q.to(dev), k.to(dev), lse_p.to(dev), perm=perm.to(dev), normalize=True).cpu().double()
    assert (out - ref).abs().max() / ref.abs().max() < 2e-3
    # reference-compatible wrapper on already permuted queries: mean, rounded to q.dtype
    tp = _compute_token_probs(qp.to(dev), k.to(dev), lse_p.to(dev), 128, 1.0 / D ** 0.5)
    assert tp.dtype == torch.bfloat16 and tuple(tp.shape) == (B, H, 3, L)
    assert (tp.cpu().double() - ref).abs().max() / ref.abs().max() < 1e-2


def test_mass_with_keys_shared_by_heads(cuda_device):
    """K expanded over the heads (head stride 0): no tensor map describes that layout, so the kernel copies the key
    tiles with cp.async instead of TMA; the result must not depend on the route."""
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import group_mass
    B, H, L, D = 1, 2, 600, 128
    q, k = _clustered(B, H, L, D, 4, torch.bfloat16)
    k1 = k[:, :1]
    lse = dense_lse_ref(q, k1.expand(B, H, L, D)).float()
    ref = group_mass_ref(q, k1.expand(B, H, L, D).contiguous(), lse)
    dev = cuda_device
    kd = k1.to(dev).expand(B, H, L, D)
    assert kd.stride(1) == 0
    out = group_mass(q.to(dev), kd, lse.to(dev)).cpu().double()
    assert (out - ref).abs().max() / ref.abs().max() < 2e-3
    both = group_mass(q.to(dev), kd.contiguous(), lse.to(dev)).cpu().double()      # TMA route, same numbers
    assert torch.equal(out, both)


def test_mass_matches_reference_kernel_output(cuda_device):
    """The CUDA kernel against outputs of the reference's own Triton kernel (block_probs.py:27-117) on the same
    seeded inputs; the fixtures were produced by tests/golden/make_golden.py with Triton's CPU interpreter.
    fp16 cases run the kernel on the very same fp16 tensors; the "bf16_as_f32" cases carry bf16 values in fp32
    (exact products), so the kernel runs on their bf16 form."""
    import sys
    from pathlib import Path
    golden = Path(__file__).resolve().parent / "golden"
    sys.path.insert(0, str(golden))
    from mass_cases import mass_inputs
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import _compute_token_probs, group_mass
    dev = cuda_device
    for c in torch.load(golden / "mass_reference.pt"):
        q, k, lse, scale = mass_inputs(c)
        if c["dtype"] == "bf16_as_f32":
            q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)       # exact: the values are bf16 already
        ref = c["token_probs"].double()
        mean = group_mass(q.to(dev), k.to(dev), lse.to(dev), scale=scale, normalize=True).cpu().double()
        assert (mean - ref).abs().max() / ref.abs().max() < 2e-3, c
        # fp32 sum (what the selection ranks on) = the reference's mean times the rows of the block
        rows = torch.tensor([min(128, c["Lq"] - 128 * m) for m in range(ref.shape[2])], dtype=torch.float64)
        total = group_mass(q.to(dev), k.to(dev), lse.to(dev), scale=scale).cpu().double()
        assert (total - ref * rows.view(1, 1, -1, 1)).abs().max() / (ref * rows.view(1, 1, -1, 1)).abs().max() < 2e-3
        # reference-shaped wrapper: mean rounded to the input dtype, as the reference stores it
        tp = _compute_token_probs(q.to(dev), k.to(dev), lse.to(dev), 128, scale)
        assert tp.dtype == q.dtype
        assert (tp.cpu().double() - ref).abs().max() / ref.abs().max() < (1e-2 if q.dtype == torch.bfloat16 else 3e-3)


@pytest.mark.parametrize("D", [96, 144, 160, 192, 256, 32])
def test_mass_other_head_dims(cuda_device, D):
    """Head dimensions other than 64 and 128 (the reference's Triton kernel takes any; its head-dimension table lists
    96, 144, 160, 192, 256): padded tile layouts, by TMA (contiguous keys) and by cp.async (keys shared by the heads),
    with a permutation and ragged last group / last key tile."""
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import group_mass
    B, H, L = 1, 2, 600
    q, k = _clustered(B, H, L, D, 10 + D, torch.bfloat16)
    g = torch.Generator().manual_seed(D)
    perm = torch.stack([torch.randperm(L, generator=g) for _ in range(B * H)])
    qp = torch.stack([q[0, h][perm[h]] for h in range(H)]).unsqueeze(0)
    lse_p = dense_lse_ref(qp, k).float()
    ref = group_mass_ref(q, k, lse_p, perm=perm)
    dev = cuda_device
    out = group_mass(q.to(dev), k.to(dev), lse_p.to(dev), perm=perm.to(dev)).cpu().double()
    assert (out - ref).abs().max() / ref.abs().max() < 2e-3
    # keys of head 0 shared by both heads: no tensor map, the cp.async route
    k1 = k[:, :1]
    lse1 = dense_lse_ref(q, k1.expand(B, H, L, D)).float()
    ref1 = group_mass_ref(q, k1.expand(B, H, L, D).contiguous(), lse1)
    kd = k1.to(dev).expand(B, H, L, D)
    out1 = group_mass(q.to(dev), kd, lse1.to(dev)).cpu().double()
    assert (out1 - ref1).abs().max() / ref1.abs().max() < 2e-3
    assert torch.equal(out1, group_mass(q.to(dev), kd.contiguous(), lse1.to(dev)).cpu().double())
