"""GPU parity: dense attention with LSE (the attention kernel's dense mode) against the fp32 oracle.

Tolerances as for the sparse path: max-abs 2e-2, mean-rel 1e-2 on the output; the LSE is fp32 arithmetic
on bf16-rounded products and must agree to 2e-3 absolute."""

import pytest
import torch

from oracle.gather_attn import dense_attn_ref, error_metrics

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Lq,Lk,D", [(1000, 1000, 128), (384, 1300, 64), (130, 70, 128), (256, 128, 128), (77, 4000, 128)])
def test_dense_matches_oracle(cuda_device, dtype, Lq, Lk, D):
    from mcsparse_b200.kernels.flash_mcsa.ops.full_attn import full_attention, full_attention_with_lse
    B, H = 2, 3
    g = torch.Generator().manual_seed(Lq * 7 + Lk)
    q = torch.randn(B, H, Lq, D, generator=g).to(dtype)
    k = torch.randn(B, H, Lk, D, generator=g).to(dtype)
    v = torch.randn(B, H, Lk, D, generator=g).to(dtype)
    ref, ref_lse = dense_attn_ref(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    out, lse = full_attention_with_lse(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
    assert out.shape == q.shape and out.dtype == dtype and lse.shape == (B, H, Lq) and lse.dtype == torch.float32
    mx, mr = error_metrics(out.float().cpu().transpose(1, 2), ref)
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)
    assert float((lse.cpu() - ref_lse).abs().max()) < 2e-3
    out2 = full_attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
    assert torch.equal(out2, out)


def test_dense_peaked_rows_and_scale(cuda_device):
    """Rows whose maximum sits in the masked-off part's neighbourhood (last, partial tile) and a custom scale."""
    from mcsparse_b200.kernels.flash_mcsa.ops.full_attn import full_attention_with_lse
    B, H, L, D = 1, 2, 300, 128
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)
    k[:, :, -1] = 4 * q[:, :, 0]                      # the very last key dominates row 0
    v = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)
    ref, ref_lse = dense_attn_ref(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), softmax_scale=0.2)
    out, lse = full_attention_with_lse(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), scale=0.2)
    mx, mr = error_metrics(out.float().cpu().transpose(1, 2), ref)
    assert mx < 3e-2 and mr < 1e-2, (mx, mr)
    assert float(((lse.cpu() - ref_lse).abs() / ref_lse.abs().clamp_min(1)).max()) < 2e-3


def test_dense_argument_errors(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.ops.full_attn import full_attention
    q = torch.randn(1, 2, 64, 128, device=cuda_device)
    with pytest.raises(TypeError):
        full_attention(q, q, q)                        # fp32 is not supported
    qh = q.to(torch.bfloat16)
    with pytest.raises(ValueError):
        full_attention(qh, qh[:, :1], qh)              # head count mismatch
