"""GPU parity: gather-KV attention at the head dimensions other than 64 and 128 (the reference's table:
96, 144 padded to 160, 192, 256; cute/interface.py:45-74, :138-159) against the CPU oracle, through the C ABI.

Tolerances as for the main kernel: max-abs 2e-2 / mean-rel 1e-2 on the output, 2e-2 on the LSE."""

import math

import pytest
import torch

from oracle.gather_attn import dense_attn_ref, error_metrics, gather_attn_ref

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 2e-2, 1e-2


def _make(B, H, Sq, Sk, D, gather_len, group_rows, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    k = torch.randn(B, Sk, H, D, generator=g).to(dtype)
    v = torch.randn(B, Sk, H, D, generator=g).to(dtype)
    M = math.ceil(Sq / group_rows)
    gi = torch.empty(B, H, M, gather_len, dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            for m in range(M):
                rest = torch.randperm(Sk - 4, generator=g)[: gather_len - 4] + 4
                gi[b, h, m] = torch.cat([torch.arange(4), rest.sort().values]).to(torch.int32)
    return q, k, v, gi


def _run(dev, q, k, v, gi, **kw):
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
    kw = {kk: (vv.to(dev) if torch.is_tensor(vv) else vv) for kk, vv in kw.items()}
    out, lse = flash_attn_gather_kv_func(q.to(dev), k.to(dev), v.to(dev), gi.to(dev), return_lse=True, **kw)
    torch.cuda.synchronize()
    return out.float().cpu(), lse.cpu()


@pytest.mark.parametrize("D", [32, 96, 144, 160, 192, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_head_dims_of_the_reference_table(cuda_device, D, dtype):
    # 5 key tiles per group: the 2-slot ring of D = 256 and the 3-slot ring of 144..192 wrap several times
    q, k, v, gi = _make(1, 2, 300, 900, D, 640, 128, dtype, seed=D)
    out, lse = _run(cuda_device, q, k, v, gi)
    ref, ref_lse = gather_attn_ref(q, k, v, gi)
    mx, mr = error_metrics(out, ref)
    assert mx < MAX_ABS and mr < MEAN_REL, (D, mx, mr)
    assert (lse - ref_lse).abs().max() < 2e-2


@pytest.mark.parametrize("D", [144, 256])
def test_residual_perm_lengths_and_many_items(cuda_device, D):
    """Residual, query permutation, per-group tile counts (1..6) and more work items than SMs."""
    B, H, Sq, Sk = 2, 3, 4000, 1500
    q, k, v, gi = _make(B, H, Sq, Sk, D, 768, 128, torch.bfloat16, seed=11 + D)
    g = torch.Generator().manual_seed(12)
    M = gi.shape[2]
    assert B * H * M > 148
    gl = torch.randint(1, 7, (B, H, M), dtype=torch.int32, generator=g)
    residual = (0.1 * torch.randn(B, H, Sq, D, generator=g)).to(torch.bfloat16)
    perm = torch.stack([torch.randperm(Sq, generator=g) for _ in range(B * H)])
    out, lse = _run(cuda_device, q, k, v, gi, gather_kv_lengths=gl, residual=residual, perm=perm)
    ref, ref_lse = gather_attn_ref(q, k, v, gi, gl=gl, residual=residual, perm=perm)
    mx, mr = error_metrics(out, ref)
    assert mx < MAX_ABS and mr < MEAN_REL, (mx, mr)
    assert (lse - ref_lse).abs().max() < 2e-2


def test_clustered_logits_raise_the_maximum_late(cuda_device):
    """Keys ordered so that every row meets its own cluster late: the running maximum rises between tiles."""
    Sq, Sk, D = 128, 2048, 144
    g = torch.Generator().manual_seed(8)
    cent = torch.randn(8, D, generator=g)
    cid_q = torch.randint(0, 8, (Sq,), generator=g)
    cid_k = torch.arange(Sk) * 8 // Sk
    q = (cent[cid_q] + 0.3 * torch.randn(Sq, D, generator=g)).view(1, Sq, 1, D).to(torch.bfloat16)
    k = (cent[cid_k] + 0.3 * torch.randn(Sk, D, generator=g)).view(1, Sk, 1, D).to(torch.bfloat16)
    v = torch.randn(1, Sk, 1, D, generator=g).to(torch.bfloat16)
    gi = torch.arange(Sk, dtype=torch.int32).view(1, 1, 1, Sk)
    out, lse = _run(cuda_device, q, k, v, gi)
    ref, ref_lse = gather_attn_ref(q, k, v, gi)
    mx, mr = error_metrics(out, ref)
    assert mx < MAX_ABS and mr < MEAN_REL, (mx, mr)
    assert (lse - ref_lse).abs().max() < 2e-2


@pytest.mark.parametrize("Lq,Lk,D", [(300, 1000, 144), (130, 70, 96), (200, 513, 256)])
def test_dense_mode(cuda_device, Lq, Lk, D):
    from mcsparse_b200.kernels.flash_mcsa.ops.full_attn import full_attention_with_lse
    B, H = 1, 2
    g = torch.Generator().manual_seed(Lq + Lk)
    q = torch.randn(B, H, Lq, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H, Lk, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, Lk, D, generator=g).to(torch.bfloat16)
    ref, ref_lse = dense_attn_ref(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    out, lse = full_attention_with_lse(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
    mx, mr = error_metrics(out.float().cpu().transpose(1, 2), ref)
    assert mx < MAX_ABS and mr < MEAN_REL, (mx, mr)
    assert float((lse.cpu() - ref_lse).abs().max()) < 2e-3


def test_head_dim_errors(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
    gi = torch.zeros(1, 1, 1, 128, dtype=torch.int32, device=cuda_device)
    for D in (100, 264):          # not a multiple of 8; beyond 256
        x = torch.randn(1, 128, 1, D, device=cuda_device).to(torch.bfloat16)
        with pytest.raises(ValueError):
            flash_attn_gather_kv_func(x, x, x, gi)
