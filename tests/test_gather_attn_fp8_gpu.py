"""GPU parity: FP8-e4m3 gather-KV attention vs the CPU oracle (tolerance: max-abs 6e-2, mean-rel 3e-2)."""

import math

import pytest
import torch

from oracle.gather_attn import error_metrics, gather_attn_fp8_ref

pytestmark = pytest.mark.gpu

FP8_MAX_ABS, FP8_MEAN_REL = 6e-2, 3e-2


def _case(B, H, Sq, Sk, K, seed, clustered=True, D=128):
    from mcsparse_b200.synth import quantize_e4m3_per_head
    g = torch.Generator().manual_seed(seed)
    if clustered:
        cent = torch.randn(H, 16, D, generator=g)
        cq = torch.randint(0, 16, (Sq,), generator=g)
        ck = torch.randint(0, 16, (Sk,), generator=g)
        q = cent[:, cq].permute(1, 0, 2).unsqueeze(0) + 0.3 * torch.randn(B, Sq, H, D, generator=g)
        k = cent[:, ck].permute(1, 0, 2).unsqueeze(0) + 0.3 * torch.randn(B, Sk, H, D, generator=g)
    else:
        q, k = torch.randn(B, Sq, H, D, generator=g), torch.randn(B, Sk, H, D, generator=g)
    v = torch.randn(B, Sk, H, D, generator=g)
    q8, sq = quantize_e4m3_per_head(q)
    k8, sk = quantize_e4m3_per_head(k)
    v8, sv = quantize_e4m3_per_head(v)
    M = math.ceil(Sq / 128)
    gi = torch.stack([torch.cat([torch.arange(4), (torch.randperm(Sk - 4, generator=g)[:K - 4] + 4).sort().values])
                      for _ in range(B * H * M)]).view(B, H, M, K).to(torch.int32)
    scale_qk = (sq * sk * (1.0 / math.sqrt(D)) * math.log2(math.e))[:, :, None].expand(B, H, M).contiguous()
    return q8, k8, v8, gi, scale_qk.float(), sv


@pytest.mark.parametrize("clustered", [True, False])
def test_fp8_matches_oracle(cuda_device, clustered):
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_fp8_func
    q8, k8, v8, gi, sqk, sv = _case(1, 2, 300, 1024, 512, 11, clustered)
    dev = cuda_device
    out, lse = flash_attn_gather_kv_fp8_func(q8.to(dev), k8.to(dev), v8.to(dev), gi.to(dev), sqk.to(dev), sv.to(dev),
                                             return_lse=True)
    assert out.dtype == torch.bfloat16
    ref, ref_lse = gather_attn_fp8_ref(q8, k8, v8, gi, sqk, sv)
    mx, mr = error_metrics(out.float().cpu(), ref)
    assert mx < FP8_MAX_ABS and mr < FP8_MEAN_REL, (mx, mr)
    assert (lse.cpu() - ref_lse).abs().max() < 5e-2


def test_fp8_residual_perm_lengths(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_fp8_func
    q8, k8, v8, gi, sqk, sv = _case(1, 2, 256, 700, 384, 12)
    g = torch.Generator().manual_seed(1)
    res = (0.1 * torch.randn(1, 2, 256, 128, generator=g)).to(torch.bfloat16)
    perm = torch.stack([torch.randperm(256, generator=g) for _ in range(2)])
    gl = torch.tensor([[[3, 2], [1, 3]]], dtype=torch.int32)
    dev = cuda_device
    out, _ = flash_attn_gather_kv_fp8_func(q8.to(dev), k8.to(dev), v8.to(dev), gi.to(dev), sqk.to(dev), sv.to(dev),
                                           gather_kv_lengths=gl.to(dev), residual=res.to(dev), perm=perm.to(dev))
    ref, _ = gather_attn_fp8_ref(q8, k8, v8, gi, sqk, sv, gl=gl, residual=res, perm=perm)
    mx, mr = error_metrics(out.float().cpu(), ref)
    assert mx < FP8_MAX_ABS and mr < FP8_MEAN_REL, (mx, mr)


def test_fp8_argument_errors(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_fp8_func
    q8, k8, v8, gi, sqk, sv = (t.to(cuda_device) for t in _case(1, 2, 128, 256, 128, 13))
    with pytest.raises(TypeError):
        flash_attn_gather_kv_fp8_func(q8.to(torch.bfloat16), k8, v8, gi, sqk, sv)
    with pytest.raises(ValueError):
        flash_attn_gather_kv_fp8_func(q8, k8, v8, gi, sqk[:, :1], sv)
    with pytest.raises(TypeError):
        flash_attn_gather_kv_fp8_func(q8, k8, v8, gi, sqk.double(), sv)


@pytest.mark.parametrize("D", [160, 256, 64])
def test_fp8_other_head_dims(cuda_device, D):
    """The head dimensions other than 128 (the reference's FP8 kernel lists 160, cute/interface.py:358-373) run on the
    kernel that pads rows into shared memory; residual, permutation, ragged last group, 5 key tiles per group."""
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_fp8_func
    B, H, Sq, Sk, K = 1, 2, 300, 1500, 640
    q8, k8, v8, gi, sqk, sv = _case(B, H, Sq, Sk, K, 20 + D, clustered=True, D=D)
    g = torch.Generator().manual_seed(5)
    residual = (0.1 * torch.randn(B, H, Sq, D, generator=g)).to(torch.bfloat16)
    perm = torch.stack([torch.randperm(Sq, generator=g) for _ in range(B * H)])
    dev = cuda_device
    out, lse = flash_attn_gather_kv_fp8_func(q8.to(dev), k8.to(dev), v8.to(dev), gi.to(dev), sqk.to(dev), sv.to(dev),
                                             return_lse=True, residual=residual.to(dev), perm=perm.to(dev))
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16 and out.shape == (B, Sq, H, D)
    ref, ref_lse = gather_attn_fp8_ref(q8, k8, v8, gi, sqk, sv, residual=residual, perm=perm)
    mx, mr = error_metrics(out.float().cpu(), ref)
    assert mx < FP8_MAX_ABS and mr < FP8_MEAN_REL, (D, mx, mr)
    assert (lse.cpu() - ref_lse).abs().max() < 5e-2
    again, _ = flash_attn_gather_kv_fp8_func(q8.to(dev), k8.to(dev), v8.to(dev), gi.to(dev), sqk.to(dev), sv.to(dev),
                                             residual=residual.to(dev), perm=perm.to(dev))
    assert torch.equal(again, out)
