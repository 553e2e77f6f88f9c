"""GPU parity: gather-KV attention kernels vs the CPU oracle (through the C ABI)."""

import math

import pytest
import torch

from oracle.gather_attn import error_metrics, gather_attn_ref

pytestmark = pytest.mark.gpu

# tolerances stated for the path: bf16 max-abs 2e-2 / mean-rel 1e-2
BF16_MAX_ABS, BF16_MEAN_REL = 2e-2, 1e-2


def _make(B, H, Sq, Sk, D, gather_len, group_rows, dtype, seed, with_sinks=True, dup=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    k = torch.randn(B, Sk, H, D, generator=g).to(dtype)
    v = torch.randn(B, Sk, H, D, generator=g).to(dtype)
    M = math.ceil(Sq / group_rows)
    gi = torch.empty(B, H, M, gather_len, dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            for m in range(M):
                if dup:
                    gi[b, h, m] = torch.randint(0, Sk, (gather_len,), generator=g, dtype=torch.int32)
                else:
                    n_s = 4 if with_sinks else 0
                    rest = torch.randperm(Sk - n_s, generator=g)[: gather_len - n_s] + n_s
                    gi[b, h, m] = torch.cat([torch.arange(n_s), rest.sort().values]).to(torch.int32)
    return q, k, v, gi


def _run(cuda_device, q, k, v, gi, **kw):
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
    dev = cuda_device
    kw = {kk: (vv.to(dev) if torch.is_tensor(vv) else vv) for kk, vv in kw.items()}
    out, lse = flash_attn_gather_kv_func(q.to(dev), k.to(dev), v.to(dev), gi.to(dev), return_lse=True, **kw)
    torch.cuda.synchronize()
    return out.float().cpu(), lse.cpu()


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_small_exact_shapes(cuda_device, D, dtype):
    q, k, v, gi = _make(1, 2, 256, 512, D, 256, 128, dtype, seed=1)
    out, lse = _run(cuda_device, q, k, v, gi)
    ref, ref_lse = gather_attn_ref(q, k, v, gi)
    mx, mr = error_metrics(out, ref)
    assert mx < BF16_MAX_ABS and mr < BF16_MEAN_REL, (mx, mr)
    assert (lse - ref_lse).abs().max() < 2e-2


def test_ragged_last_group_and_lengths(cuda_device):
    # Sq not a multiple of 128 (last group has 72 rows), per-group tile counts
    q, k, v, gi = _make(2, 3, 328, 700, 128, 384, 128, torch.bfloat16, seed=2)
    M = gi.shape[2]
    gl = torch.randint(1, 4, (2, 3, M), dtype=torch.int32, generator=torch.Generator().manual_seed(3))
    out, lse = _run(cuda_device, q, k, v, gi, gather_kv_lengths=gl)
    ref, ref_lse = gather_attn_ref(q, k, v, gi, gl=gl)
    mx, mr = error_metrics(out, ref)
    assert mx < BF16_MAX_ABS and mr < BF16_MEAN_REL, (mx, mr)
    assert (lse - ref_lse).abs().max() < 2e-2


def test_duplicate_indices(cuda_device):
    q, k, v, gi = _make(1, 2, 256, 300, 128, 256, 128, torch.bfloat16, seed=4, dup=True)
    out, _ = _run(cuda_device, q, k, v, gi)
    ref, _ = gather_attn_ref(q, k, v, gi)
    mx, mr = error_metrics(out, ref)
    assert mx < BF16_MAX_ABS and mr < BF16_MEAN_REL, (mx, mr)


def test_residual_and_perm_fused(cuda_device):
    B, H, Sq, Sk, D = 1, 2, 300, 512, 128
    q, k, v, gi = _make(B, H, Sq, Sk, D, 256, 128, torch.bfloat16, seed=5)
    g = torch.Generator().manual_seed(6)
    residual = (0.1 * torch.randn(B, H, Sq, D, generator=g)).to(torch.bfloat16)
    perm = torch.stack([torch.randperm(Sq, generator=g) for _ in range(B * H)])
    out, lse = _run(cuda_device, q, k, v, gi, residual=residual, perm=perm)
    ref, ref_lse = gather_attn_ref(q, k, v, gi, residual=residual, perm=perm)
    mx, mr = error_metrics(out, ref)
    assert mx < BF16_MAX_ABS and mr < BF16_MEAN_REL, (mx, mr)
    assert (lse - ref_lse).abs().max() < 2e-2


def test_config1_cpu_reference_case(cuda_device):
    """B=1,H=2,L=4096,D=64, 64 groups of 64 queries, 512 indices (4 sinks + 508 sorted), residual, seed 0."""
    torch.manual_seed(0)
    B, H, L, D, G, KS = 1, 2, 4096, 64, 64, 512
    q, k, v = (torch.randn(B, L, H, D) for _ in range(3))
    gi = torch.empty(B, H, L // G, KS, dtype=torch.int32)
    for h in range(H):
        for m in range(L // G):
            rest = (torch.randperm(L - 4)[: KS - 4] + 4).sort().values
            gi[0, h, m] = torch.cat([torch.arange(4), rest]).to(torch.int32)
    residual = 0.1 * torch.randn(B, H, L, D)
    qb, kb, vb, rb = (t.to(torch.bfloat16) for t in (q, k, v, residual))
    out, _ = _run(cuda_device, qb, kb, vb, gi, residual=rb, group_rows=G, softmax_scale=1.0 / 8.0)
    ref, _ = gather_attn_ref(qb, kb, vb, gi, softmax_scale=1.0 / 8.0, residual=rb, group_rows=G)
    mx, mr = error_metrics(out, ref)
    assert mx < BF16_MAX_ABS and mr < BF16_MEAN_REL, (mx, mr)
    # against the fp32 inputs of the config (adds the bf16 input rounding)
    ref32, _ = gather_attn_ref(q, k, v, gi, softmax_scale=1.0 / 8.0, residual=residual, group_rows=G)
    mx32, mr32 = error_metrics(out, ref32)
    assert mx32 < 6e-2 and mr32 < 2e-2, (mx32, mr32)


def test_strided_bhsd_views(cuda_device):
    """BHSD storage viewed as BSHD (no copy) must give the same result."""
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
    q, k, v, gi = _make(1, 2, 256, 384, 128, 256, 128, torch.bfloat16, seed=7)
    dev = cuda_device
    qv, kv, vv = (t.permute(0, 2, 1, 3).contiguous().to(dev).permute(0, 2, 1, 3) for t in (q, k, v))
    assert not qv.is_contiguous()
    out, _ = flash_attn_gather_kv_func(qv, kv, vv, gi.to(dev))
    ref, _ = gather_attn_ref(q, k, v, gi)
    mx, mr = error_metrics(out.float().cpu(), ref)
    assert mx < BF16_MAX_ABS and mr < BF16_MEAN_REL, (mx, mr)


def test_large_logits_rescale_path(cuda_device):
    """Clustered Q/K give large logits whose row max jumps between tiles (exercises the O rescale)."""
    B, H, Sq, Sk, D = 1, 1, 128, 2048, 128
    g = torch.Generator().manual_seed(8)
    cent = torch.randn(8, D, generator=g)
    cid_q = torch.randint(0, 8, (Sq,), generator=g)
    cid_k = torch.arange(Sk) * 8 // Sk     # keys ordered so that each cluster appears late for some rows
    q = (cent[cid_q] + 0.3 * torch.randn(Sq, D, generator=g)).view(1, Sq, 1, D).to(torch.bfloat16)
    k = (cent[cid_k] + 0.3 * torch.randn(Sk, D, generator=g)).view(1, Sk, 1, D).to(torch.bfloat16)
    v = torch.randn(1, Sk, 1, D, generator=g).to(torch.bfloat16)
    gi = torch.arange(Sk, dtype=torch.int32).view(1, 1, 1, Sk)
    out, lse = _run(cuda_device, q, k, v, gi)
    ref, ref_lse = gather_attn_ref(q, k, v, gi)
    mx, mr = error_metrics(out, ref)
    assert mx < BF16_MAX_ABS and mr < BF16_MEAN_REL, (mx, mr)
    assert (lse - ref_lse).abs().max() < 2e-2


def test_late_maxima_repeated_launches_bit_identical(cuda_device):
    """Many rows whose running maximum is raised several times (every raise rescales the output accumulator, half
    of the columns by each of the row's two softmax threads, between two P V products): results within tolerance
    and the same bits on every launch."""
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
    H, Sq, Sk, D = 4, 2048, 4096, 128
    g = torch.Generator().manual_seed(21)
    cent = 1.5 * torch.randn(16, D, generator=g)
    cid_q = torch.randint(0, 16, (Sq,), generator=g)
    cid_k = torch.arange(Sk) * 16 // Sk              # keys in cluster order: each row meets its own cluster late
    q = (cent[cid_q].unsqueeze(1) + 0.3 * torch.randn(Sq, H, D, generator=g)).unsqueeze(0).to(torch.bfloat16)
    k = (cent[cid_k].unsqueeze(1) + 0.3 * torch.randn(Sk, H, D, generator=g)).unsqueeze(0).to(torch.bfloat16)
    v = torch.randn(1, Sk, H, D, generator=g).to(torch.bfloat16)
    gi = torch.arange(0, Sk, 2, dtype=torch.int32).view(1, 1, 1, Sk // 2).expand(1, H, Sq // 128, Sk // 2).contiguous()
    dev = cuda_device
    qd, kd, vd, gd = q.to(dev), k.to(dev), v.to(dev), gi.to(dev)
    out, _ = flash_attn_gather_kv_func(qd, kd, vd, gd)
    torch.cuda.synchronize()
    ref, _ = gather_attn_ref(q, k, v, gi)
    mx, mr = error_metrics(out.float().cpu(), ref)
    assert mx < BF16_MAX_ABS and mr < BF16_MEAN_REL, (mx, mr)
    for _ in range(10):
        again, _ = flash_attn_gather_kv_func(qd, kd, vd, gd)
        assert torch.equal(again, out)


def test_gather_rate_probe_launches(cuda_device):
    """The measurement aid (only the K/V row gather of a launch) accepts the attention call's arguments, touches no
    output and leaves the status word clear."""
    from mcsparse_b200 import _lib
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute.interface import gather_rate_probe
    dev = cuda_device
    q, k, v, gi = (t.to(dev) for t in _make(1, 3, 1000, 2000, 128, 512, 128, torch.bfloat16, seed=12))
    q0 = q.clone()
    gather_rate_probe(q, k, v, gi)
    torch.cuda.synchronize()
    _lib.check_status(dev, "gather_rate_probe")
    assert torch.equal(q, q0)
    with pytest.raises(ValueError):
        gather_rate_probe(q, k, v, gi.long())


def test_argument_errors(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_func, flash_attn_gather_kv_func
    dev = cuda_device
    q, k, v, gi = (t.to(dev) for t in _make(1, 2, 128, 256, 128, 128, 128, torch.bfloat16, seed=9))
    with pytest.raises(TypeError):
        flash_attn_gather_kv_func(q.float(), k.float(), v.float(), gi)
    with pytest.raises(TypeError):
        flash_attn_gather_kv_func(q, k, v, gi.long())
    with pytest.raises(ValueError):
        flash_attn_gather_kv_func(q, k, v, gi[..., :100])
    with pytest.raises(ValueError):
        flash_attn_gather_kv_func(q, k, v, gi[:, :1])
    with pytest.raises(NotImplementedError):
        flash_attn_gather_kv_func(q, k[:, :, :1], v[:, :, :1], gi)
    with pytest.raises(NotImplementedError):
        flash_attn_func(q, k, v, None)
    with pytest.raises(NotImplementedError):
        flash_attn_func(q, k, v, gi, causal=True)
    with pytest.raises(RuntimeError):
        flash_attn_gather_kv_func(q.requires_grad_(True), k, v, gi)


def test_residual_minus_attention(cuda_device):
    """Residual construction in one pass: out = residual - attention (fp32 subtraction, one rounding)."""
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
    from mcsparse_b200 import synth
    B, H, L, D, KS = 1, 2, 640, 128, 256
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(B, L, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    dense = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)
    gi = synth.random_sorted_indices(B, H, L // 128, KS, L, seed=4)
    sparse, _ = gather_attn_ref(q, k, v, gi)
    ref = dense.float().permute(0, 2, 1, 3) - sparse
    out, _ = flash_attn_gather_kv_func(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), gi.to(cuda_device),
                                       residual=dense.to(cuda_device), residual_minus_attention=True)
    mx, mr = error_metrics(out.float().cpu(), ref)
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)
    with pytest.raises(ValueError):
        flash_attn_gather_kv_func(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), gi.to(cuda_device),
                                  residual_minus_attention=True)


@pytest.mark.parametrize("Sk", [3000, 98280])
def test_packed_indices_give_the_same_bits(cuda_device, Sk):
    """17-bit packed indices (16 bits + a bit plane) read by the kernel directly: same output as int32 indices."""
    from mcsparse_b200 import synth
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import PackedIndices, flash_attn_gather_kv_func
    dev = cuda_device
    B, H, Sq, D, KS = 1, 3, 900, 128, 384
    g = torch.Generator().manual_seed(Sk)
    q = torch.randn(B, Sq, H, D, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(B, Sk, H, D, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(B, Sk, H, D, generator=g).to(torch.bfloat16).to(dev)
    M = math.ceil(Sq / 128)
    gi = synth.random_sorted_indices(B, H, M, KS, Sk, seed=1, device=dev)
    if Sk > 65536:
        assert int(gi.max()) > 65535                                   # bit 16 is in use
    gl = torch.randint(1, 4, (B, H, M), generator=g, dtype=torch.int32).to(dev)
    packed = PackedIndices.pack(gi)
    assert packed.nbytes() * 512 == gi.numel() * 4 * 272 and torch.equal(packed.unpack(), gi)
    want, _ = flash_attn_gather_kv_func(q, k, v, gi, gather_kv_lengths=gl)
    got, _ = flash_attn_gather_kv_func(q, k, v, packed, gather_kv_lengths=gl)
    assert torch.equal(got, want)
    # a head slice of the packed form, as the chunked callers take it
    got1, _ = flash_attn_gather_kv_func(q[:, :, 1:3], k[:, :, 1:3], v[:, :, 1:3], packed[:, 1:3], gather_kv_lengths=gl[:, 1:3].contiguous())
    assert torch.equal(got1, want[:, :, 1:3])
    if Sk <= 65536:
        return
    with pytest.raises(ValueError):
        big_k = torch.zeros(B, (1 << 17) + 128, H, D, dtype=torch.bfloat16, device=dev)
        flash_attn_gather_kv_func(q, big_k, big_k, packed)
