"""GPU: the context-parallel DiT attention layer (QKV projection, fused RMSNorm + 3-D RoPE + exchange kernel,
sparse attention with the sharded epilogue, output projection) against the fp32 CPU restatement, on one rank
and with 2 / 4 ranks emulated in one process."""

import math

import pytest
import torch

from oracle.gather_attn import error_metrics
from oracle.ulysses_layer import layer_ref, norm_rope_ref, rope_angles

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (64, torch.bfloat16), (128, torch.float16)])
def test_qkv_epilogue_kernel(cuda_device, D, dtype):
    """RMSNorm + RoPE + scatter of a mix of query / key / value slices, rows offset inside a larger grid."""
    from mcsparse_b200.h3.ulysses_layer import qkv_norm_rope_scatter, rope_table
    dev = cuda_device
    grid = (3, 5, 7)                                     # 105 tokens
    rows, token0, row0 = 61, 37, 11                      # an odd number of slices: the last half-warp runs alone
    kinds = [0, 1, 2, 1, 0, 2, 0]
    n = len(kinds)
    g = torch.Generator().manual_seed(D)
    src = torch.randn(rows, n * D, generator=g).to(dtype)
    gq = 1.0 + 0.1 * torch.randn(D, generator=g)
    gk = 1.0 + 0.1 * torch.randn(D, generator=g)
    pad = 16
    dst = [torch.full((row0 + rows + 3, D + pad), 7.0, dtype=dtype, device=dev) for _ in range(n)]
    qkv_norm_rope_scatter(src.to(dev), [t.data_ptr() for t in dst], [D + pad] * n, kinds, gq.to(dev), gk.to(dev),
                          rope_table(grid, D).to(dev), grid, D, row0=row0, token0=token0)
    torch.cuda.synchronize()
    ang = rope_angles(grid, D)[token0:token0 + rows]
    for s, kind in enumerate(kinds):
        x = src[:, s * D:(s + 1) * D].float()
        want = x if kind == 2 else norm_rope_ref(x.view(rows, 1, D), gq if kind == 0 else gk, ang)[:, 0]
        got = dst[s].cpu().float()
        tol = 2 ** -8 if dtype == torch.bfloat16 else 2 ** -10           # one rounding to the 16-bit type
        assert float((got[row0:row0 + rows, :D] - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), (s, kind)
        # nothing outside the target rows and columns was touched
        assert bool((got[:row0] == 7).all()) and bool((got[row0 + rows:] == 7).all()) and bool((got[:, D:] == 7).all())


def test_qkv_epilogue_argument_errors(cuda_device):
    import ctypes as C
    from mcsparse_b200 import _lib
    from mcsparse_b200.h3.ulysses_layer import qkv_norm_rope_scatter, rope_table
    dev = cuda_device
    grid, D = (2, 2, 4), 128
    src = torch.zeros(16, 2 * D, dtype=torch.bfloat16, device=dev)
    dst = torch.zeros(16, D, dtype=torch.bfloat16, device=dev)
    g = torch.ones(D, device=dev)
    tab = rope_table(grid, D).to(dev)
    ok = dict(gamma_q=g, gamma_k=g, rope_cs=tab, grid=grid, head_dim=D, row0=0, token0=0)
    with pytest.raises(_lib.KernelLaunchError):                              # tokens beyond the grid
        qkv_norm_rope_scatter(src, [dst.data_ptr()] * 2, [D, D], [0, 2], **{**ok, "token0": 8})
    with pytest.raises(_lib.KernelLaunchError):                              # destination rows overlap (stride < D)
        qkv_norm_rope_scatter(src, [dst.data_ptr()] * 2, [64, D], [0, 2], **ok)
    with pytest.raises(_lib.KernelLaunchError):                              # unknown slice kind
        qkv_norm_rope_scatter(src, [dst.data_ptr()] * 2, [D, D], [0, 3], **ok)
    with pytest.raises(ValueError):
        qkv_norm_rope_scatter(src, [dst.data_ptr()], [D], [0], **ok)         # 2 slices per row, one destination
    assert _lib.lib().mcs_qkv_norm_rope_scatter(None, None) == _lib.MCS_ERR_NULL_POINTER


def _layer_case(dev, grid, hidden, H, D, topk, seed=0):
    from mcsparse_b200 import synth
    from mcsparse_b200.h3.ulysses_layer import layer_weights
    L = grid[0] * grid[1] * grid[2]
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(L, hidden, generator=g).to(torch.bfloat16)
    w = layer_weights(hidden, H, D, seed=seed)
    gi = synth.random_sorted_indices(1, H, math.ceil(L / 128), topk, L, seed=seed)
    res = (0.1 * torch.randn(1, H, L, D, generator=g)).to(torch.bfloat16)
    perm = torch.stack([torch.randperm(L, generator=g) for _ in range(H)])
    return L, x, w, gi, res, perm


@pytest.mark.parametrize("world,hc", [(1, 4), (1, 1), (2, 1), (2, 2), (4, 1)])
def test_layer_matches_fp32_restatement(cuda_device, world, hc):
    from mcsparse_b200.h3.context_parallel import PeerBuffers
    from mcsparse_b200.h3.ulysses_layer import UlyssesDiTAttentionLayer
    dev = cuda_device
    grid, hidden, H, D, topk = (4, 12, 16), 512, 4, 128, 256            # 768 tokens, 6 query groups
    L, x, w, gi, res, perm = _layer_case(dev, grid, hidden, H, D, topk)
    ref, q_ref, k_ref, v_ref = layer_ref(x, w, grid, H, D, gi, residual=res, perm=perm, round_to=torch.bfloat16)
    wd = {n: t.to(dev) for n, t in w.items()}
    Ls, Hl = L // world, H // world
    hc = min(hc, Hl)
    bufs = PeerBuffers.emulated(world, L, Ls, H, hc, Hl // hc, D, torch.bfloat16, dev)
    ranks = [UlyssesDiTAttentionLayer(None, hidden, H, D, grid, wd, dev, heads_per_chunk=hc, buffers=bufs[r], rank=r, world=world)
             for r in range(world)]
    for r, lay in enumerate(ranks):
        lay.set_metadata(gi[:, r * Hl:(r + 1) * Hl].to(dev), res[:, r * Hl:(r + 1) * Hl].to(dev),
                         perm[r * Hl:(r + 1) * Hl].to(dev))
    xs = [x[r * Ls:(r + 1) * Ls].contiguous().to(dev) for r in range(world)]
    for r, lay in enumerate(ranks):                                       # phase 1 on every rank
        lay.project_and_scatter(xs[r])
    torch.cuda.synchronize()
    # every rank now holds q, k, v of its heads for ALL tokens: normalised, rotated, in (L, hc, D) per chunk
    for r, lay in enumerate(ranks):
        for c in range(lay.chunks):
            h0 = r * Hl + c * hc
            for got, want in zip(lay.local_qkv(c), (q_ref, k_ref, v_ref)):
                d = (got[0].float().cpu() - want[0, :, h0:h0 + hc]).abs().max()
                assert float(d) < 0.05, (r, c, float(d))                  # bf16 GEMM + one bf16 rounding of O(1) values
    for lay in ranks:                                                     # phase 2
        lay.attend()
    torch.cuda.synchronize()
    out = torch.cat([lay.project_out() for lay in ranks], dim=0).float().cpu()
    mx, mr = error_metrics(out, ref)
    assert mr < 2e-2 and mx < 0.1, (mx, mr)


def test_layer_forward_single_rank_equals_phases(cuda_device):
    """forward() on one rank (streams and events inside) gives the bits of the three phases run one by one."""
    from mcsparse_b200.h3.ulysses_layer import UlyssesDiTAttentionLayer
    dev = cuda_device
    grid, hidden, H, D, topk = (4, 12, 16), 512, 4, 128, 256
    L, x, w, gi, res, perm = _layer_case(dev, grid, hidden, H, D, topk, seed=3)
    wd = {n: t.to(dev) for n, t in w.items()}
    lay = UlyssesDiTAttentionLayer(None, hidden, H, D, grid, wd, dev, heads_per_chunk=1)
    lay.set_metadata(gi.to(dev), res.to(dev), perm.to(dev))
    xd = x.to(dev)
    a = lay.forward(xd).clone()
    b = lay.forward(xd).clone()                                           # buffers reused between calls
    lay.project_and_scatter(xd)
    torch.cuda.synchronize()
    lay.attend()
    c = lay.project_out()
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(a, c)
    f = lay.flops(topk)
    assert f["gemm"] == 2.0 * L * hidden * 4 * H * D and f["attention"] == 4.0 * L * topk * D * H
