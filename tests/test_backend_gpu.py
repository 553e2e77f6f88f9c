"""GPU end-to-end: anchor step then reuse steps through the host-side state machine, against the oracle's
composition of the same stages (dense attention, exact mass, selection, sparse attention + residual)."""

import math

import pytest
import torch

from oracle.gather_attn import dense_attn_ref, error_metrics, gather_attn_ref

pytestmark = pytest.mark.gpu


def _qkv(B, H, L, D, seed):
    g = torch.Generator().manual_seed(seed)
    cent = torch.randn(H, 16, D, generator=g)
    cid = torch.randint(0, 16, (L,), generator=g)
    mk = lambda: (cent[:, cid].unsqueeze(0) + 0.3 * torch.randn(B, H, L, D, generator=g)).to(torch.bfloat16)
    return mk(), mk(), torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)


# D = 144 is the second head dimension of the reference's dispatch (token_sparse_dispatch.py:121): every stage of the
# state machine runs on the padded-layout kernels there
@pytest.mark.parametrize("pca,D", [(False, 128), (True, 128), (True, 144), (False, 144), (True, 64), (True, 256)])
def test_calibrate_then_reuse(cuda_device, pca, D):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
    B, H, L = 1, 2, 1500
    cfg = TokenSparseConfig(topk=0.25, calibrate_steps=[0], sink_ranges=[(0, 4)], bias_correction=True, pca_reorder=pca,
                            pca_pow_iters=4)
    ctx = TokenSparseContext(cfg, num_layers=1)
    q, k, v = _qkv(B, H, L, D, 1)
    dev = cuda_device
    # step 0: anchor step returns the dense result
    out0 = ctx.forward(0, q.to(dev), k.to(dev), v.to(dev)).float().cpu()
    dense, _ = dense_attn_ref(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    mx, mr = error_metrics(out0.transpose(1, 2), dense)
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)
    cache = ctx.caches[0]
    gi, gl, perm, res = cache._cached_indices, cache._cached_lengths, cache._cached_perm, cache._cached_residual
    assert gi.shape[-1] % 128 == 0 and (gi[..., :4].cpu() == torch.arange(4)).all() and res is not None
    assert (perm is not None) == pca
    # reuse step on the SAME q/k/v: sparse + cached residual must reproduce the dense output
    ctx.step()
    assert cache.mode == "reuse"
    out1 = ctx.forward(0, q.to(dev), k.to(dev), v.to(dev)).float().cpu()
    mx, mr = error_metrics(out1.transpose(1, 2), dense)
    assert mx < 3e-2 and mr < 1.5e-2, (mx, mr)
    # reuse step on fresh q/k/v: equals the oracle's sparse attention with the cached metadata
    ctx.step()
    q2, k2, v2 = _qkv(B, H, L, D, 2)
    out2 = ctx.forward(0, q2.to(dev), k2.to(dev), v2.to(dev)).float().cpu()
    ref2, _ = gather_attn_ref(q2.transpose(1, 2), k2.transpose(1, 2), v2.transpose(1, 2), gi.cpu(),
                              gl=None if gl is None else gl.cpu(), residual=res.cpu(),
                              perm=None if perm is None else perm.cpu())
    mx, mr = error_metrics(out2.transpose(1, 2), ref2)
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)


def test_topmass_indices_helper(cuda_device):
    from mcsparse_b200 import synth
    from oracle.group_mass import dense_lse_ref, group_mass_ref
    from oracle.select import select_topk_ref
    shape = synth.VideoShape("tiny", 2, (4, 10, 16), (2, 5, 4), topk=256, n_centroids=8)
    q, k, _ = synth.clustered_qkv(shape, device=cuda_device)
    gi = synth.topmass_indices(q, k, shape).cpu()
    qh, kh = q.cpu().transpose(1, 2), k.cpu().transpose(1, 2)
    mass = group_mass_ref(qh, kh, dense_lse_ref(qh, kh).float())
    ref = select_topk_ref(mass.float(), 256, range(4))
    # selection from the kernel's own fp32 mass is exact; against the fp64 oracle mass near-ties may swap
    agree = (gi == ref).float().mean().item()
    assert agree > 0.97, agree


def test_update_step_refreshes_residual(cuda_device):
    """An update step re-selects the tokens from the cached LSE; with bias correction it must also renew the
    residual against a fresh dense pass and return the dense output (reference token_sparse.py:1333-1341), so
    that the next reuse step adds a residual that belongs to the selection it uses."""
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
    B, H, L, D = 1, 2, 1500, 128
    cfg = TokenSparseConfig(topk=0.25, calibrate_steps=[0], update_steps=[1], sink_ranges=[(0, 4)], bias_correction=True,
                            pca_reorder=True, pca_pow_iters=4)
    ctx = TokenSparseContext(cfg, num_layers=1)
    dev = cuda_device
    q, k, v = _qkv(B, H, L, D, 1)
    ctx.forward(0, q.to(dev), k.to(dev), v.to(dev))
    cache = ctx.caches[0]
    gi0, res0, gen0 = cache._cached_indices.clone(), cache._cached_residual.clone(), cache._perm_generation
    ctx.step()
    assert cache.mode == "update"
    q2, k2, v2 = _qkv(B, H, L, D, 2)
    out1 = ctx.forward(0, q2.to(dev), k2.to(dev), v2.to(dev)).float().cpu()
    dense2, _ = dense_attn_ref(q2.transpose(1, 2), k2.transpose(1, 2), v2.transpose(1, 2))
    mx, mr = error_metrics(out1.transpose(1, 2), dense2)
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)                       # the update step returns the dense result
    assert cache._perm_generation == gen0                          # the permutation is kept
    assert not torch.equal(cache._cached_indices, gi0)             # the selection is new
    assert not torch.equal(cache._cached_residual, res0)           # and so is the residual
    # the new residual is dense - sparse(new selection) in group order: a reuse step on the same tensors gives dense
    ctx.step()
    assert cache.mode == "reuse"
    out2 = ctx.forward(0, q2.to(dev), k2.to(dev), v2.to(dev)).float().cpu()
    mx, mr = error_metrics(out2.transpose(1, 2), dense2)
    assert mx < 3e-2 and mr < 1.5e-2, (mx, mr)
    gi, gl, perm = cache._cached_indices.cpu(), cache._cached_lengths, cache._cached_perm.cpu()
    sparse2, _ = gather_attn_ref(q2.transpose(1, 2), k2.transpose(1, 2), v2.transpose(1, 2), gi,
                                 gl=None if gl is None else gl.cpu(), perm=perm)
    want = torch.stack([(dense2 - sparse2)[0, perm[h], h] for h in range(H)]).unsqueeze(0)      # (1,H,L,D) group order
    assert float((cache._cached_residual.float().cpu() - want).abs().max()) < 2e-2


def test_plain_calibrate_returns_sparse_output(cuda_device):
    """Without bias correction an anchor step returns the sparse result (reference token_sparse.py:1290)."""
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
    B, H, L, D = 1, 2, 1024, 128
    cfg = TokenSparseConfig(topk=0.25, calibrate_steps=[0], bias_correction=False, pca_reorder=False)
    ctx = TokenSparseContext(cfg, num_layers=1)
    q, k, v = _qkv(B, H, L, D, 3)
    dev = cuda_device
    out = ctx.forward(0, q.to(dev), k.to(dev), v.to(dev)).float().cpu()
    cache = ctx.caches[0]
    assert cache._cached_residual is None and cache._cached_lengths is None
    ref, _ = gather_attn_ref(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), cache._cached_indices.cpu())
    mx, mr = error_metrics(out.transpose(1, 2), ref)
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)


def test_offloaded_metadata_gives_the_same_results(cuda_device):
    """Indices and residual parked in pinned host memory and prefetched one layer ahead (the reference's
    offload_indices / cache_offload='residual', token_sparse.py:313-487): bit-identical outputs over anchor and reuse
    steps of a three-layer context, every use after the anchor step served by a prefetch."""
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
    B, H, L, D, layers, steps = 1, 2, 1500, 128, 3, 4
    dev = cuda_device
    inputs = [[tuple(t.to(dev) for t in _qkv(B, H, L, D, 10 * s + li)) for li in range(layers)] for s in range(steps)]

    def run(**kw):
        cfg = TokenSparseConfig(topk=0.25, calibrate_steps=[0], sink_ranges=[(0, 4)], bias_correction=True, pca_reorder=True,
                                pca_pow_iters=4, **kw)
        ctx = TokenSparseContext(cfg, num_layers=layers)
        outs = []
        for s in range(steps):
            for li in range(layers):
                outs.append(ctx.forward(li, *inputs[s][li]).clone())
            ctx.step()
        torch.cuda.synchronize()
        return outs, ctx

    base, _ = run()
    off, ctx = run(offload_indices=True, cache_offload="residual")
    assert all(torch.equal(a, b) for a, b in zip(base, off))
    for c in ctx.caches:
        assert c._idx.offloaded and c._res.offloaded and c._idx.gpu is None       # nothing of it stays in HBM between uses
    st = ctx.offload_stats()
    uses = layers * (steps - 1)
    assert st["idx_prefetch_hit"] + st["idx_prefetch_miss"] == uses and st["res_prefetch_hit"] + st["res_prefetch_miss"] == uses
    assert st["idx_prefetch_miss"] == 0 and st["res_prefetch_miss"] == 0, st
    # without prefetching every use is a miss (a copy on the consuming stream), still the same numbers
    off0, ctx0 = run(offload_indices=True, cache_offload="residual", offload_prefetch_ahead=0)
    assert all(torch.equal(a, b) for a, b in zip(base, off0))
    assert ctx0.offload_stats()["idx_prefetch_hit"] == 0 and ctx0.offload_stats()["idx_prefetch_miss"] == uses


def test_compact_index_cache(cuda_device):
    """``compact_indices=True``: the cache holds the packed 17-bit indices and every later step reads them in place."""
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import PackedIndices
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
    B, H, L, D = 1, 2, 1500, 128
    dev = cuda_device
    steps = [tuple(t.to(dev) for t in _qkv(B, H, L, D, 30 + s)) for s in range(3)]

    def run(**kw):
        cfg = TokenSparseConfig(topk=0.25, calibrate_steps=[0], sink_ranges=[(0, 4)], bias_correction=True, pca_reorder=True,
                                pca_pow_iters=4, **kw)
        ctx = TokenSparseContext(cfg, num_layers=1)
        outs = []
        for s in range(3):
            outs.append(ctx.forward(0, *steps[s]).clone())
            ctx.step()
        return outs, ctx

    base, ctx0 = run()
    comp, ctx1 = run(compact_indices=True)
    assert all(torch.equal(a, b) for a, b in zip(base, comp))
    gi = ctx1.caches[0]._cached_indices
    assert isinstance(gi, PackedIndices) and torch.equal(gi.unpack(), ctx0.caches[0]._cached_indices)
