"""GPU end-to-end through the drop-in entry point: ``make_mcsa_token_dispatch`` on (B, T, H, D) tensors with the real
kernels behind it, over a schedule with a dense step, a dense layer, an anchor step and reuse steps, with a
conditioning prefix (``sink_tokens``) whose query rows are spliced in from the original dispatch."""

import math

import pytest
import torch

from oracle.gather_attn import dense_attn_ref, error_metrics, gather_attn_ref

pytestmark = pytest.mark.gpu


def _qkv(B, T, H, D, seed):
    g = torch.Generator().manual_seed(seed)
    cent = torch.randn(H, 16, D, generator=g)
    cid = torch.randint(0, 16, (T,), generator=g)
    mk = lambda: (cent[:, cid].permute(1, 0, 2).unsqueeze(0) + 0.3 * torch.randn(B, T, H, D, generator=g)).to(torch.bfloat16)
    return mk(), mk(), torch.randn(B, T, H, D, generator=g).to(torch.bfloat16)


@pytest.mark.parametrize("D", [128, 144])
def test_dispatch_schedule_end_to_end(cuda_device, D):
    from mcsparse_b200.h3 import token_sparse_dispatch as tsd
    dev = cuda_device
    B, T, H, P = 1, 2000, 2, 64
    calls = {"original": 0}

    def original(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
                 attention_kwargs=None, *, backend=None, parallel_config=None):
        # the host model's own attention: a library call in fp32 (an independent implementation)
        calls["original"] += 1
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                                             v.transpose(1, 2).float(), scale=scale)
        return o.transpose(1, 2).to(q.dtype).contiguous()

    d = tsd.make_mcsa_token_dispatch(original, sink_tokens=P, num_layers=2, num_steps=4, topk=0.25, dense_steps=1,
                                     dense_layers="0", calibrate_steps=(1,), min_seq_len=1024, pca_reorder=True,
                                     pca_pow_iters=4, bias_correction=True)
    q, k, v = _qkv(B, T, H, D, 1)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    dense, _ = dense_attn_ref(q, k, v)
    short = torch.randn(B, 77, H, D, device=dev).to(torch.bfloat16)
    for step in range(3):
        tsd.mcsa_token_begin_forward()
        for layer in range(2):
            assert d(short, short, short).shape == short.shape            # the text-length call: original dispatch
            out = d(qd, kd, vd)
            assert out.shape == qd.shape and out.dtype == qd.dtype and out.is_contiguous()
            mx, mr = error_metrics(out.float().cpu(), dense)
            # dense step / dense layer: the original dispatch; anchor and reuse steps on the same tensors: the cached
            # residual makes the sparse result the dense one again (two roundings)
            assert mx < 3e-2 and mr < 1.5e-2, (step, layer, mx, mr)
    s = tsd.get_mcsa_token_stats()
    assert s["dispatch_calls"] == 12 and s["fallback_calls"] == 6
    assert s["dense_guard_calls"] == 4 and s["kernel_calls"] == 2          # step 0 and layer 0 dense; layer 1 at steps 1, 2
    assert s["calibrate_calls"] == 1 and s["splice_calls"] == 2 and s["kernel_error_calls"] == 0
    assert s["seq_len"] == T and s["sink_tokens"] == P and s["layers_per_step"] == 2
    # a reuse step on fresh tensors: prefix rows from the original dispatch, the rest = sparse attention with the cached
    # selection, permutation and residual
    tsd.mcsa_token_begin_forward()
    q2, k2, v2 = _qkv(B, T, H, D, 2)
    d(q2.to(dev), k2.to(dev), v2.to(dev))                                   # layer 0 (dense layer)
    out2 = d(q2.to(dev), k2.to(dev), v2.to(dev)).float().cpu()              # layer 1
    cache = tsd._CTX["ctx"].caches[1]
    gi, gl, perm, res = cache._cached_indices, cache._cached_lengths, cache._cached_perm, cache._cached_residual
    assert bool((gi[..., :P].cpu() == torch.arange(P)).all())               # the prefix keys are always selected
    ref2, _ = gather_attn_ref(q2, k2, v2, gi.cpu(), gl=None if gl is None else gl.cpu(), residual=res.cpu(), perm=perm.cpu())
    dense2, _ = dense_attn_ref(q2, k2, v2)
    mx, mr = error_metrics(out2[:, P:], ref2[:, P:])
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)
    mx, mr = error_metrics(out2[:, :P], dense2[:, :P])
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)
    tsd.reset_mcsa_token_state()
    assert tsd.get_mcsa_token_stats()["dispatch_calls"] == 0


def test_ulysses_wrapper_without_context_parallelism_runs_the_local_kernel(cuda_device):
    """``with_ulysses_sparse`` with no parallel configuration is the plain token-sparse dispatch (reference
    context_parallel.py:201-209): ``local_calls`` counts, the original dispatch only sees what the inner dispatch
    hands it."""
    from mcsparse_b200.h3 import context_parallel as cp, token_sparse_dispatch as tsd
    dev = cuda_device
    B, T, H, D = 1, 1536, 2, 128

    def original(q, k, v, *a, **kw):
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                                             v.transpose(1, 2).float())
        return o.transpose(1, 2).to(q.dtype).contiguous()

    cp.reset_cp_stats()
    d = cp.with_ulysses_sparse(original, kind="mcsa_token", sink_tokens=0, allow_no_sink=True, num_layers=1, topk=0.25,
                               dense_steps=0, dense_layers="", calibrate_steps=(0,), min_seq_len=1024)
    q, k, v = _qkv(B, T, H, D, 3)
    dense, _ = dense_attn_ref(q, k, v)
    for step in range(2):                                  # anchor step, then a reuse step on the same tensors
        tsd.mcsa_token_begin_forward()
        out = d(q.to(dev), k.to(dev), v.to(dev))
        mx, mr = error_metrics(out.float().cpu(), dense)
        assert mx < 3e-2 and mr < 1.5e-2, (step, mx, mr)
    st = cp.get_cp_stats()
    assert st["local_calls"] == 2 and st["cp_calls"] == 0
    assert tsd.get_mcsa_token_stats()["kernel_calls"] == 2
