"""GPU: the fused Ulysses path (peer-store scatter in front, attention epilogue that stores each row into the
owning rank's sequence shard) with all ranks emulated in one process on one GPU.

The kernels of this path never wait for another GPU (ranks are ordered between kernels), so running the
ranks' launches one after the other on one device exercises exactly the code an N-GPU job runs; only the
addresses in the peer tables differ.  Checked against the oracle on the unsharded tensors."""

import pytest
import torch

from oracle.gather_attn import error_metrics, gather_attn_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,chunks,with_perm", [(2, 1, False), (2, 2, True), (4, 2, False)])
def test_fused_ulysses_emulated(cuda_device, world, chunks, with_perm):
    from mcsparse_b200 import synth
    from mcsparse_b200.h3.context_parallel import PeerBuffers, UlyssesFusedAttention
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
    dev = cuda_device
    L, H, D, topk = 1024, 8, 128, 256
    Ls, Hl = L // world, H // world
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(1, L, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    res = (0.1 * torch.randn(1, H, L, D, generator=g)).to(torch.bfloat16)
    gi = synth.random_sorted_indices(1, H, L // 128, topk, L, seed=3)
    perm = torch.stack([torch.randperm(L, generator=g) for _ in range(H)]) if with_perm else None
    ref, _ = gather_attn_ref(q, k, v, gi, residual=res, perm=perm)

    qd, kd, vd, resd, gid = (t.to(dev) for t in (q, k, v, res, gi))
    permd = perm.to(dev) if with_perm else None
    hc = Hl // min(chunks, Hl)
    bufs = PeerBuffers.emulated(world, L, Ls, H, hc, Hl // hc, D, torch.bfloat16, dev)
    ranks = [UlyssesFusedAttention(None, L, H, D, torch.bfloat16, dev, chunks=chunks, buffers=bufs[r], rank=r, world=world)
             for r in range(world)]
    shard = lambda t, r: t[:, r * Ls:(r + 1) * Ls].contiguous()
    # phase 1 on every rank: scatter all head chunks (what the communication stream does)
    for r, u in enumerate(ranks):
        for c in range(u.chunks):
            u.scatter_chunk(shard(qd, r), shard(kd, r), shard(vd, r), c)
    torch.cuda.synchronize()
    # the scatter alone must reproduce the head-sharded full-sequence tensors
    for r, u in enumerate(ranks):
        for c in range(u.chunks):
            h0 = r * Hl + c * u.hc
            for i, t in enumerate((qd, kd, vd)):
                assert torch.equal(u.buf.recv[c][i], t[0, :, h0:h0 + u.hc]), (r, c, i)
    # phase 2 on every rank: attention per chunk, rows stored straight into the owners' shards
    for r, u in enumerate(ranks):
        for c in range(u.chunks):
            h0 = r * Hl + c * u.hc
            rc = u.buf.recv[c]
            flash_attn_gather_kv_func(rc[0].unsqueeze(0), rc[1].unsqueeze(0), rc[2].unsqueeze(0), gid[:, h0:h0 + u.hc],
                                      residual=resd[:, h0:h0 + u.hc],
                                      perm=None if permd is None else permd[h0:h0 + u.hc].contiguous(),
                                      out_peers=u.out_peers(c))
    torch.cuda.synchronize()
    out = torch.cat([bufs[r].out for r in range(world)], dim=0).unsqueeze(0).float().cpu()   # (1, L, H, D)
    mx, mr = error_metrics(out, ref)
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)


def test_scatter_and_sharded_argument_checks(cuda_device):
    import ctypes as C
    from mcsparse_b200 import _lib
    L = _lib.lib()
    x = torch.zeros(64, 256, dtype=torch.bfloat16, device=cuda_device)
    ok = (C.c_void_p * 2)(x.data_ptr(), x.data_ptr())
    bad = (C.c_void_p * 2)(x.data_ptr(), 0)
    s = C.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    src = C.c_void_p(x.data_ptr())
    assert L.mcs_ulysses_scatter(src, bad, 2, 0, 4, 256, 256, 512, s) == _lib.MCS_ERR_NULL_POINTER
    assert L.mcs_ulysses_scatter(src, ok, 2, 2, 4, 256, 256, 512, s) == _lib.MCS_ERR_BAD_SHAPE      # rank out of range
    assert L.mcs_ulysses_scatter(src, ok, 2, 0, 4, 250, 256, 512, s) == _lib.MCS_ERR_BAD_ALIGNMENT  # segment not 16-byte
    assert L.mcs_ulysses_scatter(src, ok, 2, 0, 4, 256, 256, 384, s) == _lib.MCS_ERR_BAD_SHAPE      # row too short
    assert L.mcs_ulysses_scatter(src, ok, 17, 0, 4, 256, 256, 8192, s) == _lib.MCS_ERR_BAD_SHAPE    # too many peers
