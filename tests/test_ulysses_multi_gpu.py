"""GPU, two or more devices: the fused Ulysses path on REAL peers (symmetric memory, NVLink stores, the two
ordering all-reduces) against the same computation on one GPU, and the ``with_ulysses_sparse`` wrapper through
an anchor step and reuse steps.  Skipped on a single-GPU box."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), MCSPARSE_B200_CHECK="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok, notes = True, []
    try:
        from mcsparse_b200 import _lib, synth
        from mcsparse_b200.h3 import context_parallel as cp
        from mcsparse_b200.h3 import token_sparse_dispatch as tsd
        from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
        L, H, D, topk = 8192, 4 * world, 128, 512
        Ls, Hl = L // world, H // world
        g = torch.Generator(device=dev).manual_seed(3)                     # same seed on every rank: same tensors
        cent = torch.randn(H, 16, D, generator=g, device=dev)
        cid = torch.randint(0, 16, (L,), generator=g, device=dev)
        mk = lambda: (cent[:, cid].permute(1, 0, 2) + 0.3 * torch.randn(L, H, D, generator=g, device=dev)).to(torch.bfloat16).unsqueeze(0)
        qf, kf = mk(), mk()
        vf = torch.randn(1, L, H, D, generator=g, device=dev).to(torch.bfloat16)
        res = (0.1 * torch.randn(1, H, L, D, generator=g, device=dev)).to(torch.bfloat16)
        gi = torch.cat([synth.random_sorted_indices(1, 1, L // 128, topk, L, seed=h, device=dev) for h in range(H)], dim=1)
        shard = lambda t: t[:, rank * Ls:(rank + 1) * Ls].contiguous()
        # ---- (1) fused attention core on real peers == one GPU, bit for bit
        want, _ = flash_attn_gather_kv_func(qf, kf, vf, gi, residual=res)
        for chunks in (1, 2):
            ul = cp.UlyssesFusedAttention(dist.group.WORLD, L, H, D, torch.bfloat16, dev, chunks=chunks)
            h_lo = rank * Hl

            def attn(qh, kh, vh, h0, h1, out_peers):
                flash_attn_gather_kv_func(qh, kh, vh, gi[:, h_lo + h0:h_lo + h1], residual=res[:, h_lo + h0:h_lo + h1],
                                          out_peers=out_peers)
            for _ in range(2):                                               # twice: buffers are reused between steps
                got = ul.forward(shard(qf), shard(kf), shard(vf), attn)
            torch.cuda.synchronize()
            same = torch.equal(got, want[:, rank * Ls:(rank + 1) * Ls])
            ok = ok and same
            notes.append(f"fused chunks={chunks}: {'equal' if same else 'DIFFERENT'}")
        # ---- (2) the wrapper: anchor step (tensor comes back through a library exchange), then reuse steps
        #          (rows stored straight into the owners' shards) == the plain dispatch on one GPU
        dense = cp._make_dense(False)
        orig = lambda q_, k_, v_, *a, **kw: dense(q_, k_, v_)
        common = dict(num_layers=1, topk=0.125, sink_tokens=0, allow_no_sink=True, dense_steps=0, dense_layers="",
                      calibrate_steps=(0,), pca_reorder=True, bias_correction=True, min_seq_len=1024)
        outs_single = []
        d1 = tsd.make_mcsa_token_dispatch(orig, **common)
        for step in range(3):
            tsd.mcsa_token_begin_forward()
            outs_single.append(d1(qf, kf, vf).clone())
        single_stats = tsd.get_mcsa_token_stats()
        cp.reset_cp_stats()
        d2 = cp.with_ulysses_sparse(orig, kind="mcsa_token", **common)
        pc = _Cfg(context_parallel_config=_Cfg(ulysses_degree=world, ring_degree=1))
        for step in range(3):
            tsd.mcsa_token_begin_forward()
            got = d2(shard(qf), shard(kf), shard(vf), parallel_config=pc)
            torch.cuda.synchronize()
            wantw = outs_single[step][:, rank * Ls:(rank + 1) * Ls]
            err = float((got.float() - wantw.float()).abs().max())
            # per-head metadata is computed from the same values on both paths, so the results agree to rounding
            ok = ok and err < 2e-2
            notes.append(f"wrapper step {step}: max diff {err:.2e}")
        st = tsd.get_mcsa_token_stats()
        ok = ok and cp.get_cp_stats() == {"cp_calls": 3, "local_calls": 0} and st["kernel_calls"] == 3 and st["calibrate_calls"] == 1
        ok = ok and single_stats["kernel_calls"] == 3
        # ---- (3) the whole layer on real peers == the same layer on one GPU (rows of this rank), to GEMM rounding
        from mcsparse_b200.h3.ulysses_layer import UlyssesDiTAttentionLayer, layer_weights
        grid, hidden = (8, 16, 64), 1024
        H2 = 2 * world * 2
        w = layer_weights(hidden, H2, D, seed=1, device=dev)
        x = torch.randn(L, hidden, generator=g, device=dev).to(torch.bfloat16)
        gi2 = torch.cat([synth.random_sorted_indices(1, 1, L // 128, topk, L, seed=50 + h, device=dev) for h in range(H2)], dim=1)
        res2 = (0.1 * torch.randn(1, H2, L, D, generator=g, device=dev)).to(torch.bfloat16)
        one = UlyssesDiTAttentionLayer(None, hidden, H2, D, grid, w, dev, heads_per_chunk=2)
        one.set_metadata(gi2, res2)
        want_l = one.forward(x)
        Hl2 = H2 // world
        lay = UlyssesDiTAttentionLayer(dist.group.WORLD, hidden, H2, D, grid, w, dev, heads_per_chunk=2)
        lay.set_metadata(gi2[:, rank * Hl2:(rank + 1) * Hl2].contiguous(), res2[:, rank * Hl2:(rank + 1) * Hl2].contiguous())
        for _ in range(2):
            got_l = lay.forward(x[rank * Ls:(rank + 1) * Ls].contiguous())
        torch.cuda.synchronize()
        dl = (got_l.float() - want_l[rank * Ls:(rank + 1) * Ls].float()).abs()
        rel = float(dl.mean() / want_l.float().abs().mean())
        ok = ok and rel < 1e-2
        notes.append(f"layer: mean-rel diff {rel:.2e}, max {float(dl.max()):.2e}")
        _lib.check_status(dev, "multi-gpu test")
        q.put((rank, bool(ok), notes))
    except Exception as e:                                                    # report instead of hanging the peers
        import traceback
        q.put((rank, False, notes + [traceback.format_exc()]))
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)          # no teardown of symmetric-memory handles and communicators (undefined order between them)


def test_fused_ulysses_on_real_peers():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
    assert all(ok for _, ok, _ in res), res
