"""CPU (gloo, world_size 2) tests of the Ulysses resharding: sharded == unsharded, error cases on the host."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, B, L, H, D, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mcsparse_b200.h3.context_parallel import UlyssesReshard
        g = torch.Generator().manual_seed(0)
        full = [torch.randn(B, L, H, D, generator=g) for _ in range(3)]         # same on every rank
        Ls, Hl = L // world, H // world
        shard = [t[:, rank * Ls:(rank + 1) * Ls].contiguous() for t in full]
        r = UlyssesReshard(dist.group.WORLD, L, H, D, torch.float32, "cpu", batch=B)
        qh, kh, vh = r.seq_to_head(*shard)
        ok = all(torch.equal(a, t[:, :, rank * Hl:(rank + 1) * Hl]) for a, t in zip((qh, kh, vh), full))
        # "attention" stand-in that mixes the whole sequence of a head: reverse along the sequence
        o = qh.flip(1).contiguous()
        back = r.head_to_seq(o)
        expect = full[0].flip(1)[:, rank * Ls:(rank + 1) * Ls]
        ok = ok and torch.equal(back, expect)
        if B == 1:
            # chunked attention core: per-head "attention" = reverse the sequence and add the head index
            from mcsparse_b200.h3.context_parallel import UlyssesSparseAttention
            ul = UlyssesSparseAttention(dist.group.WORLD, L, H, D, torch.float32, "cpu", chunks=2)

            def attn(qh, kh, vh, h0, h1):
                hidx = torch.arange(rank * Hl + h0, rank * Hl + h1, dtype=torch.float32).view(1, 1, -1, 1)
                return qh.flip(1) + kh + 2 * vh + hidx
            got = ul.forward(*shard, attn)
            hall = torch.arange(H, dtype=torch.float32).view(1, 1, H, 1)
            want = (full[0].flip(1) + full[1] + 2 * full[2] + hall)[:, rank * Ls:(rank + 1) * Ls]
            ok = ok and torch.equal(got, want)
        try:
            UlyssesReshard(dist.group.WORLD, L, H + 1, D, torch.float32, "cpu")
            ok = False
        except ValueError:
            pass
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B", [1, 2])
def test_ulysses_reshard_roundtrip_gloo(B):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, B, 16, 4, 8, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok in res), res


class _Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def _sdpa_bthd(q, k, v):
    return torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)


def _wrapper_worker(rank, world, port, B, L, H, D, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mcsparse_b200.h3 import context_parallel as cp
        g = torch.Generator().manual_seed(1)
        full = [torch.randn(B, L, H, D, generator=g) for _ in range(3)]
        Ls, Hl = L // world, H // world
        shard = [t[:, rank * Ls:(rank + 1) * Ls].contiguous() for t in full]
        pc = _Cfg(context_parallel_config=_Cfg(ulysses_degree=world, ring_degree=1))
        seen = []

        # (1) dense arm through the wrapper's own exchange == unsharded attention, sharded
        d = cp.with_ulysses_sparse(lambda *a, **k: (_ for _ in ()).throw(AssertionError("original dispatch called")),
                                   kind="dense", _dense=_sdpa_bthd, _allow_cpu=True)
        got = d(*shard, parallel_config=pc)
        want = _sdpa_bthd(*full)[:, rank * Ls:(rank + 1) * Ls]
        ok = torch.allclose(got, want, atol=1e-5) and cp.get_cp_stats() == {"cp_calls": 1, "local_calls": 0}

        # (2) sparse arm: the inner dispatch must see full sequences of the LOCAL heads and no parallel_config
        def inner(qh, kh, vh, *a, **kw):
            seen.append((tuple(qh.shape), kw.get("parallel_config")))
            local = qh.shape[2] == Hl
            hidx = torch.arange(rank * Hl if local else 0, (rank + 1) * Hl if local else H, dtype=torch.float32).view(1, 1, -1, 1)
            return qh.flip(1) + 2 * kh + vh + hidx

        d2 = cp.with_ulysses_sparse(lambda *a, **k: None, kind="mcsa_token", _inner_dispatch=inner, _allow_cpu=True)
        got = d2(*shard, parallel_config=pc)
        hall = torch.arange(H, dtype=torch.float32).view(1, 1, H, 1)
        want = (full[0].flip(1) + 2 * full[1] + full[2] + hall)[:, rank * Ls:(rank + 1) * Ls]
        ok = ok and torch.equal(got, want) and seen == [((B, L, Hl, D), None)]
        ok = ok and cp.get_cp_stats() == {"cp_calls": 2, "local_calls": 0}
        # (3) no context-parallel part: runs locally on whatever it is given
        got = d2(*full)
        ok = ok and cp.get_cp_stats()["local_calls"] == 1 and seen[-1] == ((B, L, H, D), None)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B", [1, 2])
def test_with_ulysses_sparse_gloo(B):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_wrapper_worker, args=(r, world, port, B, 16, 4, 8, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok in res), res
