"""Ulysses context parallelism for the token-sparse attention path.

Sequence-sharded activations (B, L/N, H, D) are resharded to head-sharded full-sequence
tensors (B, L, H/N, D) with one all-to-all, the sparse attention runs on the local heads
with rank-local metadata (indices, residual and permutation are per head, so no metadata
ever crosses ranks), and one all-to-all brings the output back to (B, L/N, H, D).

The reference delegates the two all-to-alls to diffusers'
``_templated_context_parallel_attention`` and runs its kernel as the ``forward_op``
(mcsparse/h3/context_parallel.py:154-231); ring / KV-rotation parallelism is rejected there
(:212-218) and here, because sparse routing needs the whole KV sequence of a head.

Semantics restated (standard Ulysses): sequence shards are concatenated in rank order;
heads are split contiguously in rank order.  Received data lands in this rank's own HBM
buffers and the kernels only ever read local memory.
"""

from __future__ import annotations

import math
from typing import Callable, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

# cp_calls: went through the Ulysses exchange; local_calls: did not (one GPU, or a call that came without a
# context-parallel configuration).  Same two counters as the reference (context_parallel.py:64-73).
_STATS = {"cp_calls": 0, "local_calls": 0}


def get_cp_stats() -> dict:
    return dict(_STATS)


def reset_cp_stats() -> None:
    for k in _STATS:
        _STATS[k] = 0


class UlyssesReshard:
    """Pre-allocated sequence<->head resharding for one attention layer shape.

    ``seq_to_head`` issues all peer transfers of q, k and v as ONE grouped NCCL operation;
    the received tensors are used in place (for B == 1 the receive buffer already is the
    (1, L, H/N, D) tensor the attention kernel wants, so there is no unpack copy).
    """

    def __init__(self, group, seq_len: int, heads: int, head_dim: int, dtype, device, batch: int = 1):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if heads % self.world != 0:
            raise ValueError(f"Ulysses needs heads ({heads}) divisible by the number of ranks ({self.world})")
        if seq_len % self.world != 0:
            raise ValueError(f"Ulysses needs sequence length ({seq_len}) divisible by the number of ranks ({self.world})")
        self.B, self.L, self.H, self.D = batch, seq_len, heads, head_dim
        self.Ls, self.Hl = seq_len // self.world, heads // self.world
        N, B, Ls, Hl, D = self.world, batch, self.Ls, self.Hl, head_dim
        mk = lambda: torch.empty(N, B, Ls, Hl, D, dtype=dtype, device=device)
        self._send = [mk() for _ in range(3)]
        self._recv = [mk() for _ in range(3)]
        self._osend = mk() if B > 1 else None
        self._orecv = mk()
        self.kernels_per_step = 0

    # -- helpers ---------------------------------------------------------------------------
    def _a2a(self, sends: Sequence[torch.Tensor], recvs: Sequence[torch.Tensor]) -> None:
        if self.world == 1:
            for s, r in zip(sends, recvs):
                r.copy_(s)
            return
        if dist.get_backend(self.group) == "nccl":
            ops = []
            for s, r in zip(sends, recvs):
                for peer in range(self.world):
                    g = dist.get_global_rank(self.group, peer)
                    ops.append(dist.P2POp(dist.isend, s[peer], g, self.group))
                    ops.append(dist.P2POp(dist.irecv, r[peer], g, self.group))
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        else:
            for s, r in zip(sends, recvs):
                dist.all_to_all_single(r.view(-1), s.view(-1), group=self.group)

    def _as_bshd(self, buf: torch.Tensor) -> torch.Tensor:
        N, B, Ls, Hl, D = buf.shape
        if B == 1:
            return buf.view(1, N * Ls, Hl, D)
        return buf.permute(1, 0, 2, 3, 4).reshape(B, N * Ls, Hl, D)

    # -- API -------------------------------------------------------------------------------
    def seq_to_head(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, ...]:
        """(B, L/N, H, D) x3 -> (B, L, H/N, D) x3."""
        N, B, Ls, Hl, D = self.world, self.B, self.Ls, self.Hl, self.D
        for t, s in zip((q, k, v), self._send):
            if tuple(t.shape) != (B, Ls, self.H, D):
                raise ValueError(f"expected a sequence shard of shape {(B, Ls, self.H, D)}, got {tuple(t.shape)}")
            s.copy_(t.view(B, Ls, N, Hl, D).permute(2, 0, 1, 3, 4))
        self._a2a(self._send, self._recv)
        return tuple(self._as_bshd(r) for r in self._recv)

    def head_to_seq(self, o: torch.Tensor) -> torch.Tensor:
        """(B, L, H/N, D) -> (B, L/N, H, D)."""
        N, B, Ls, Hl, D = self.world, self.B, self.Ls, self.Hl, self.D
        if tuple(o.shape) != (B, self.L, Hl, D):
            raise ValueError(f"expected a head shard of shape {(B, self.L, Hl, D)}, got {tuple(o.shape)}")
        if B == 1 and o.is_contiguous():
            send = o.view(N, 1, Ls, Hl, D)
        else:
            send = self._osend if self._osend is not None else torch.empty_like(self._orecv)
            send.copy_(o.reshape(B, N, Ls, Hl, D).permute(1, 0, 2, 3, 4))
        self._a2a([send], [self._orecv])
        # received block i holds heads [i*Hl, (i+1)*Hl) of this rank's tokens
        return self._orecv.permute(1, 2, 0, 3, 4).reshape(B, Ls, self.H, D)


class UlyssesSparseAttention:
    """Ulysses attention core with the two all-to-alls overlapped with the attention kernel.

    The local heads are processed in chunks: while the attention kernel works on chunk c (compute stream),
    the all-to-all of chunk c+1 runs on a communication stream, and the reverse all-to-all of finished chunks
    runs on a second communication stream with its own communicator (two NCCL operations of one communicator
    must not run concurrently).  Received data always lands in this rank's own buffers; the attention kernel
    reads them in place through strides (no unpack copy on the way in, no pack copy on the way out for B == 1).

    ``attn_fn(q, k, v, h0, h1)`` gets (1, L, hc, D) tensors of local heads [h0, h1) and returns (1, L, hc, D).
    Replaces the role of diffusers' ``_templated_context_parallel_attention`` in the reference
    (mcsparse/h3/context_parallel.py:220-229) for batch size 1.
    """

    def __init__(self, group, seq_len: int, heads: int, head_dim: int, dtype, device, chunks: int = 3):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if heads % self.world or seq_len % self.world:
            raise ValueError(f"Ulysses needs heads ({heads}) and sequence ({seq_len}) divisible by the ranks ({self.world})")
        self.L, self.H, self.D = seq_len, heads, head_dim
        self.Ls, self.Hl = seq_len // self.world, heads // self.world
        self.chunks = max(1, min(chunks, self.Hl))
        while self.Hl % self.chunks:
            self.chunks -= 1
        self.hc = self.Hl // self.chunks
        N, Ls, hc, D = self.world, self.Ls, self.hc, head_dim
        mk = lambda: torch.empty(N, Ls, hc, D, dtype=dtype, device=device)
        self._send = [[mk() for _ in range(3)] for _ in range(self.chunks)]
        self._recv = [[mk() for _ in range(3)] for _ in range(self.chunks)]
        self._orecv = [mk() for _ in range(self.chunks)]
        self._out = torch.empty(1, Ls, heads, head_dim, dtype=dtype, device=device)
        self.is_cuda = torch.device(device).type == "cuda"
        # second communicator for the reverse direction (every rank must create it)
        self.group_back = dist.new_group(ranks=list(range(self.world))) if self.world > 1 else None
        if self.is_cuda:
            self.s_fwd, self.s_bwd = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.kernels_per_step = 0

    def _a2a(self, sends, recvs, group):
        if self.world == 1:
            for s, r in zip(sends, recvs):
                r.copy_(s)
            return
        if dist.get_backend(group) == "nccl":
            ops = []
            for s, r in zip(sends, recvs):
                for peer in range(self.world):
                    g = dist.get_global_rank(group, peer)
                    ops.append(dist.P2POp(dist.isend, s[peer], g, group))
                    ops.append(dist.P2POp(dist.irecv, r[peer], g, group))
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        else:
            for s, r in zip(sends, recvs):
                dist.all_to_all_single(r.view(-1), s.view(-1), group=group)

    def forward(self, q, k, v, attn_fn):
        """q, k, v: (1, L/N, H, D) sequence shards.  Returns the (1, L/N, H, D) shard of the attention output."""
        N, Ls, Hl, hc, D = self.world, self.Ls, self.Hl, self.hc, self.D
        for t in (q, k, v):
            if tuple(t.shape) != (1, Ls, self.H, D):
                raise ValueError(f"expected a sequence shard of shape {(1, Ls, self.H, D)}, got {tuple(t.shape)}")
        views = [t.view(Ls, N, Hl, D) for t in (q, k, v)]
        out_view = self._out.view(Ls, N, Hl, D)
        if not self.is_cuda:
            for c in range(self.chunks):
                for t, s in zip(views, self._send[c]):
                    s.copy_(t[:, :, c * hc:(c + 1) * hc].permute(1, 0, 2, 3))
                self._a2a(self._send[c], self._recv[c], self.group)
                o = attn_fn(*[r.view(1, N * Ls, hc, D) for r in self._recv[c]], c * hc, (c + 1) * hc)
                self._a2a([o.contiguous().view(N, Ls, hc, D)], [self._orecv[c]], self.group_back or self.group)
                out_view[:, :, c * hc:(c + 1) * hc].copy_(self._orecv[c].permute(1, 0, 2, 3))
            return self._out
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        ev_in = [torch.cuda.Event() for _ in range(self.chunks)]
        ev_attn = [torch.cuda.Event() for _ in range(self.chunks)]
        with torch.cuda.stream(self.s_fwd):
            self.s_fwd.wait_event(ready)
            for c in range(self.chunks):
                for t, s in zip(views, self._send[c]):
                    s.copy_(t[:, :, c * hc:(c + 1) * hc].permute(1, 0, 2, 3))
                self._a2a(self._send[c], self._recv[c], self.group)
                ev_in[c].record(self.s_fwd)
        outs = []
        for c in range(self.chunks):
            main.wait_event(ev_in[c])
            o = attn_fn(*[r.view(1, N * Ls, hc, D) for r in self._recv[c]], c * hc, (c + 1) * hc)
            outs.append(o)
            ev_attn[c].record(main)
            with torch.cuda.stream(self.s_bwd):
                self.s_bwd.wait_event(ev_attn[c])
                self._a2a([o.view(N, Ls, hc, D)], [self._orecv[c]], self.group_back)
                out_view[:, :, c * hc:(c + 1) * hc].copy_(self._orecv[c].permute(1, 0, 2, 3))
        done = torch.cuda.Event()
        done.record(self.s_bwd)
        main.wait_event(done)
        for o in outs:
            o.record_stream(self.s_bwd)
        return self._out


def ulysses_scatter(src: torch.Tensor, dst_ptrs: Sequence[int], rank: int, rows: int, seg_bytes: int,
                    seg_stride_bytes: int, src_row_bytes: int, dma: bool = False) -> None:
    """Launch ``mcs_ulysses_scatter`` on the current stream: segment r of every local row goes to peer r.
    ``dma`` issues the same reshard as strided device copies on the copy engines (``mcs_ulysses_scatter_dma``)."""
    import ctypes as C
    from .. import _lib
    table = (C.c_void_p * len(dst_ptrs))(*[int(x) for x in dst_ptrs])
    stream = torch.cuda.current_stream(src.device).cuda_stream
    fn = _lib.lib().mcs_ulysses_scatter_dma if dma else _lib.lib().mcs_ulysses_scatter
    rc = fn(C.c_void_p(src.data_ptr()), table, len(dst_ptrs), int(rank), int(rows), int(seg_bytes), int(seg_stride_bytes),
            int(src_row_bytes), C.c_void_p(stream))
    _lib.raise_on_error(rc, f"mcs_ulysses_scatter{'_dma' if dma else ''}")


class PeerBuffers:
    """Peer-mapped buffers of the fused Ulysses path for one rank.

    ``recv[c]`` is this rank's (3, L, hc, D) buffer for head chunk c (q, k, v of hc local heads, all tokens),
    ``out`` its (Ls, H, D) sequence shard of the output; ``recv_ptrs[c][r]`` / ``out_ptrs[r]`` are the
    addresses under which THIS process can store into rank r's copies.  In a real job they come from
    ``torch.distributed._symmetric_memory`` (:meth:`symmetric`); a single process can emulate all ranks on
    one GPU with plain tensors (:meth:`emulated`), which is how the kernels are tested without N GPUs.
    """

    def __init__(self, recv, out, recv_ptrs, out_ptrs, keep=None):
        self.recv, self.out, self.recv_ptrs, self.out_ptrs, self._keep = recv, out, recv_ptrs, out_ptrs, keep

    @staticmethod
    def symmetric(group, world, L, Ls, H, hc, chunks, D, dtype, device) -> "PeerBuffers":
        import torch.distributed._symmetric_memory as symm_mem
        recv, recv_ptrs, keep = [], [], []
        for _ in range(chunks):
            t = symm_mem.empty((3, L, hc, D), dtype=dtype, device=device)
            h = symm_mem.rendezvous(t, group)
            recv.append(t)
            recv_ptrs.append([int(h.buffer_ptrs[r]) for r in range(world)])
            keep.append(h)
        out = symm_mem.empty((Ls, H, D), dtype=dtype, device=device)
        ho = symm_mem.rendezvous(out, group)
        keep.append(ho)
        return PeerBuffers(recv, out, recv_ptrs, [int(ho.buffer_ptrs[r]) for r in range(world)], keep)

    @staticmethod
    def emulated(world, L, Ls, H, hc, chunks, D, dtype, device) -> list:
        """Buffers of all ``world`` ranks in this process (one GPU)."""
        recv = [[torch.empty(3, L, hc, D, dtype=dtype, device=device) for _ in range(chunks)] for _ in range(world)]
        out = [torch.empty(Ls, H, D, dtype=dtype, device=device) for _ in range(world)]
        recv_ptrs = [[recv[r][c].data_ptr() for r in range(world)] for c in range(chunks)]
        out_ptrs = [out[r].data_ptr() for r in range(world)]
        return [PeerBuffers(recv[r], out[r], recv_ptrs, out_ptrs) for r in range(world)]


class UlyssesFusedAttention:
    """Ulysses attention core on peer memory, for batch size 1.

    Forward reshard: one ``mcs_ulysses_scatter`` launch per tensor pushes the head slices of the local
    sequence shard into the peers' (L, heads, D) buffers with NVLink stores (no pack copy, no library
    all-to-all).  Backward reshard: none as a separate step - the attention kernel's epilogue stores every
    finished row straight into the sequence shard of the rank that owns its token
    (``mcs_gather_attn_fwd_sharded``).  The local heads are processed in chunks so that the scatter of
    chunk c+1 (communication stream) runs under the attention of chunk c.  Kernels of different ranks are
    ordered by two stream-ordered one-element all-reduces per step (one per chunk in front of the
    attention, one behind the last attention); no kernel ever waits for another GPU.

    ``attn_fn(q, k, v, h0, h1, out_peers)`` gets (1, L, hc, D) tensors of local heads [h0, h1) and must call
    the attention with ``out_peers=out_peers``.  Replaces diffusers'
    ``_templated_context_parallel_attention`` around the reference's forward_op
    (mcsparse/h3/context_parallel.py:220-229).
    """

    def __init__(self, group, seq_len: int, heads: int, head_dim: int, dtype, device, chunks: int = 2,
                 buffers: Optional[PeerBuffers] = None, rank: Optional[int] = None, world: Optional[int] = None,
                 dma_from_chunk: Optional[int] = 1):
        # head chunks from this one on are exchanged by the copy engines: they move while the attention of
        # an earlier chunk owns the SMs, where a scatter kernel could not become resident.  Chunk 0 has
        # the GPU to itself and uses the kernel.  None: the kernel for every chunk.
        self.dma_from_chunk = dma_from_chunk
        self.group = group
        self.world = world if world is not None else dist.get_world_size(group)
        self.rank = rank if rank is not None else dist.get_rank(group)
        if heads % self.world or seq_len % self.world:
            raise ValueError(f"Ulysses needs heads ({heads}) and sequence ({seq_len}) divisible by the ranks ({self.world})")
        self.L, self.H, self.D = seq_len, heads, head_dim
        self.Ls, self.Hl = seq_len // self.world, heads // self.world
        self.chunks = max(1, min(chunks, self.Hl))
        while self.Hl % self.chunks:
            self.chunks -= 1
        self.hc = self.Hl // self.chunks
        self.esize = torch.empty(0, dtype=dtype).element_size()
        if (self.hc * head_dim * self.esize) % 16:
            raise ValueError("a head chunk of one token must be a multiple of 16 bytes")
        self.emulated = buffers is not None
        self.buf = buffers if buffers is not None else PeerBuffers.symmetric(
            group, self.world, self.L, self.Ls, self.H, self.hc, self.chunks, self.D, dtype, device)
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.flag_back = torch.zeros(1, dtype=torch.float32, device=device)
        self.group_back = None
        if not self.emulated and self.world > 1:
            self.group_back = dist.new_group(ranks=list(range(self.world)))
        self.s_comm = torch.cuda.Stream(device)

    def _order(self, flag, group):
        """Orders the kernels enqueued so far on every rank before what follows on this stream."""
        if not self.emulated and self.world > 1:
            dist.all_reduce(flag, group=group)

    def scatter_chunk(self, q, k, v, c: int) -> None:
        """Pushes head chunk c of this rank's q, k, v shards to all peers (current stream)."""
        dma = self.dma_from_chunk is not None and c >= self.dma_from_chunk
        D, hc, Hl, H, es = self.D, self.hc, self.Hl, self.H, self.esize
        seg, seg_stride, row = hc * D * es, Hl * D * es, H * D * es
        plane = self.L * hc * D * es                       # bytes of one of q / k / v inside recv[c]
        for i, t in enumerate((q, k, v)):
            src = t.view(self.Ls, H, D)[:, c * hc:, :]     # chunk c of rank 0's heads; peers follow at seg_stride
            ulysses_scatter(src, [p + i * plane for p in self.buf.recv_ptrs[c]], self.rank, self.Ls, seg, seg_stride, row, dma=dma)

    def out_peers(self, c: int):
        """(pointers, rows per peer, strides) for the attention of head chunk c."""
        off = (self.rank * self.Hl + c * self.hc) * self.D * self.esize
        return ([p + off for p in self.buf.out_ptrs], self.Ls, (self.Ls * self.H * self.D, self.H * self.D, self.D))

    def forward(self, q, k, v, attn_fn):
        """q, k, v: (1, L/N, H, D) sequence shards.  Returns this rank's (1, L/N, H, D) output shard."""
        for t in (q, k, v):
            if tuple(t.shape) != (1, self.Ls, self.H, self.D) or not t.is_contiguous():
                raise ValueError(f"expected a contiguous sequence shard of shape {(1, self.Ls, self.H, self.D)}")
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        ev = [torch.cuda.Event() for _ in range(self.chunks)]
        with torch.cuda.stream(self.s_comm):
            self.s_comm.wait_event(ready)
            for c in range(self.chunks):
                self.scatter_chunk(q, k, v, c)
                self._order(self.flag, self.group)
                ev[c].record(self.s_comm)
        for c in range(self.chunks):
            main.wait_event(ev[c])
            r = self.buf.recv[c]
            attn_fn(r[0].unsqueeze(0), r[1].unsqueeze(0), r[2].unsqueeze(0), c * self.hc, (c + 1) * self.hc, self.out_peers(c))
        self._order(self.flag_back, self.group_back)
        return self.buf.out.unsqueeze(0)

    def capture(self, q, k, v, attn_fn):
        """Captures one forward (both streams, the ordering collectives included) into a CUDA graph.

        A forward is a dozen short launches on two streams; replaying them as one graph takes the host out of
        the step, which is what lets the scatter of one head chunk actually run under the attention of the
        previous one.  Returns (graph, output shard); ``graph.replay()`` recomputes the output from the
        current contents of q, k, v (same tensors)."""
        self.forward(q, k, v, attn_fn)          # eager once: communicators and lazy initialisation
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.forward(q, k, v, attn_fn)
        return graph, out


# =====================================================================================================
# with_ulysses_sparse: the dispatch wrapper of the reference (context_parallel.py:154-231)
# =====================================================================================================
def _make_dense(fa3: bool) -> Callable:
    """Dense attention on BTHD tensors used by the sparse dispatch for its full layers / steps.  The
    reference chooses between FA3 and SDPA by ``fa3`` (context_parallel.py:76-88); here both spell this
    package's dense mode, which accepts different query and key lengths."""
    def dense(q, k, v):
        from mcsparse_b200.kernels.flash_mcsa.ops.full_attn import full_attention
        return full_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).contiguous()
    return dense


def _make_kernel(kind: str, cfg: dict, dense: Callable) -> Callable:
    """The attention itself on full-sequence, head-local BTHD tensors: ``kernel(q, k, v, out_peers=None)``.

    "mcsa_token" builds the token-sparse dispatch with the original dispatch replaced by ``dense``;
    "dense" routes the dense arm through the same exchange (context_parallel.py:91-151)."""
    if kind == "mcsa_token":
        from mcsparse_b200.h3 import token_sparse_dispatch as tsd
        inner = cfg.get("_inner_dispatch")
        if inner is None:
            known = ("sink_tokens", "num_layers", "num_steps", "topk", "dense_steps", "dense_layers", "calibrate_every",
                     "calibrate_steps", "pca_reorder", "pca_pow_iters", "pca_proj_dim", "bias_correction", "selection_mode",
                     "topp", "adaptive_layers", "use_chunk_selector", "chunk_selector_size", "offload_indices",
                     "cache_offload", "offload_prefetch_ahead", "update_steps", "approx_steps", "full_attn_impl",
                     "allow_no_sink", "min_seq_len", "ticks_per_step", "cfg_slots")
            kw = {k: cfg[k] for k in known if k in cfg}
            inner = tsd.make_mcsa_token_dispatch(lambda q, k, v, *a, **k2: dense(q, k, v), **kw)

        def kernel(q, k, v, out_peers=None):
            # parallel_config=None on purpose: past the exchange this is an ordinary full-sequence problem
            if out_peers is None:
                return inner(q, k, v, None, 0.0, False, None, False, None, backend=None, parallel_config=None)
            return inner(q, k, v, None, 0.0, False, None, False, None, backend=None, parallel_config=None,
                         out_peers=out_peers)
        return kernel
    if kind == "dense":
        def kernel(q, k, v, out_peers=None):
            return dense(q, k, v)
        return kernel
    raise ValueError(f"kind must be 'mcsa_token' or 'dense'; got {kind!r}")


def _cp_group(cp):
    """Process group of the Ulysses dimension of a context-parallel configuration (diffusers keeps a device
    mesh on it; a plain ``ulysses_group`` attribute is accepted as well), default: the world."""
    g = getattr(cp, "ulysses_group", None)
    if g is not None:
        return g
    mesh = getattr(cp, "_ulysses_mesh", None)
    if mesh is not None and hasattr(mesh, "get_group"):
        return mesh.get_group()
    return dist.group.WORLD


class UlyssesRoute:
    """Runs ``kernel`` between the two reshards for one (shape, group); built on first use.

    CUDA, batch 1, 16-bit tensors and peer-mappable memory: the fused path (``UlyssesFusedAttention``) -
    scatter kernel in front, and when the kernel call ends in the sparse attention its epilogue stores
    the rows straight into the owners' shards; a call that returns a tensor instead (anchor step, dense
    layer) is brought back by a library all-to-all.  Everything else (CPU tensors under gloo, batches):
    ``UlyssesReshard`` with library all-to-alls on both sides."""

    def __init__(self, group, q: torch.Tensor, fused: Optional[bool] = None):
        B, Ls, H, D = q.shape
        self.group = group
        self.world = dist.get_world_size(group)
        self.shape = (B, Ls, H, D, q.dtype, q.device)
        L = Ls * self.world
        self.reshard = UlyssesReshard(group, L, H, D, q.dtype, q.device, batch=B)
        can_fuse = q.is_cuda and B == 1 and q.dtype in (torch.bfloat16, torch.float16) and self.world > 1
        self.fused = None
        if can_fuse and fused is not False:
            try:
                self.fused = UlyssesFusedAttention(group, L, H, D, q.dtype, q.device, chunks=1, dma_from_chunk=None)
            except Exception:
                if fused:
                    raise
                self.fused = None

    def run(self, kernel: Callable, q, k, v):
        if self.fused is None:
            qh, kh, vh = self.reshard.seq_to_head(q.contiguous(), k.contiguous(), v.contiguous())
            return self.reshard.head_to_seq(kernel(qh, kh, vh).contiguous())
        u = self.fused
        stored = []

        def attn(qh, kh, vh, h0, h1, out_peers):
            o = kernel(qh, kh, vh, out_peers=out_peers)
            stored.append(o)

        out = u.forward(q.contiguous(), k.contiguous(), v.contiguous(), attn)
        if stored and stored[0] is not None:
            # the kernel returned a head-sharded tensor (anchor step, dense layer): library exchange back
            return self.reshard.head_to_seq(stored[0].contiguous())
        return out


def with_ulysses_sparse(original_dispatch: Callable, *, kind: str, fa3: bool = False, **cfg) -> Callable:
    """Wrap an attention dispatch so that the sparse kernel runs after the Ulysses exchange.

    Same contract as the reference's wrapper (context_parallel.py:154-231): unsupported arguments go to
    ``original_dispatch`` untouched; without a ``parallel_config`` (or without a context-parallel part in
    it) the kernel runs locally and ``local_calls`` counts; ``ring_degree > 1`` raises ``ValueError``
    because no rank ever holds a whole KV sequence under ring attention; with Ulysses the sequence shards
    are exchanged for head shards, the kernel runs on full sequences of the local heads with rank-local
    metadata, and the result returns to sequence shards (``cp_calls``).  The reference hands its kernel to
    diffusers' ``_templated_context_parallel_attention`` as ``forward_op``; this wrapper owns the exchange
    (:class:`UlyssesRoute`).  ``cfg`` are the arguments of ``make_mcsa_token_dispatch``; ``fused`` (True /
    False / None = decide by device) picks the exchange implementation.
    """
    fused = cfg.pop("fused", None)
    dense = cfg.pop("_dense", None) or _make_dense(fa3)
    kernel = _make_kernel(kind, cfg, dense)
    routes: dict = {}

    def forward_op(ctx, query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
                   return_lse=False, _save_ctx=True, _parallel_config=None):
        """The kernel in the calling convention of a diffusers context-parallel forward op, for a caller that
        drives the exchange itself (context_parallel.py:165-176)."""
        if return_lse:
            raise ValueError("sparse CP forward_op produces no LSE, so it cannot serve ring attention. "
                             "Use ulysses_degree with ring_degree=1.")
        _STATS["cp_calls"] += 1
        return kernel(query.contiguous(), key.contiguous(), value.contiguous())

    def dispatch(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
                 attention_kwargs=None, *, backend=None, parallel_config=None):
        supported = (attn_mask is None and not is_causal and dropout_p == 0.0 and not enable_gqa
                     and getattr(query, "ndim", 0) == 4
                     and (scale is None or math.isclose(float(scale), 1.0 / math.sqrt(query.shape[-1])))
                     and tuple(query.shape) == tuple(key.shape) == tuple(value.shape)
                     and (bool(getattr(query, "is_cuda", False)) or cfg.get("_allow_cpu", False)))
        if not supported:
            return original_dispatch(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa,
                                     attention_kwargs, backend=backend, parallel_config=parallel_config)
        cp = None if parallel_config is None else getattr(parallel_config, "context_parallel_config", None)
        if cp is None:
            _STATS["local_calls"] += 1
            return kernel(query.contiguous(), key.contiguous(), value.contiguous())
        if getattr(cp, "ring_degree", 1) > 1:
            raise ValueError(f"ring_degree={cp.ring_degree}: ring attention hands each rank rotating KV chunks, so a "
                             "sparse kernel never sees a whole KV sequence and its routing would be wrong. "
                             "Use ulysses_degree instead.")
        if getattr(cp, "ulysses_degree", 1) <= 1:
            _STATS["local_calls"] += 1
            return kernel(query.contiguous(), key.contiguous(), value.contiguous())
        group = _cp_group(cp)
        key_ = (tuple(query.shape), query.dtype, str(query.device), id(group))
        route = routes.get(key_)
        if route is None:
            route = routes[key_] = UlyssesRoute(group, query, fused=fused)
        _STATS["cp_calls"] += 1
        return route.run(kernel, query, key, value)

    dispatch.forward_op = forward_op
    return dispatch


__all__ = ["get_cp_stats", "reset_cp_stats", "with_ulysses_sparse", "UlyssesReshard", "UlyssesSparseAttention",
           "UlyssesFusedAttention", "UlyssesRoute", "PeerBuffers", "ulysses_scatter"]
