"""A context-parallel DiT attention layer around the token-sparse attention: QKV projection, RMSNorm on q and
k, 3-D rotary embedding, Ulysses exchange, sparse attention with reused metadata, exchange back, output
projection.  This is the workload of the multi-GPU benchmark configuration (hidden 5120, 40 heads x 128,
21 x 72 x 65 latent grid, tokens sharded evenly over the ranks).

The reference enters this layer only at the attention call: the host model does the projections, the
normalisation and the rotary embedding, diffusers' ``_templated_context_parallel_attention`` does the two
all-to-alls, and the reference's ``forward_op`` (mcsparse/h3/context_parallel.py:165-176) is the kernel in
between.  Here the stretch from the projection output to the attention input is ONE kernel per head chunk
(``mcs_qkv_norm_rope_scatter``): it normalises, rotates and stores every head slice straight into the (L, heads,
D) buffer of the rank that owns the head, over NVLink, while the projection GEMM of the next head chunk runs.
The way back is the attention kernel's own epilogue (``mcs_gather_attn_fwd_sharded``).  The projections are
library GEMMs (``torch.matmul``): they are sequence-sharded, exchange nothing and are not part of the path this
package accelerates; what matters is that the exchange hides behind them.

Definitions (fixed here because the checkpoint of the host model is not available; they follow common video-DiT
practice): RMSNorm over the head dimension with a learned weight per element, applied to q and k before the
rotation; rotary pairs are (2p, 2p+1); of the D/2 pairs the last 2*(D//6) are split evenly between grid row and
grid column and the rest follow the frame index; pair i of an axis with n pairs turns by position * theta^(-i/n),
theta = 10000.
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from mcsparse_b200 import _lib
from mcsparse_b200.h3.context_parallel import PeerBuffers


def rope_pairs(head_dim: int) -> Tuple[int, int, int]:
    """Rotation pairs per axis (frame, row, column)."""
    per = head_dim // 6
    return head_dim // 2 - 2 * per, per, per


def rope_table(grid: Tuple[int, int, int], head_dim: int, theta: float = 10000.0) -> torch.Tensor:
    """(F + H + W, D/2, 2) fp32 table of (cos, sin): row = axis offset + position, column = rotation pair.
    Only the columns of an axis' own pairs are meaningful in its rows."""
    F, Hh, W = grid
    n_t, n_h, n_w = rope_pairs(head_dim)
    tab = torch.zeros(F + Hh + W, head_dim // 2, 2, dtype=torch.float64)
    tab[..., 0] = 1.0
    row0, col0 = 0, 0
    for size, n in ((F, n_t), (Hh, n_h), (W, n_w)):
        if n > 0:
            freq = theta ** (-torch.arange(n, dtype=torch.float64) / n)
            ang = torch.arange(size, dtype=torch.float64)[:, None] * freq[None, :]
            tab[row0:row0 + size, col0:col0 + n, 0] = torch.cos(ang)
            tab[row0:row0 + size, col0:col0 + n, 1] = torch.sin(ang)
        row0 += size
        col0 += n
    return tab.float().contiguous()


def qkv_norm_rope_scatter(src: torch.Tensor, dst_ptrs: Sequence[int], dst_row_strides: Sequence[int], kinds: Sequence[int],
                          gamma_q: torch.Tensor, gamma_k: torch.Tensor, rope_cs: torch.Tensor, grid: Tuple[int, int, int],
                          head_dim: int, row0: int, token0: int, eps: float = 1e-6) -> None:
    """Launch ``mcs_qkv_norm_rope_scatter`` on the current stream.  ``src``: (rows, n_seg * head_dim) 16-bit CUDA tensor
    with contiguous rows; slice s of row i goes to ``dst_ptrs[s] + (row0 + i) * dst_row_strides[s]`` elements."""
    if src.dim() != 2 or src.stride(1) != 1:
        raise ValueError("src must be (rows, n_seg * head_dim) with contiguous rows")
    n = len(dst_ptrs)
    if not (len(dst_row_strides) == len(kinds) == n) or src.shape[1] != n * head_dim:
        raise ValueError("one destination, stride and kind per head slice of a row")
    if src.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("src must be bf16 or fp16")
    n_t, n_h, _ = rope_pairs(head_dim)
    a = _lib.QkvEpilogueArgs()
    a.src, a.gamma_q, a.gamma_k, a.rope_cs = src.data_ptr(), gamma_q.data_ptr(), gamma_k.data_ptr(), rope_cs.data_ptr()
    dst = (C.c_void_p * n)(*[int(x) for x in dst_ptrs])
    strides = (C.c_int64 * n)(*[int(x) for x in dst_row_strides])
    kind = (C.c_int32 * n)(*[int(x) for x in kinds])
    a.dst, a.dst_row_stride, a.kind = dst, strides, kind
    a.src_row_stride, a.rows, a.row0, a.token0 = src.stride(0), src.shape[0], int(row0), int(token0)
    a.n_seg, a.D = n, head_dim
    a.grid_f, a.grid_h, a.grid_w = grid
    a.pairs_t, a.pairs_h = n_t, n_h
    a.dtype = _lib.MCS_DTYPE_BF16 if src.dtype == torch.bfloat16 else _lib.MCS_DTYPE_FP16
    a.eps = float(eps)
    stream = torch.cuda.current_stream(src.device).cuda_stream
    _lib.raise_on_error(_lib.lib().mcs_qkv_norm_rope_scatter(C.byref(a), C.c_void_p(stream)), "mcs_qkv_norm_rope_scatter")
    if _lib.check_enabled():
        _lib.check_status(src.device, "qkv_norm_rope_scatter")


def layer_weights(hidden: int, heads: int, head_dim: int, seed: int = 0, device="cpu", dtype=torch.bfloat16):
    """Random-init weights of the layer, the same on every rank: Wq, Wk, Wv (H*D, hidden), Wo (hidden, H*D) ~
    N(0, 1/hidden) resp. N(0, 1/(H*D)); RMSNorm weights around 1."""
    g = torch.Generator(device="cpu").manual_seed(seed * 9176 + 5)
    HD = heads * head_dim
    mk = lambda o, i: (torch.randn(o, i, generator=g) / math.sqrt(i)).to(dtype).to(device)
    w = {"wq": mk(HD, hidden), "wk": mk(HD, hidden), "wv": mk(HD, hidden), "wo": mk(hidden, HD)}
    w["gq"] = (1.0 + 0.1 * torch.randn(head_dim, generator=g)).float().to(device)
    w["gk"] = (1.0 + 0.1 * torch.randn(head_dim, generator=g)).float().to(device)
    return w


class UlyssesDiTAttentionLayer:
    """One attention layer of a sequence-sharded DiT, for batch size 1.

    ``forward(x)`` takes this rank's (L/N, hidden) activations and returns its (L/N, hidden) share of the layer
    output.  The local heads are processed in chunks of ``heads_per_chunk``; chunk c of EVERY rank is projected by
    one GEMM, so each chunk's exchange runs under the GEMM of the next chunk and the attention kernels start when
    the projections are through.  The attention metadata (indices, residual, optional permutation) is per local
    head and set by :meth:`set_metadata`.

    With ``buffers`` / ``rank`` / ``world`` given the peers are plain tensors of this process (all ranks emulated on
    one GPU, phases driven by the caller: :meth:`project_and_scatter`, :meth:`attend`, :meth:`project_out`); the
    kernels and their arguments are the ones an N-GPU job runs.
    """

    def __init__(self, group, hidden: int, heads: int, head_dim: int, grid: Tuple[int, int, int], weights: dict, device,
                 dtype=torch.bfloat16, heads_per_chunk: int = 1, buffers: Optional[PeerBuffers] = None,
                 rank: Optional[int] = None, world: Optional[int] = None, eps: float = 1e-6):
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if group is not None else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if group is not None else 0)
        N = self.world
        self.hidden, self.H, self.D, self.grid, self.eps, self.dtype = hidden, heads, head_dim, tuple(grid), eps, dtype
        self.L = grid[0] * grid[1] * grid[2]
        if heads % N or self.L % N:
            raise ValueError(f"Ulysses needs heads ({heads}) and sequence ({self.L}) divisible by the ranks ({N})")
        self.Ls, self.Hl = self.L // N, heads // N
        hc = max(1, min(heads_per_chunk, self.Hl))
        while self.Hl % hc:
            hc -= 1
        if 3 * N * hc > 128:
            raise ValueError("too many head slices per chunk for one epilogue launch (3 * ranks * heads_per_chunk <= 128)")
        self.hc, self.chunks = hc, self.Hl // hc
        D, es = head_dim, 2
        self.emulated = buffers is not None
        if buffers is not None:
            self.buf = buffers
        elif N == 1:
            self.buf = PeerBuffers.emulated(1, self.L, self.Ls, heads, hc, self.chunks, D, dtype, device)[0]
        else:
            self.buf = PeerBuffers.symmetric(group, N, self.L, self.Ls, heads, hc, self.chunks, D, dtype, device)
        # projection weights of chunk c: rows ordered (q | k | v) x (destination rank) x (head inside the chunk)
        wq, wk, wv = (weights[n].view(heads, D, hidden) for n in ("wq", "wk", "wv"))
        self.w_chunk: List[torch.Tensor] = []
        for c in range(self.chunks):
            hs = [r * self.Hl + c * hc + j for r in range(N) for j in range(hc)]
            self.w_chunk.append(torch.cat([w[hs].reshape(-1, hidden) for w in (wq, wk, wv)], dim=0).contiguous())
        self.wo = weights["wo"]
        self.gq, self.gk = weights["gq"].float().contiguous(), weights["gk"].float().contiguous()
        self.rope = rope_table(self.grid, D).to(device)
        plane = self.L * hc * D * es                   # bytes of one of q / k / v inside recv[c]
        self.seg: List[Tuple[list, list, list]] = []
        for c in range(self.chunks):
            ptrs, strides, kinds = [], [], []
            for kind in range(3):
                for r in range(N):
                    for j in range(hc):
                        ptrs.append(self.buf.recv_ptrs[c][r] + kind * plane + j * D * es)
                        strides.append(hc * D)
                        kinds.append(kind)
            self.seg.append((ptrs, strides, kinds))
        self._y = [torch.empty(self.Ls, 3 * N * hc * D, dtype=dtype, device=device) for _ in range(min(2, self.chunks))]
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.flag_back = torch.zeros(1, dtype=torch.float32, device=device)
        self.group_back = dist.new_group(ranks=list(range(N))) if (not self.emulated and N > 1) else None
        self.s_comm = torch.cuda.Stream(device)
        self.gi = self.residual = self.perm = None
        self.attn_fn: Optional[Callable] = None
        self._trace = None          # list of (name, start event, end event) while a traced forward runs

    def _span(self, name: str, stream):
        """Context manager that brackets the enclosed launches with two timing events when a trace is being taken."""
        layer = self

        class _Span:
            def __enter__(self_inner):
                if layer._trace is not None:
                    self_inner.e0 = torch.cuda.Event(enable_timing=True)
                    self_inner.e0.record(stream)

            def __exit__(self_inner, *exc):
                if layer._trace is not None:
                    e1 = torch.cuda.Event(enable_timing=True)
                    e1.record(stream)
                    layer._trace.append((name, self_inner.e0, e1))
                return False
        return _Span()

    def traced_forward(self, x: torch.Tensor):
        """One forward with timing events around every phase.  Returns (output, [(name, start_ms, end_ms)]) with
        times relative to the first launch: what runs under what on the two streams of this rank."""
        self._trace = []
        t0 = torch.cuda.Event(enable_timing=True)
        t0.record(torch.cuda.current_stream())
        try:
            out = self.forward(x)
            torch.cuda.synchronize()
            spans = [(n, t0.elapsed_time(a), t0.elapsed_time(b)) for n, a, b in self._trace]
        finally:
            self._trace = None
        return out, sorted(spans, key=lambda r: r[1])

    # ------------------------------------------------------------------------------------------ metadata
    def set_metadata(self, gi: torch.Tensor, residual: Optional[torch.Tensor] = None, perm: Optional[torch.Tensor] = None):
        """gi: (1, H/N, M, K) int32 indices of this rank's heads; residual: (1, H/N, L, D); perm: (H/N, L) int64."""
        if gi.shape[1] != self.Hl:
            raise ValueError(f"metadata must cover the {self.Hl} local heads")
        self.gi, self.residual, self.perm = gi, residual, perm

    def local_qkv(self, c: int):
        """(q, k, v) of head chunk c as (1, L, hc, D) views of this rank's receive buffer."""
        r = self.buf.recv[c]
        return r[0].unsqueeze(0), r[1].unsqueeze(0), r[2].unsqueeze(0)

    def out_peers(self, c: int):
        off = (self.rank * self.Hl + c * self.hc) * self.D * 2
        return ([p + off for p in self.buf.out_ptrs], self.Ls, (self.Ls * self.H * self.D, self.H * self.D, self.D))

    # ------------------------------------------------------------------------------------------ phases
    def _order(self, flag, group):
        if not self.emulated and self.world > 1:
            dist.all_reduce(flag, group=group)

    def project_chunk(self, x: torch.Tensor, c: int) -> torch.Tensor:
        y = self._y[c % len(self._y)]
        torch.matmul(x, self.w_chunk[c].t(), out=y)
        return y

    def scatter_chunk(self, y: torch.Tensor, c: int) -> None:
        ptrs, strides, kinds = self.seg[c]
        qkv_norm_rope_scatter(y, ptrs, strides, kinds, self.gq, self.gk, self.rope, self.grid, self.D,
                              row0=self.rank * self.Ls, token0=self.rank * self.Ls, eps=self.eps)

    def project_and_scatter(self, x: torch.Tensor) -> List[torch.cuda.Event]:
        """QKV projection by head chunk on the current stream; epilogue + exchange of each chunk on the communication
        stream under the next chunk's GEMM.  Returns one event per chunk (chunk delivered and ordered)."""
        if tuple(x.shape) != (self.Ls, self.hidden) or not x.is_contiguous():
            raise ValueError(f"expected contiguous activations of shape {(self.Ls, self.hidden)}")
        main = torch.cuda.current_stream()
        ev_done, ev_read = [], [None] * self.chunks
        for c in range(self.chunks):
            if c >= len(self._y) and ev_read[c - len(self._y)] is not None:
                main.wait_event(ev_read[c - len(self._y)])           # the epilogue has read the GEMM buffer about to be reused
            with self._span(f"qkv_gemm[{c}]", main):
                y = self.project_chunk(x, c)
            ev_g = torch.cuda.Event()
            ev_g.record(main)
            with torch.cuda.stream(self.s_comm):
                self.s_comm.wait_event(ev_g)
                with self._span(f"norm_rope_scatter[{c}]", self.s_comm):
                    self.scatter_chunk(y, c)
                ev_read[c] = torch.cuda.Event()
                ev_read[c].record(self.s_comm)
                with self._span(f"order[{c}]", self.s_comm):
                    self._order(self.flag, self.group)
                e = torch.cuda.Event()
                e.record(self.s_comm)
                ev_done.append(e)
        return ev_done

    def attend(self, events: Optional[List[torch.cuda.Event]] = None) -> None:
        """Sparse attention of every head chunk; rows are stored into the owners' sequence shards."""
        from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
        if self.gi is None:
            raise RuntimeError("set_metadata() first: the layer reuses cached indices")
        main = torch.cuda.current_stream()
        for c in range(self.chunks):
            if events is not None:
                main.wait_event(events[c])
            h0, h1 = c * self.hc, (c + 1) * self.hc
            q, k, v = self.local_qkv(c)
            with self._span(f"attention[{c}]", main):
                flash_attn_gather_kv_func(q, k, v, self.gi[:, h0:h1], residual=None if self.residual is None else self.residual[:, h0:h1],
                                          perm=None if self.perm is None else self.perm[h0:h1].contiguous(),
                                          out_peers=self.out_peers(c))

    def project_out(self) -> torch.Tensor:
        with self._span("out_gemm", torch.cuda.current_stream()):
            return torch.matmul(self.buf.out.view(self.Ls, self.H * self.D), self.wo.t())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        events = self.project_and_scatter(x)
        self.attend(events)
        with self._span("order[back]", torch.cuda.current_stream()):
            self._order(self.flag_back, self.group_back)   # every rank's rows have arrived before the projection reads them
        return self.project_out()

    # FLOPs of one layer call over all ranks: the two projections and the attention on the selected tokens
    def flops(self, topk: int) -> dict:
        gemm = 2.0 * self.L * self.hidden * (4 * self.H * self.D)
        attn = 4.0 * self.L * topk * self.D * self.H
        return {"gemm": gemm, "attention": attn, "total": gemm + attn}
