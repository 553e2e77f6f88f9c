"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations.

They stand in for MiniMax-H3 video latents (the checkpoint is not available):
clustered Q/K (centroid + noise) on a flattened (frames, height, width) latent grid,
Gaussian V, Gaussian residual.  Used by ``bench.py``, ``__graft_entry__.smoke`` and the
tests; everything is generated from explicit ``torch.Generator`` seeds.

Distribution convention: ``N(0, 0.01)`` is read as (mean, variance), so the residual has
standard deviation 0.1; the Q/K noise has standard deviation 0.3.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

N_SINK = 4


@dataclass(frozen=True)
class VideoShape:
    """One attention workload on a flattened latent grid (t-major)."""
    name: str
    heads: int
    grid: Tuple[int, int, int]      # (frames, height, width)
    block: Tuple[int, int, int]     # spatial-temporal block that shares a centroid
    head_dim: int = 128
    group_rows: int = 128
    topk: int = 2048
    n_centroids: int = 64

    @property
    def seq_len(self) -> int:
        f, h, w = self.grid
        return f * h * w

    @property
    def n_groups(self) -> int:
        return math.ceil(self.seq_len / self.group_rows)

    def attn_flops(self, heads: Optional[int] = None) -> float:
        """Algorithmic FLOPs of one gather-KV attention call: 4 * L_Q * K_sel * D * H."""
        return 4.0 * self.seq_len * self.topk * self.head_dim * (heads or self.heads)


# bf16 single-GPU video-DiT shape: H=24, L=32,760 (21x39x40), top-k 2048 -> 256 groups
C2 = VideoShape("dit_L32760_H24_D128_topk2048", 24, (21, 39, 40), (3, 6, 6), topk=2048)
# FP8 long-video shape: H=40, L=98,280 (21x72x65), top-k 4096 -> 768 groups
C3 = VideoShape("dit_L98280_H40_D128_topk4096", 40, (21, 72, 65), (7, 12, 11), topk=4096)
# attention of the Ulysses context-parallel layer: the long-video grid in bf16, 40 heads sharded over the ranks
C5 = VideoShape("ulysses_dit_L98280_H40_D128_topk4096", 40, (21, 72, 65), (7, 12, 11), topk=4096)


def cluster_ids(shape: VideoShape) -> torch.Tensor:
    """Centroid id of every token: its spatial-temporal block index modulo the centroid count."""
    F, Hh, W = shape.grid
    bf, bh, bw = shape.block
    nby, nbx = math.ceil(Hh / bh), math.ceil(W / bw)
    f = torch.arange(F).view(F, 1, 1) // bf
    y = torch.arange(Hh).view(1, Hh, 1) // bh
    x = torch.arange(W).view(1, 1, W) // bw
    cid = (f * (nby * nbx) + y * nbx + x) % shape.n_centroids
    return cid.reshape(-1)


def clustered_qkv(shape: VideoShape, heads: Optional[int] = None, seed: int = 0,
                  device="cpu", dtype=torch.bfloat16, head_offset: int = 0):
    """Q, K = centroid[c(t)] + N(0, 0.3^2); V ~ N(0,1).  Returns (B=1, L, H, D) tensors.

    Heads are generated one at a time from per-head seeds so that any head subset
    (``head_offset``, ``heads``) reproduces the same values as the full tensor.
    """
    H = heads or shape.heads
    L, D = shape.seq_len, shape.head_dim
    cid = cluster_ids(shape).to(device)
    q = torch.empty(1, L, H, D, dtype=dtype, device=device)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    for h in range(H):
        g = torch.Generator(device=device).manual_seed(seed * 100003 + (head_offset + h) * 7919 + 17)
        cent = torch.randn(shape.n_centroids, D, generator=g, device=device)
        q[0, :, h] = (cent[cid] + 0.3 * torch.randn(L, D, generator=g, device=device)).to(dtype)
        k[0, :, h] = (cent[cid] + 0.3 * torch.randn(L, D, generator=g, device=device)).to(dtype)
        v[0, :, h] = torch.randn(L, D, generator=g, device=device).to(dtype)
    return q, k, v


def residual_like(shape: VideoShape, heads: Optional[int] = None, seed: int = 1, device="cpu",
                  dtype=torch.bfloat16, head_offset: int = 0) -> torch.Tensor:
    """Cached dense-minus-sparse residual stand-in: (1, H, L, D) ~ N(0, 0.01) (sigma 0.1).  Generated head by
    head from per-head seeds, so any head subset reproduces the values of the full tensor."""
    H = heads or shape.heads
    out = torch.empty(1, H, shape.seq_len, shape.head_dim, dtype=dtype, device=device)
    for h in range(H):
        g = torch.Generator(device=device).manual_seed(seed * 7 + 3 + (head_offset + h) * 104729)
        out[0, h] = (0.1 * torch.randn(shape.seq_len, shape.head_dim, generator=g, device=device)).to(dtype)
    return out


def random_sorted_indices(B, H, M, gather_len, Sk, seed=0, n_sink=N_SINK, device="cpu") -> torch.Tensor:
    """Per group: the sink tokens plus a uniform sample without replacement of the rest, ascending int32."""
    g = torch.Generator(device=device).manual_seed(seed + 11)
    scores = torch.rand(B, H, M, Sk - n_sink, generator=g, device=device)
    rest = scores.topk(gather_len - n_sink, dim=-1).indices + n_sink
    sinks = torch.arange(n_sink, device=device).expand(B, H, M, n_sink)
    return torch.cat([sinks, rest.sort(dim=-1).values], dim=-1).to(torch.int32).contiguous()


def quantize_e4m3_per_head(x: torch.Tensor):
    """Per-head symmetric e4m3 quantisation of a (B, L, H, D) tensor with scale = amax / 448.
    Returns (x8 float8_e4m3fn, scale (B, H) fp32) with x ~= x8 * scale."""
    amax = x.float().abs().amax(dim=(1, 3)).clamp_min(1e-12)          # (B, H)
    scale = amax / 448.0
    x8 = (x.float() / scale[:, None, :, None]).to(torch.float8_e4m3fn)
    return x8, scale.to(torch.float32)


def topmass_indices(q: torch.Tensor, k: torch.Tensor, shape: VideoShape, heads_per_chunk: int = 4) -> torch.Tensor:
    """Anchor-step selection with this package's own kernels, as the benchmark configuration defines its
    indices: per query group the 4 sink tokens plus the (topk - 4) tokens of highest exact fp32 group
    mass, ascending int32 (1, H, M, topk).  q, k: (1, L, H, D) CUDA tensors.  The dense log-sum-exp that
    the mass needs comes from the attention kernel's dense mode."""
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import dense_attention_with_lse, group_mass, select_topk_with_sinks
    H, D = q.shape[2], q.shape[3]
    scale = 1.0 / math.sqrt(D)
    out = torch.empty(1, H, shape.n_groups, shape.topk, dtype=torch.int32, device=q.device)
    for h0 in range(0, H, heads_per_chunk):
        h1 = min(H, h0 + heads_per_chunk)
        qh = q[:, :, h0:h1].transpose(1, 2)            # (1, h, L, D) views
        kh = k[:, :, h0:h1].transpose(1, 2)
        _, lse = dense_attention_with_lse(qh.contiguous(), kh.contiguous(), kh.contiguous(), scale)
        mass = group_mass(qh, kh, lse, group_rows=shape.group_rows, scale=scale)
        out[:, h0:h1] = select_topk_with_sinks(mass, shape.topk, [(0, N_SINK)])
    return out
