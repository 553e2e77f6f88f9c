"""Fast PDDP query grouping on B200: same callables as the reference's
``mcsparse/kernels/flash_mcsa/pca_group.py`` (``pca_group_perm`` :141-243, ``apply_perm`` :40,
``invert_perm`` :45, ``*_bhld`` :52-61, ``identity_perm`` :64, ``leaf_inertia`` :69), with the
levels of the bisection running as CUDA kernels without any host synchronisation.

Only Q is reordered; K and V keep their order, so gather indices keep addressing the original
keys.  The attention kernel can read Q through the permutation and write its output back through
it (``perm=`` of ``flash_attn_gather_kv_func``), in which case ``apply_perm`` / ``invert_perm`` are
not needed on the hot path at all.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from mcsparse_b200 import _lib

__all__ = ["pca_group_perm", "apply_perm", "invert_perm", "apply_perm_bhld", "invert_perm_bhld",
           "leaf_inertia", "identity_perm", "pddp_start_vectors"]


def identity_perm(BH: int, N: int, device) -> Tensor:
    """Identity permutation (the no-reordering baseline)."""
    return torch.arange(N, device=device).unsqueeze(0).expand(BH, N).contiguous()


def pddp_start_vectors(BH: int, N: int, C: int, D: int, seed: int = 0) -> Tensor:
    """Power-iteration start vectors for every level, level-major, (rows, D) fp32 on the CPU.

    One N(0,1) draw per node per level from a single generator seeded once, consumed level by
    level, like the reference (pca_group.py:184-185, :224).  The generator lives on the CPU so that
    the vectors — and with them the grouping — do not depend on the device.
    """
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    rows = int(_lib.lib().mcs_pddp_start_vector_rows(BH, N, C))
    # draw level by level so that the stream of random numbers matches a per-level randn(M, D)
    out, K = [], (N + C - 1) // C
    ranges = [(0, K)]
    while any(hi - lo > 1 for lo, hi in ranges):
        out.append(torch.randn(BH * len(ranges), D, generator=gen))
        nxt = []
        for lo, hi in ranges:
            if hi - lo <= 1:
                nxt.append((lo, hi))
            else:
                mid = lo + (hi - lo) // 2
                nxt += [(lo, mid), (mid, hi)]
        ranges = nxt
    v = torch.cat(out) if out else torch.zeros(0, D)
    assert v.shape[0] == rows
    return v


@torch.no_grad()
def pca_group_perm(x: Tensor, C: int = 128, pow_iters: int = 4, seed: int = 0, proj_dim: Optional[int] = None,
                   *, start_vectors: Optional[Tensor] = None, return_debug: bool = False):
    """Per-head permutation from recursive principal-direction bisection.

    x: (BH, N, D) bf16/fp16 CUDA tensor with contiguous rows (any batch/row strides), D a multiple of 8 up to 256
    (64 and 128 on the tensor-core Gram path, the others on Gram-free power iterations).
    Returns perm (BH, N) int64: ``x[b, perm[b, i]]`` is the i-th reordered token.  ``proj_dim`` (an
    option the reference leaves off by default) is not part of this path.  ``return_debug`` adds the
    per-level fp32 projections (levels, BH, N) and orders (levels + 1, BH, N).
    """
    if proj_dim is not None:
        raise NotImplementedError("proj_dim is not part of the accelerated path")
    if x.ndim != 3:
        raise ValueError("x must be (BH, N, D)")
    BH, N, D = x.shape
    if not x.is_cuda:
        raise RuntimeError("x must be a CUDA tensor")
    if N <= C:
        return identity_perm(BH, N, x.device)
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"x must be bf16 or fp16, got {x.dtype}")
    if D % 8 != 0 or not (8 <= D <= 256):
        raise ValueError(f"head_dim must be a multiple of 8 up to 256, got {D}")
    if x.stride(-1) != 1:
        x = x.contiguous()
    L = _lib.lib()
    ws_bytes = int(L.mcs_pddp_workspace_bytes(BH, N, C))
    if ws_bytes <= 0:
        raise ValueError("sequence too long for the grouping tables")
    if start_vectors is None:
        start_vectors = pddp_start_vectors(BH, N, C, D, seed)
    sv = start_vectors.to(device=x.device, dtype=torch.float32).contiguous()
    levels = int(L.mcs_pddp_levels(N, C))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    perm = torch.empty(BH, N, dtype=torch.int64, device=x.device)
    proj = torch.zeros(levels, BH, N, dtype=torch.float32, device=x.device) if return_debug else None
    orders = torch.empty(levels + 1, BH, N, dtype=torch.int32, device=x.device) if return_debug else None
    a = _lib.PddpArgs()
    a.x, a.start_vectors, a.perm_out = x.data_ptr(), sv.data_ptr(), perm.data_ptr()
    a.proj_levels = None if proj is None else proj.data_ptr()
    a.perm_levels = None if orders is None else orders.data_ptr()
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws_bytes
    a.status = _lib.status_word(x.device).data_ptr()
    a.x_stride_bh, a.x_stride_row = x.stride(0), x.stride(1)
    a.BH, a.N, a.D, a.C, a.pow_iters = BH, N, D, int(C), int(pow_iters)
    a.dtype = _lib.MCS_DTYPE_BF16 if x.dtype == torch.bfloat16 else _lib.MCS_DTYPE_FP16
    _lib.launch("mcs_pddp_perm", a, x.device, "pca_group_perm")
    ws.record_stream(torch.cuda.current_stream(x.device))
    return (perm, proj, orders) if return_debug else perm


def _perm_rows(x: Tensor, perm: Tensor, invert: bool) -> Tensor:
    if x.ndim != 3:
        raise ValueError("x must be (BH, N, D)")
    BH, N, D = x.shape
    if tuple(perm.shape) != (BH, N) or perm.dtype != torch.int64:
        raise ValueError(f"perm must be int64 of shape {(BH, N)}")
    if x.stride(-1) != 1:
        x = x.contiguous()
    es = x.element_size()
    if (D * es) % 16:
        raise ValueError("row size must be a multiple of 16 bytes")
    out = torch.empty(BH, N, D, dtype=x.dtype, device=x.device)
    fn = _lib.lib().mcs_perm_invert if invert else _lib.lib().mcs_perm_apply
    stream = torch.cuda.current_stream(x.device).cuda_stream
    rc = fn(x.data_ptr(), out.data_ptr(), perm.contiguous().data_ptr(), BH, N, D * es,
            x.stride(0) * es, x.stride(1) * es, out.stride(0) * es, out.stride(1) * es, stream)
    _lib.raise_on_error(rc, f"perm rows")
    return out


def apply_perm(x: Tensor, perm: Tensor) -> Tensor:
    """Reorder (BH, N, D) into leaf order using a (BH, N) permutation."""
    return _perm_rows(x, perm, invert=False)


def invert_perm(x_permuted: Tensor, perm: Tensor) -> Tensor:
    """Invert apply_perm and restore the original token order (a scatter; no argsort)."""
    return _perm_rows(x_permuted, perm, invert=True)


def apply_perm_bhld(x: Tensor, perm: Tensor) -> Tensor:
    """Apply a (B*H, L) permutation to a (B, H, L, D) tensor."""
    B, H, L, D = x.shape
    return apply_perm(x.reshape(B * H, L, D), perm).reshape(B, H, L, D)


def invert_perm_bhld(x: Tensor, perm: Tensor) -> Tensor:
    """Invert apply_perm_bhld and restore the original query order."""
    B, H, L, D = x.shape
    return invert_perm(x.reshape(B * H, L, D), perm).reshape(B, H, L, D)


def leaf_inertia(x: Tensor, perm: Tensor, C: int) -> float:
    """Mean squared distance of tokens to their leaf centroid (diagnostic; plain torch)."""
    BH, N, D = x.shape
    xp = x.gather(1, perm.unsqueeze(-1).expand(-1, -1, D)).float()
    total, count = 0.0, 0
    for start in range(0, N, C):
        blk = xp[:, start:start + C]
        if blk.shape[1] < 2:
            continue
        dev = blk - blk.mean(dim=1, keepdim=True)
        total += dev.pow(2).sum(-1).sum().item()
        count += blk.shape[0] * blk.shape[1]
    return total / max(count, 1)
