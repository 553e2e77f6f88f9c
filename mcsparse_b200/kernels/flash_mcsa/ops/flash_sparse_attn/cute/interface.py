"""Host wrappers of the gather-KV sparse attention kernels (B200 / sm_100a).

Same callables, argument meaning and error behaviour as the reference's
``mcsparse/kernels/flash_mcsa/ops/flash_sparse_attn/cute/interface.py``
(``flash_attn_gather_kv_func`` :108-340, ``flash_attn_gather_kv_fp8_func`` :346-570,
``flash_attn_func`` :576-603); the arch gate is sm_100 instead of sm_9x and the
launch goes through the C ABI (``mcs_gather_attn_fwd``) on the current torch CUDA
stream, asynchronously.

Extensions (keyword-only, all optional) fold the copies the reference's caller
makes around the kernel into the kernel itself:

``residual``  (B, H, Sq, D) tensor in (permuted) query order added to the output in
              fp32 before the single rounding to the output dtype
              (reference: ``out + residual`` as a separate pass, token_sparse.py:1112);
``perm``      (B*H, Sq) int64 permutation as returned by ``pca_group_perm``: query row
              ``i`` of a head is ``q[b, perm[i], h]`` and output row ``i`` is written to
              ``out[b, perm[i], h]`` (reference: apply_perm before / invert_perm after,
              token_sparse.py:1057-1060);
``group_rows`` query rows per index group (reference tile: 128);
``out_group_order`` with ``perm``: only Q is read through the permutation, output and lse rows stay in
              the permuted order (what the anchor step's residual construction works in).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from mcsparse_b200 import _lib

_TILE_N = 128


class PackedIndices:
    """An index tensor (B, H, M, gather_len) for sequences of up to 131,072 keys in 17-bit form: ``lo`` holds the low 16
    bits of every entry (int16 storage), ``hi`` bit 16 of 32 consecutive entries per int32 word: 272 instead of 512
    bytes per tile of 128.  The attention kernels read this form directly; pass it wherever ``gather_kv_indices`` is
    expected.  (The reference keeps int32 indices and offloads them to host memory; there is no such format there.)"""

    def __init__(self, lo: torch.Tensor, hi: torch.Tensor, shape):
        self.lo, self.hi, self.shape = lo, hi, tuple(shape)

    @property
    def device(self):
        return self.lo.device

    @property
    def is_cuda(self) -> bool:
        return self.lo.is_cuda

    def nbytes(self) -> int:
        return self.lo.numel() * 2 + self.hi.numel() * 4

    @staticmethod
    def pack(gi: torch.Tensor) -> "PackedIndices":
        if gi.dtype != torch.int32 or not gi.is_cuda or gi.shape[-1] % 128 != 0:
            raise ValueError("pack() takes an int32 CUDA tensor whose last dimension is a multiple of 128")
        gi = gi.contiguous()
        n = gi.numel()
        lo = torch.empty(gi.shape, dtype=torch.int16, device=gi.device)
        hi = torch.empty(n // 32, dtype=torch.int32, device=gi.device)
        stream = torch.cuda.current_stream(gi.device).cuda_stream
        _lib.raise_on_error(_lib.lib().mcs_index_pack17(gi.data_ptr(), n, lo.data_ptr(), hi.data_ptr(), stream), "mcs_index_pack17")
        return PackedIndices(lo, hi, gi.shape)

    def unpack(self) -> torch.Tensor:
        gi = torch.empty(self.shape, dtype=torch.int32, device=self.lo.device)
        stream = torch.cuda.current_stream(self.lo.device).cuda_stream
        _lib.raise_on_error(_lib.lib().mcs_index_unpack17(self.lo.data_ptr(), self.hi.data_ptr(), gi.numel(), gi.data_ptr(), stream),
                            "mcs_index_unpack17")
        return gi

    def __getitem__(self, key):
        # head slices are what the callers take (e.g. gi[:, h0:h1]); anything else goes through the int32 form
        if (isinstance(key, tuple) and len(key) == 2 and key[0] == slice(None) and isinstance(key[1], slice)
                and key[1].step in (None, 1)):
            B, H, M, K = self.shape
            h0, h1, _ = key[1].indices(H)
            if B == 1:
                per = M * K
                return PackedIndices(self.lo[:, h0:h1], self.hi.view(B, H, per // 32)[:, h0:h1].reshape(-1), (B, h1 - h0, M, K))
        raise TypeError("only gi[:, h0:h1] on a batch-1 tensor can be sliced in packed form; unpack() first")


def maybe_contiguous(x: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _get_device_arch() -> int:
    major, minor = torch.cuda.get_device_capability()
    return major * 10 + minor


def _validate_head_dims(head_dim: int, head_dim_v: int, alignment: int) -> None:
    if head_dim % alignment != 0:
        raise ValueError(f"head_dim must be a multiple of {alignment}, got {head_dim}")
    if head_dim_v % alignment != 0:
        raise ValueError(f"head_dim_v must be a multiple of {alignment}, got {head_dim_v}")
    if head_dim > 256:
        raise ValueError(f"head_dim > 256 is unsupported, got {head_dim}")
    if head_dim_v > 512:
        raise ValueError(f"head_dim_v > 512 is unsupported, got {head_dim_v}")


def _validate_tensor(tensor, name, shape, dtype, device) -> None:
    if tuple(tensor.shape) != tuple(shape):
        raise ValueError(f"{name}.shape must be {tuple(shape)}, got {tuple(tensor.shape)}")
    if tensor.dtype != dtype:
        raise ValueError(f"{name}.dtype must be {dtype}, got {tensor.dtype}")
    if tensor.device != device:
        raise ValueError(f"{name}.device must be {device}, got {tensor.device}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check_common(q, k, v, gather_kv_indices, what: str):
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is required")
    arch = _get_device_arch()
    if arch // 10 != 10:
        raise RuntimeError(f"{what} requires SM100/Blackwell (B200), got sm_{arch}")
    if q.requires_grad or k.requires_grad or v.requires_grad:
        raise RuntimeError("This package is forward-only; detach inputs or use torch.inference_mode().")


def _shape_checks(q, k, v):
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k and v must be 4D tensors")
    batch_size, seqlen_q, num_head, head_dim = q.shape
    batch_k, seqlen_k, num_head_kv, head_dim_k = k.shape
    batch_v, seqlen_v, num_head_kv_v, head_dim_v = v.shape
    if batch_k != batch_size or batch_v != batch_size:
        raise ValueError("q, k and v must have the same batch size")
    if seqlen_v != seqlen_k:
        raise ValueError("k and v must have the same sequence length")
    if num_head_kv_v != num_head_kv:
        raise ValueError("k and v must have the same number of KV heads")
    if head_dim_k != head_dim:
        raise ValueError("k head_dim must match q head_dim")
    if num_head % num_head_kv != 0:
        raise ValueError("num_head must be divisible by num_head_kv")
    if num_head != num_head_kv:
        raise NotImplementedError(
            "head-independent gather_kv_indices currently supports MHA only (num_head == num_head_kv)")
    return batch_size, seqlen_q, seqlen_k, num_head, head_dim, head_dim_v


def _index_checks(gather_kv_indices, gather_kv_lengths, batch_size, num_head, num_m_blocks, seqlen_k):
    gather_len = gather_kv_indices.shape[-1]
    packed = isinstance(gather_kv_indices, PackedIndices)
    if packed:
        if seqlen_k > (1 << 17):
            raise ValueError("packed indices carry 17 bits: seqlen_k must be <= 131072")
        if not gather_kv_indices.lo.is_contiguous() or not gather_kv_indices.hi.is_contiguous():
            gather_kv_indices = PackedIndices(gather_kv_indices.lo.contiguous(), gather_kv_indices.hi.contiguous(), gather_kv_indices.shape)
    elif gather_kv_indices.dtype != torch.int32:
        raise TypeError("gather_kv_indices must be int32")
    elif gather_kv_indices.stride(-1) != 1:
        raise ValueError("gather_kv_indices must be contiguous in the last dimension")
    if gather_len % _TILE_N != 0:
        raise ValueError(f"gather_len must be divisible by {_TILE_N}, got {gather_len}")
    if gather_len > math.ceil(seqlen_k / _TILE_N) * _TILE_N:
        raise ValueError(
            f"gather_len must be <= ceil_align(seqlen_k, {_TILE_N})={math.ceil(seqlen_k / _TILE_N) * _TILE_N}, "
            f"got gather_len={gather_len}, seqlen_k={seqlen_k}")
    expected = (batch_size, num_head, num_m_blocks, gather_len)
    if tuple(gather_kv_indices.shape) != expected:
        raise ValueError(f"gather_kv_indices must have shape {expected}, got {tuple(gather_kv_indices.shape)}")
    if gather_kv_lengths is not None:
        if gather_kv_lengths.dtype != torch.int32:
            raise TypeError("gather_kv_lengths must be int32")
        if tuple(gather_kv_lengths.shape) != expected[:3]:
            raise ValueError(
                f"gather_kv_lengths must have shape {expected[:3]}, got {tuple(gather_kv_lengths.shape)}")
        if not gather_kv_lengths.is_contiguous():
            gather_kv_lengths = gather_kv_lengths.contiguous()
    if not packed and not gather_kv_indices.is_contiguous():
        gather_kv_indices = gather_kv_indices.contiguous()
    return gather_kv_indices, gather_kv_lengths, gather_len


def _extras_checks(residual, perm, q, out_dtype, batch_size, num_head, seqlen_q, head_dim_v):
    if residual is not None:
        if tuple(residual.shape) != (batch_size, num_head, seqlen_q, head_dim_v):
            raise ValueError(
                f"residual must have shape {(batch_size, num_head, seqlen_q, head_dim_v)} (B,H,Sq,D), "
                f"got {tuple(residual.shape)}")
        if residual.dtype != out_dtype:
            raise TypeError(f"residual must have the output dtype {out_dtype}, got {residual.dtype}")
        if residual.device != q.device:
            raise ValueError("residual must be on the same device as q")
        residual = maybe_contiguous(residual)
    if perm is not None:
        if perm.dtype != torch.int64:
            raise TypeError("perm must be int64")
        if tuple(perm.shape) != (batch_size * num_head, seqlen_q):
            raise ValueError(
                f"perm must have shape {(batch_size * num_head, seqlen_q)} (B*H,Sq), got {tuple(perm.shape)}")
        if perm.device != q.device:
            raise ValueError("perm must be on the same device as q")
        perm = perm.contiguous()
    return residual, perm


def _launch(args: "_lib.GatherAttnArgs", device, where: str, out_peers=None, subtract: bool = False) -> None:
    stream = torch.cuda.current_stream(device).cuda_stream
    if subtract:
        if out_peers is not None:
            raise ValueError("residual_minus_attention and out_peers cannot be combined")
        rc = _lib.lib().mcs_gather_attn_residual_fwd(args, stream)
    elif out_peers is None:
        rc = _lib.lib().mcs_gather_attn_fwd(args, stream)
    else:
        import ctypes as C
        ptrs, rows_per_peer, _ = out_peers
        table = (C.c_void_p * len(ptrs))(*[int(x) for x in ptrs])
        rc = _lib.lib().mcs_gather_attn_fwd_sharded(args, table, len(ptrs), int(rows_per_peer), stream)
    _lib.raise_on_error(rc, f"{where}")
    if _lib.check_enabled():
        _lib.check_status(device, where)


def _fill_args(q, k, v, out, lse, gi, gl, residual, perm, gather_len, group_rows, dtype_code, softmax_scale,
               scale_qk_log2=None, scale_v=None) -> "_lib.GatherAttnArgs":
    a = _lib.GatherAttnArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    if isinstance(gi, PackedIndices):
        a.gi, a.gi16, a.gi_hi = None, gi.lo.data_ptr(), gi.hi.data_ptr()
    else:
        a.gi = gi.data_ptr()
    a.lse, a.gl = _ptr(lse), _ptr(gl)
    a.residual, a.perm = _ptr(residual), _ptr(perm)
    a.scale_qk_log2, a.scale_v = _ptr(scale_qk_log2), _ptr(scale_v)
    a.status = _lib.status_word(q.device).data_ptr()
    for dst, t in ((a.q_stride, q), (a.k_stride, k), (a.v_stride, v), (a.o_stride, out)):
        dst[0], dst[1], dst[2] = t.stride(0), t.stride(1), t.stride(2)
    if residual is not None:
        a.r_stride[0], a.r_stride[1], a.r_stride[2] = residual.stride(0), residual.stride(1), residual.stride(2)
    a.B, a.Sq, a.H, a.D = q.shape[0], q.shape[1], q.shape[2], q.shape[3]
    a.Sk = k.shape[1]
    a.gather_len, a.group_rows, a.dtype = gather_len, group_rows, dtype_code
    a.softmax_scale = float(softmax_scale)
    return a


def gather_rate_probe(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gather_kv_indices: torch.Tensor,
                      group_rows: int = 128) -> None:
    """Measurement aid: launch only the K/V row gather of the sparse attention call with these arguments (same
    grid, item walk and copy routine as the attention kernel's producer warps; the tiles land in shared memory
    that nothing reads).  Timed with CUDA events it gives the floor that the L2-to-shared-memory gather puts under
    the attention launch.  bf16 / fp16 / e4m3 inputs, head dimension 64 or 128 (e4m3: 128), int32 indices."""
    if not all(t.is_cuda for t in (q, k, v, gather_kv_indices)) or gather_kv_indices.dtype != torch.int32:
        raise ValueError("gather_rate_probe needs CUDA tensors and an int32 index list")
    if q.dtype == torch.bfloat16:
        code = _lib.MCS_DTYPE_BF16
    elif q.dtype == torch.float16:
        code = _lib.MCS_DTYPE_FP16
    elif q.dtype == torch.float8_e4m3fn:
        code = _lib.MCS_DTYPE_E4M3
    else:
        raise TypeError(f"unsupported dtype {q.dtype}")
    gi = gather_kv_indices.contiguous()
    args = _fill_args(q, k, v, q, None, gi, None, None, None, gi.shape[-1], int(group_rows), code, 1.0)
    rc = _lib.lib().mcs_gather_rate_probe(args, torch.cuda.current_stream(q.device).cuda_stream)
    _lib.raise_on_error(rc, "mcs_gather_rate_probe")


def flash_attn_gather_kv_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    gather_kv_indices: torch.Tensor,
    softmax_scale: Optional[float] = None,
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    tile_mn: Optional[Tuple[int, int]] = None,
    num_threads: int = 384,
    gather_kv_lengths: Optional[torch.Tensor] = None,
    *,
    residual: Optional[torch.Tensor] = None,
    perm: Optional[torch.Tensor] = None,
    group_rows: int = 128,
    out_peers=None,
    residual_minus_attention: bool = False,
    out_group_order: bool = False,
):
    """Forward-only token-level sparse gather-KV attention on B200.

    - MHA layout: q=(B, Sq, H, D), k=(B, Sk, H, D), v=(B, Sk, H, D), fp16 or bf16,
      last dimension contiguous; any batch/sequence/head strides that keep rows
      16-byte aligned (so BHSD tensors viewed as BSHD need no copy).
    - gather_kv_indices: (B, H, ceil(Sq / group_rows), gather_len) int32, gather_len a
      multiple of 128; entries address rows of the original K/V of that head.
      Duplicates count as separate softmax columns.
    - gather_kv_lengths: optional (B, H, ceil(Sq / group_rows)) int32 count of valid
      128-token tiles per group; None uses gather_len / 128 everywhere.
    - ``tile_mn`` and ``num_threads`` are accepted for signature compatibility; the
      tile is 128x128 (``tile_mn`` other than (128, 128) raises) and the CTA shape is
      fixed by the kernel.
    - Head dimension 64 or 128 (144 is zero-padded to 160 by the reference; here it
      raises ValueError, as do 96/192/256).

    Returns ``(out, lse)`` with ``lse`` None unless ``return_lse`` (natural log,
    softmax scale included, shape (B, H, Sq)).
    """
    q, k, v = [maybe_contiguous(t) for t in (q, k, v)]
    _check_common(q, k, v, gather_kv_indices, "gather-KV forward")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"q/k/v must be fp16 or bf16, got {q.dtype}")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k and v must have the same dtype")
    if not all(t.is_cuda for t in (q, k, v, gather_kv_indices)):
        raise RuntimeError("q, k, v and gather_kv_indices must be CUDA tensors")
    batch_size, seqlen_q, seqlen_k, num_head, head_dim, head_dim_v = _shape_checks(q, k, v)

    alignment = 16 // q.element_size()
    _validate_head_dims(head_dim, head_dim_v, alignment)
    # 64 and 128 run on the persistent kernel; every other multiple of 8 up to 256 (the reference lists 96, 144 padded
    # to 160, 192 and 256, interface.py:45-74) on the kernel that pads rows on their way into shared memory
    if head_dim_v != head_dim:
        raise ValueError(f"Unsupported head_dim={head_dim}/head_dim_v={head_dim_v}: head_dim_v must equal head_dim")
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(head_dim)
    if tile_mn is not None and tuple(tile_mn) != (128, _TILE_N):
        raise ValueError("gather-KV forward currently requires tile_mn == (128, 128)")
    if not (1 <= int(group_rows) <= 128):
        raise ValueError(f"group_rows must be in [1, 128], got {group_rows}")

    num_m_blocks = math.ceil(seqlen_q / group_rows)
    gather_kv_indices, gather_kv_lengths, gather_len = _index_checks(
        gather_kv_indices, gather_kv_lengths, batch_size, num_head, num_m_blocks, seqlen_k)

    device = q.device
    out_shape = (batch_size, seqlen_q, num_head, head_dim_v)
    if out_peers is not None:
        # sequence-sharded output (Ulysses): (pointers, rows_per_peer, (batch, row, head) element strides);
        # every finished row is stored straight into the shard of the rank that owns its token
        if out is not None:
            raise ValueError("give either out or out_peers")
        ptrs, rows_per_peer, o_strides = out_peers
        if len(ptrs) * int(rows_per_peer) < seqlen_q:
            raise ValueError("out_peers does not cover the query sequence")
    elif out is None:
        out = torch.empty(out_shape, dtype=q.dtype, device=device)
    else:
        _validate_tensor(out, "out", out_shape, q.dtype, device)
    lse_shape = (batch_size, num_head, seqlen_q)
    if lse is None:
        lse = torch.empty(lse_shape, dtype=torch.float32, device=device) if return_lse else None
    else:
        _validate_tensor(lse, "lse", lse_shape, torch.float32, device)
        if not lse.is_contiguous():
            raise ValueError("lse must be contiguous")
    residual, perm = _extras_checks(residual, perm, q, q.dtype, batch_size, num_head, seqlen_q, head_dim_v)

    dtype_code = _lib.MCS_DTYPE_BF16 if q.dtype == torch.bfloat16 else _lib.MCS_DTYPE_FP16
    args = _fill_args(q.detach(), k.detach(), v.detach(), q.detach() if out is None else out.detach(), lse,
                      gather_kv_indices, gather_kv_lengths, residual, perm, gather_len, int(group_rows), dtype_code,
                      softmax_scale)
    if out_peers is not None:
        args.out = None
        args.o_stride[0], args.o_stride[1], args.o_stride[2] = (int(x) for x in out_peers[2])
    if out_group_order and perm is not None:
        if out_peers is not None:
            raise ValueError("out_group_order and out_peers cannot be combined")
        args.flags = _lib.MCS_ATTN_OUT_GROUP_ORDER
    if residual_minus_attention and residual is None:
        raise ValueError("residual_minus_attention needs residual (the dense attention output, (B,H,Sq,D))")
    _launch(args, device, "flash_attn_gather_kv_func", out_peers, subtract=residual_minus_attention)
    return (out, lse) if return_lse else (out, None)


def flash_attn_gather_kv_fp8_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    gather_kv_indices: torch.Tensor,
    scale_qk_log2: torch.Tensor,
    scale_v: torch.Tensor,
    gather_kv_lengths: Optional[torch.Tensor] = None,
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    *,
    residual: Optional[torch.Tensor] = None,
    perm: Optional[torch.Tensor] = None,
):
    """Forward-only FP8 (e4m3) token-level sparse gather-KV attention on B200.

    Pre-quantised entry point; the caller owns quantisation.

    - q=(B, Sq, H, D), k=(B, Sk, H, D), v=(B, Sk, H, D), all float8_e4m3fn, D a multiple of 16 up to 256.
      V is passed as it is: the d-column pre-permutation the reference's Hopper
      kernel needs for its in-smem transpose does not exist here.
    - scale_qk_log2=(B, H, ceil(Sq/128)) fp32 = softmax_scale*log2(e)*s_q*s_k
    - scale_v=(B, H) fp32, folded into the final O normalisation
    - out is bfloat16; lse is fp32 and always written (returned only if asked)
    """
    q, k, v = [maybe_contiguous(t) for t in (q, k, v)]
    _check_common(q, k, v, gather_kv_indices, "fp8 gather-KV forward")
    if not (q.dtype == k.dtype == v.dtype == torch.float8_e4m3fn):
        raise TypeError(f"q/k/v must all be float8_e4m3fn, got {q.dtype}/{k.dtype}/{v.dtype}")
    if not all(t.is_cuda for t in (q, k, v, gather_kv_indices, scale_qk_log2, scale_v)):
        raise RuntimeError("all inputs must be CUDA tensors")
    batch_size, seqlen_q, seqlen_k, num_head, head_dim, head_dim_v = _shape_checks(q, k, v)
    # 128 runs on the persistent kernel; other multiples of 16 up to 256 (the reference lists 160) on the kernel that
    # pads rows on their way into shared memory
    if head_dim_v != head_dim or head_dim % 16 != 0 or not (16 <= head_dim <= 256):
        raise ValueError(
            f"fp8 gather-KV forward supports head_dim == head_dim_v, a multiple of 16 up to 256, "
            f"got D={head_dim}, Dv={head_dim_v}")
    num_m_blocks = math.ceil(seqlen_q / 128)
    gather_kv_indices, gather_kv_lengths, gather_len = _index_checks(
        gather_kv_indices, gather_kv_lengths, batch_size, num_head, num_m_blocks, seqlen_k)
    expected_scale_qk_shape = (batch_size, num_head, num_m_blocks)
    if tuple(scale_qk_log2.shape) != expected_scale_qk_shape:
        raise ValueError(
            f"scale_qk_log2 must have shape {expected_scale_qk_shape}, got {tuple(scale_qk_log2.shape)}")
    if tuple(scale_v.shape) != (batch_size, num_head):
        raise ValueError(f"scale_v must have shape {(batch_size, num_head)}, got {tuple(scale_v.shape)}")
    if scale_qk_log2.dtype != torch.float32 or scale_v.dtype != torch.float32:
        raise TypeError("scale_qk_log2 and scale_v must be float32")
    scale_qk_log2 = scale_qk_log2.contiguous()
    scale_v = scale_v.contiguous()

    device = q.device
    out_shape = (batch_size, seqlen_q, num_head, head_dim_v)
    if out is None:
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=device)
    else:
        _validate_tensor(out, "out", out_shape, torch.bfloat16, device)
    lse_shape = (batch_size, num_head, seqlen_q)
    if lse is None:
        lse = torch.empty(lse_shape, dtype=torch.float32, device=device)
    else:
        _validate_tensor(lse, "lse", lse_shape, torch.float32, device)
    residual, perm = _extras_checks(residual, perm, q, torch.bfloat16, batch_size, num_head, seqlen_q, head_dim_v)

    args = _fill_args(q.detach(), k.detach(), v.detach(), out.detach(), lse, gather_kv_indices, gather_kv_lengths,
                      residual, perm, gather_len, 128, _lib.MCS_DTYPE_E4M3, 1.0, scale_qk_log2, scale_v)
    _launch(args, device, "flash_attn_gather_kv_fp8_func")
    return (out, lse) if return_lse else (out, None)


def flash_attn_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    gather_kv_indices: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    softcap: Optional[float] = None,
    return_lse: bool = False,
    **kwargs,
):
    """flash-attn style shim: only the gather-KV, non-causal, no-softcap forward exists."""
    if gather_kv_indices is None:
        raise NotImplementedError("this package only provides the gather_kv_indices forward")
    if causal:
        raise NotImplementedError("causal attention is not supported by the gather-KV forward")
    if softcap not in (None, 0.0):
        raise NotImplementedError("softcap is not supported by the gather-KV forward")
    if kwargs:
        unsupported = ", ".join(sorted(kwargs.keys()))
        raise NotImplementedError(f"Unsupported arguments: {unsupported}")
    return flash_attn_gather_kv_func(
        q, k, v, gather_kv_indices, softmax_scale=softmax_scale, return_lse=return_lse)
