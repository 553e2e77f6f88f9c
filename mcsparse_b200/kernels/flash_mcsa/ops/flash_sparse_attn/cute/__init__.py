"""Gather-KV attention entry points (same names as the reference's package export,
mcsparse/kernels/flash_mcsa/ops/flash_sparse_attn/cute/__init__.py:1-6), plus the packed index form."""
from .interface import PackedIndices, flash_attn_func, flash_attn_gather_kv_fp8_func, flash_attn_gather_kv_func

__all__ = [
    "flash_attn_func",
    "flash_attn_gather_kv_func",
    "flash_attn_gather_kv_fp8_func",
    "PackedIndices",
]
