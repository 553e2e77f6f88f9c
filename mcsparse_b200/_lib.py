"""ctypes binding of ``libmcsparse_b200.so`` (the C ABI in ``include/mcsparse_b200.h``).

There is no fallback: if the shared library is missing or does not export a
symbol, importing a kernel wrapper raises.  Build it with
``python -m mcsparse_b200.build``.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# (MCSPARSE_B200_LIB points at another build of the library, e.g. an experimental variant)
LIB_PATH = Path(os.environ.get("MCSPARSE_B200_LIB") or Path(__file__).resolve().parent / "libmcsparse_b200.so")

MCS_DTYPE_BF16 = 0
MCS_DTYPE_FP16 = 1
MCS_DTYPE_E4M3 = 2
MCS_ATTN_OUT_GROUP_ORDER = 1
# argument-error codes of include/mcsparse_b200.h
MCS_ERR_NULL_POINTER, MCS_ERR_BAD_SHAPE, MCS_ERR_BAD_HEAD_DIM, MCS_ERR_BAD_DTYPE, MCS_ERR_BAD_ALIGNMENT = -1, -2, -3, -4, -5

# Every symbol the header declares; the CPU test-suite checks this list against
# the header and against the built library.
EXPORTED_SYMBOLS = (
    "mcs_version",
    "mcs_built_for_sm",
    "mcs_error_string",
    "mcs_gather_attn_fwd",
    "mcs_gather_attn_fwd_sharded",
    "mcs_dense_attn_fwd",
    "mcs_gather_attn_residual_fwd",
    "mcs_ulysses_scatter",
    "mcs_ulysses_scatter_dma",
    "mcs_qkv_norm_rope_scatter",
    "mcs_group_mass",
    "mcs_topk_select",
    "mcs_topk_select_var",
    "mcs_index_pack17",
    "mcs_index_unpack17",
    "mcs_topp_count",
    "mcs_pddp_workspace_bytes",
    "mcs_pddp_start_vector_rows",
    "mcs_pddp_levels",
    "mcs_pddp_perm",
    "mcs_pddp_static_scratch_bytes",
    "mcs_pddp_perm_static",
    "mcs_perm_apply",
    "mcs_perm_invert",
    "mcs_sm_clock_probe",
    "mcs_gather_rate_probe",
    "mcs_set_clock_buffer",
)


class GatherAttnArgs(C.Structure):
    """Mirror of ``mcs_gather_attn_args``."""

    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("gi", C.c_void_p), ("gl", C.c_void_p),
        ("residual", C.c_void_p), ("perm", C.c_void_p),
        ("scale_qk_log2", C.c_void_p), ("scale_v", C.c_void_p), ("status", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("o_stride", C.c_int64 * 3), ("r_stride", C.c_int64 * 3),
        ("B", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32), ("H", C.c_int32), ("D", C.c_int32),
        ("gather_len", C.c_int32), ("group_rows", C.c_int32), ("dtype", C.c_int32),
        ("softmax_scale", C.c_float), ("flags", C.c_int32),
        ("gi16", C.c_void_p), ("gi_hi", C.c_void_p),
    ]


class QkvEpilogueArgs(C.Structure):
    """Mirror of ``mcs_qkv_epilogue_args``."""

    _fields_ = [
        ("src", C.c_void_p), ("gamma_q", C.c_void_p), ("gamma_k", C.c_void_p), ("rope_cs", C.c_void_p),
        ("dst", C.POINTER(C.c_void_p)), ("dst_row_stride", C.POINTER(C.c_int64)), ("kind", C.POINTER(C.c_int32)),
        ("src_row_stride", C.c_int64), ("rows", C.c_int64), ("row0", C.c_int64), ("token0", C.c_int64),
        ("n_seg", C.c_int32), ("D", C.c_int32), ("grid_f", C.c_int32), ("grid_h", C.c_int32), ("grid_w", C.c_int32),
        ("pairs_t", C.c_int32), ("pairs_h", C.c_int32), ("dtype", C.c_int32), ("eps", C.c_float),
    ]


class GroupMassArgs(C.Structure):
    """Mirror of ``mcs_group_mass_args``."""

    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("lse", C.c_void_p), ("perm", C.c_void_p),
        ("mass", C.c_void_p), ("status", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3),
        ("B", C.c_int32), ("H", C.c_int32), ("Lq", C.c_int32), ("Lk", C.c_int32), ("D", C.c_int32),
        ("group_rows", C.c_int32), ("dtype", C.c_int32), ("normalize", C.c_int32),
        ("softmax_scale", C.c_float),
    ]


class PddpArgs(C.Structure):
    """Mirror of ``mcs_pddp_args``."""

    _fields_ = [
        ("x", C.c_void_p), ("start_vectors", C.c_void_p), ("perm_out", C.c_void_p),
        ("proj_levels", C.c_void_p), ("perm_levels", C.c_void_p), ("workspace", C.c_void_p),
        ("status", C.c_void_p),
        ("x_stride_bh", C.c_int64), ("x_stride_row", C.c_int64), ("workspace_bytes", C.c_int64),
        ("BH", C.c_int32), ("N", C.c_int32), ("D", C.c_int32), ("C", C.c_int32), ("pow_iters", C.c_int32),
        ("dtype", C.c_int32),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m mcsparse_b200.build` "
            "(there is no CPU or PyTorch fallback for the kernels)")
    L = C.CDLL(str(LIB_PATH))
    L.mcs_version.restype = C.c_int
    L.mcs_built_for_sm.restype = C.c_int
    L.mcs_error_string.restype = C.c_char_p
    L.mcs_error_string.argtypes = [C.c_int]
    L.mcs_gather_attn_fwd.restype = C.c_int
    L.mcs_gather_attn_fwd.argtypes = [C.POINTER(GatherAttnArgs), C.c_void_p]
    L.mcs_gather_attn_residual_fwd.restype = C.c_int
    L.mcs_gather_attn_residual_fwd.argtypes = [C.POINTER(GatherAttnArgs), C.c_void_p]
    L.mcs_dense_attn_fwd.restype = C.c_int
    L.mcs_dense_attn_fwd.argtypes = [C.POINTER(GatherAttnArgs), C.c_void_p]
    L.mcs_gather_attn_fwd_sharded.restype = C.c_int
    L.mcs_gather_attn_fwd_sharded.argtypes = [C.POINTER(GatherAttnArgs), C.POINTER(C.c_void_p), C.c_int32, C.c_int32,
                                              C.c_void_p]
    L.mcs_ulysses_scatter.restype = C.c_int
    L.mcs_ulysses_scatter.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int64, C.c_int64,
                                      C.c_int64, C.c_int64, C.c_void_p]
    L.mcs_ulysses_scatter_dma.restype = C.c_int
    L.mcs_ulysses_scatter_dma.argtypes = L.mcs_ulysses_scatter.argtypes
    L.mcs_qkv_norm_rope_scatter.restype = C.c_int
    L.mcs_qkv_norm_rope_scatter.argtypes = [C.POINTER(QkvEpilogueArgs), C.c_void_p]
    L.mcs_set_clock_buffer.restype = None
    L.mcs_set_clock_buffer.argtypes = [C.c_void_p]
    L.mcs_gather_rate_probe.restype = C.c_int
    L.mcs_gather_rate_probe.argtypes = [C.POINTER(GatherAttnArgs), C.c_void_p]
    L.mcs_sm_clock_probe.restype = C.c_int
    L.mcs_sm_clock_probe.argtypes = [C.c_void_p, C.c_void_p]
    L.mcs_group_mass.restype = C.c_int
    L.mcs_group_mass.argtypes = [C.POINTER(GroupMassArgs), C.c_void_p]
    L.mcs_topk_select.restype = C.c_int
    L.mcs_topk_select.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                                  C.c_void_p]
    L.mcs_topk_select_var.restype = C.c_int
    L.mcs_topk_select_var.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                                      C.c_void_p, C.c_void_p]
    L.mcs_index_pack17.restype = C.c_int
    L.mcs_index_pack17.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
    L.mcs_index_unpack17.restype = C.c_int
    L.mcs_index_unpack17.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
    L.mcs_topp_count.restype = C.c_int
    L.mcs_topp_count.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_float, C.c_void_p, C.c_void_p]
    L.mcs_pddp_workspace_bytes.restype = C.c_int64
    L.mcs_pddp_workspace_bytes.argtypes = [C.c_int32] * 3
    L.mcs_pddp_start_vector_rows.restype = C.c_int64
    L.mcs_pddp_start_vector_rows.argtypes = [C.c_int32] * 3
    L.mcs_pddp_levels.restype = C.c_int32
    L.mcs_pddp_levels.argtypes = [C.c_int32] * 2
    L.mcs_pddp_perm.restype = C.c_int
    L.mcs_pddp_perm.argtypes = [C.POINTER(PddpArgs), C.c_void_p]
    L.mcs_pddp_static_scratch_bytes.restype = C.c_int64
    L.mcs_pddp_static_scratch_bytes.argtypes = []
    L.mcs_pddp_perm_static.restype = C.c_int
    L.mcs_pddp_perm_static.argtypes = [C.POINTER(PddpArgs), C.c_void_p]
    for fn in (L.mcs_perm_apply, L.mcs_perm_invert):
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                       C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]
    _lib = L
    return L


def launch(fn_name: str, args, device, where: str) -> None:
    """Call an entry point on the current torch stream of ``device``; raise on an argument error."""
    import torch
    stream = torch.cuda.current_stream(device).cuda_stream
    rc = getattr(lib(), fn_name)(args, stream)
    raise_on_error(rc, where)
    if check_enabled():
        check_status(device, where)


def error_string(code: int) -> str:
    return lib().mcs_error_string(int(code)).decode()


class KernelLaunchError(RuntimeError):
    """An entry point of the C ABI returned a negative code (rejected arguments or a failed launch)."""

    def __init__(self, code: int, where: str):
        super().__init__(f"{where}: {error_string(code)} (code {code})")
        self.code = int(code)


def raise_on_error(rc: int, where: str) -> None:
    if rc != 0:
        raise KernelLaunchError(rc, where)


class KernelStatusError(RuntimeError):
    """A kernel reported a non-zero device status (an expired bounded wait)."""


_status_words: dict = {}


def status_word(device):
    """Per-device int32 status word shared by all launches (zero = healthy)."""
    import torch
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status_words[key] = t
    return t


def check_enabled() -> bool:
    """``MCSPARSE_B200_CHECK=1`` makes every wrapper synchronise and read the status word."""
    return os.environ.get("MCSPARSE_B200_CHECK", "0") == "1"


def check_status(device, where: str = "") -> None:
    """Synchronise and raise if any kernel on ``device`` reported an error."""
    import torch
    t = status_word(device)
    torch.cuda.synchronize(t.device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise KernelStatusError(f"mcsparse_b200 kernel status {code} ({where}): a bounded device-side wait expired")


_status_polls: dict = {}


def poll_status(device, where: str = "") -> None:
    """Non-blocking health check for a point that runs once per step: looks at the copy of the status word
    that the PREVIOUS call put in flight (raises KernelStatusError if it arrived non-zero, after clearing the
    device word so that later launches are not aborted by the stale code), then enqueues a fresh copy to
    pinned host memory on the current stream.  Never synchronises; an error surfaces one call late."""
    import torch
    t = status_word(device)
    key = t.device.index
    st = _status_polls.get(key)
    if st is None:
        st = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "event": None}
        _status_polls[key] = st
    if st["event"] is not None and st["event"].query():
        code = int(st["host"][0])
        if code != 0:
            st["event"] = None
            t.zero_()
            raise KernelStatusError(f"mcsparse_b200 kernel status {code} ({where}): a bounded device-side wait expired")
    elif st["event"] is not None:
        return                                   # the previous copy is still in flight: look again next time
    st["host"].copy_(t, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(t.device))
    st["event"] = ev
