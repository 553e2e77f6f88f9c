"""CPU tests: the C ABI library builds, loads, and exports every symbol the header declares."""

import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _header_functions():
    text = (ROOT / "include" / "mcsparse_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mcs_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mcsparse_b200 import _lib, build
    build.build()
    lib = _lib.lib()
    declared = _header_functions()
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared
    assert lib.mcs_built_for_sm() == 100 and lib.mcs_version() >= 1
    assert _lib.error_string(0) == "ok" and "null" in _lib.error_string(-1)


def test_argument_errors_without_a_gpu():
    """Validation happens before any CUDA call, so it can be exercised on a CPU-only machine."""
    import ctypes as C
    from mcsparse_b200 import _lib
    lib = _lib.lib()
    assert lib.mcs_gather_attn_fwd(None, None) == -1
    a = _lib.GatherAttnArgs()
    assert lib.mcs_gather_attn_fwd(C.byref(a), None) == -1                # null tensors
    assert lib.mcs_topk_select(None, None, None, 0, 1, 10, 5, None) == -1
    assert lib.mcs_pddp_workspace_bytes(24, 32760, 128) > 0
    assert lib.mcs_pddp_levels(32760, 128) == 8 and lib.mcs_pddp_levels(98280, 128) == 10
    assert lib.mcs_pddp_start_vector_rows(24, 32760, 128) == 24 * 255
    assert lib.mcs_perm_apply(None, None, None, 1, 1, 16, 16, 16, 16, 16, None) == -1


def test_wrappers_fail_loudly_without_cuda():
    import pytest
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute import flash_attn_gather_kv_func
    q = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16)
    gi = torch.zeros(1, 1, 1, 128, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        flash_attn_gather_kv_func(q, q, q, gi)
