"""GPU test of the allocation-free grouping entry point (``mcs_pddp_perm_static``).

Some callers of this library may not allocate device memory at all (their own pool owns the GPU, or
cudaMalloc is banned on their latency path because it synchronises the device), so they cannot supply the
workspace ``mcs_pddp_perm`` wants.  The static variant uses a fixed 32 MiB scratch array inside the library.
Here it is called directly through the C ABI, twice in a row (the second call finds the first call's data in
the shared scratch), and must give exactly the permutation of the regular entry point; an oversized shape
must be refused.  Collected last on purpose, so a failure here cannot hide other tests.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(_lib, x, sv, perm, ws=None):
    a = _lib.PddpArgs()
    a.x, a.start_vectors, a.perm_out = x.data_ptr(), sv.data_ptr(), perm.data_ptr()
    a.proj_levels, a.perm_levels = None, None
    a.workspace = None if ws is None else ws.data_ptr()
    a.workspace_bytes = 0 if ws is None else ws.numel()
    a.status = _lib.status_word(x.device).data_ptr()
    a.x_stride_bh, a.x_stride_row = x.stride(0), x.stride(1)
    a.BH, a.N, a.D = x.shape
    a.C, a.pow_iters, a.dtype = 128, 4, _lib.MCS_DTYPE_BF16
    return a


def test_static_scratch_matches_workspace_entry_point_twice(cuda_device):
    from mcsparse_b200 import _lib
    from mcsparse_b200.kernels.flash_mcsa.pca_group import pddp_start_vectors
    lib = _lib.lib()
    dev = cuda_device
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert lib.mcs_pddp_static_scratch_bytes() == 32 << 20
    for seed, (BH, N, D) in enumerate([(2, 3000, 128), (3, 1500, 64)]):
        g = torch.Generator().manual_seed(seed)
        cent = torch.randn(BH, 8, D, generator=g)
        cid = torch.randint(0, 8, (N,), generator=g)
        x = (cent[:, cid] + 0.3 * torch.randn(BH, N, D, generator=g)).to(torch.bfloat16).to(dev)
        sv = pddp_start_vectors(BH, N, 128, D, 0).to(dev)
        need = lib.mcs_pddp_workspace_bytes(BH, N, 128)
        assert 0 < need <= lib.mcs_pddp_static_scratch_bytes()
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        ref = torch.empty(BH, N, dtype=torch.int64, device=dev)
        assert lib.mcs_pddp_perm(C.byref(_args(_lib, x, sv, ref, ws)), stream) == 0
        for _ in range(2):                                  # two calls in a row share the scratch
            out = torch.full((BH, N), -1, dtype=torch.int64, device=dev)
            assert lib.mcs_pddp_perm_static(C.byref(_args(_lib, x, sv, out)), stream) == 0
            torch.cuda.synchronize(dev)
            assert torch.equal(out, ref)                    # deterministic kernels: exact equality
    _lib.check_status(dev, "static scratch")


def test_static_scratch_rejects_oversized_shapes(cuda_device):
    from mcsparse_b200 import _lib
    lib = _lib.lib()
    BH, N = 24, 32760
    assert lib.mcs_pddp_workspace_bytes(BH, N, 128) > lib.mcs_pddp_static_scratch_bytes()
    x = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device=cuda_device)
    a = _args(_lib, x, x, x)
    a.BH, a.N = BH, N
    assert lib.mcs_pddp_perm_static(C.byref(a), None) == -10        # MCS_ERR_TOO_LARGE, nothing launched
