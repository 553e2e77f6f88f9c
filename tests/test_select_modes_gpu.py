"""GPU parity: variable-length selection (top-p budgets, per-row budgets, per-head adaptive budgets) against the CPU
oracle and against golden outputs of the reference's own ``_select_topk_tokens`` / ``_compute_adaptive_topk_token``."""

from pathlib import Path

import pytest
import torch

from oracle.select import select_modes_ref, select_topk_ref, topp_count_ref

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _peaked(shape, seed, temps):
    g = torch.Generator().manual_seed(seed)
    return torch.softmax(torch.randn(*shape, generator=g) * torch.tensor(temps).view(1, -1, 1, 1), dim=-1)


@pytest.mark.parametrize("L,topp,sinks", [(1000, 0.5, None), (4096, 0.9, [(0, 4)]), (32760, 0.7, [(0, 4)]), (98280, 0.95, None),
                                          (777, 1.0, [(3, 5)])])
def test_topp_count_matches_oracle(cuda_device, L, topp, sinks):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import topp_count
    tp = _peaked((1, 3, 4, L), L, [0.5, 2.0, 5.0])
    got = topp_count(tp.to(cuda_device), topp, sinks).cpu()
    flat_sinks = sorted({j for lo, hi in (sinks or []) for j in range(lo, hi)})
    want = topp_count_ref(tp, topp, flat_sinks)
    # fp32 partial sums against the oracle's fp64: a row whose prefix mass passes topp within rounding of a token's
    # mass may count one token more or less
    assert int((got - want).abs().max()) <= 1, (got, want)
    assert float((got == want).float().mean()) >= 0.75


def test_topp_count_edge_rows(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import topp_count
    L = 512
    rows = torch.zeros(1, 1, 5, L)
    rows[0, 0, 0, 17] = 1.0                                 # all mass on one token -> 1
    rows[0, 0, 1] = 1.0 / L                                 # flat row, topp 0.5 -> half of the tokens (ties enter one by one)
    rows[0, 0, 2, :10] = 0.01                               # total mass 0.1 < topp -> everything
    rows[0, 0, 3, 5], rows[0, 0, 3, 6] = 0.3, 0.3           # the second of two equal tokens still starts below topp, the third does not
    rows[0, 0, 3, 7] = 0.2
    rows[0, 0, 4, 100] = float("nan")                       # NaN carries no mass
    rows[0, 0, 4, 3] = 0.9
    got = topp_count(rows.to(cuda_device), 0.5).cpu()[0, 0].tolist()
    assert got == [1, L // 2, L, 2, 1], got


def test_selection_modes_match_reference_outputs(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import _compute_adaptive_topk_token, _select_topk_tokens
    for c in torch.load(GOLDEN / "select_modes_reference.pt"):
        if c["mode"] == "adaptive_ratio":
            g = torch.Generator().manual_seed(c["seed"])
            tp = torch.softmax(torch.randn(2, 4, 3, 1024, generator=g) * torch.tensor([0.5, 1.0, 2.0, 4.0]).view(1, 4, 1, 1), dim=-1)
            r = _compute_adaptive_topk_token(tp.to(cuda_device), c["base"]).cpu()
            rt = _compute_adaptive_topk_token(tp.to(cuda_device), c["base"], layer_t=0.25).cpu()
            assert torch.allclose(r, c["ratio"], rtol=1e-5) and torch.allclose(rt, c["ratio_t"], rtol=1e-5)
            continue
        g = torch.Generator().manual_seed(c["seed"])
        tp = torch.softmax(torch.randn(1, 2, 3, c["L"], generator=g) * torch.tensor([1.0, 3.0]).view(1, 2, 1, 1), dim=-1)
        ratio = torch.tensor([[0.08, 0.3]]) if c["ratio"] == "adaptive" else c["ratio"]
        gi, gl = _select_topk_tokens(tp.to(cuda_device), ratio if not torch.is_tensor(ratio) else ratio.to(cuda_device),
                                     selection_mode=c["mode"], topp=c["topp"], sink_ranges=c["sinks"])
        gi, gl = gi.cpu(), gl.cpu()
        # tile counts equal to the reference's; inside them the same set of tokens, ascending
        assert torch.equal(gl, c["gl"].to(torch.int32)), (c["mode"], c["L"])
        assert gi.shape == c["gi"].shape
        for r_ref, r_ours, n in zip(c["gi"].reshape(-1, gi.shape[-1]), gi.reshape(-1, gi.shape[-1]), (gl * 128).reshape(-1)):
            assert set(r_ref[:n].tolist()) == set(r_ours[:n].tolist())
            assert r_ours[:n].tolist() == sorted(r_ours[:n].tolist()) and bool((r_ours[n:] == 0).all())
        # and bit-equal to the oracle
        sinks = sorted({j for lo, hi in (c["sinks"] or []) for j in range(lo, hi)})
        o_gi, o_gl = select_modes_ref(tp, ratio, c["mode"], topp=c["topp"], sinks=sinks)
        assert torch.equal(o_gi, gi) and torch.equal(o_gl, gl)


@pytest.mark.parametrize("L,kmax", [(2000, 640), (32760, 2048), (70000, 4096)])
def test_per_row_budgets(cuda_device, L, kmax):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import select_topk_var
    g = torch.Generator().manual_seed(L)
    scores = torch.rand(2, 5, L, generator=g)
    k_rows = torch.randint(4, kmax + 1, (2, 5), generator=g, dtype=torch.int32)
    k_rows[0, 0], k_rows[1, 4] = 4, kmax                    # only the sinks / the full width
    got = select_topk_var(scores.to(cuda_device), k_rows.to(cuda_device), kmax, [(0, 4)]).cpu()
    for b in range(2):
        for r in range(5):
            k = int(k_rows[b, r])
            assert torch.equal(got[b, r, :k], select_topk_ref(scores[b, r].view(1, L), k, [0, 1, 2, 3])[0])
            assert bool((got[b, r, k:] == 0).all())


def test_backend_with_topp_selection(cuda_device):
    """Anchor step + reuse step with ``selection_mode='topk_topp'``: per-group tile counts flow into the attention."""
    from oracle.gather_attn import error_metrics, gather_attn_ref
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
    B, H, L, D = 1, 2, 1500, 128
    g = torch.Generator().manual_seed(5)
    cent = torch.randn(H, 16, D, generator=g)
    cid = torch.randint(0, 16, (L,), generator=g)
    mk = lambda: (cent[:, cid].unsqueeze(0) + 0.3 * torch.randn(B, H, L, D, generator=g)).to(torch.bfloat16)
    q, k, v = mk(), mk(), torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)
    cfg = TokenSparseConfig(topk=0.1, topp=0.9, selection_mode="topk_topp", calibrate_steps=[0], sink_ranges=[(0, 4)],
                            bias_correction=False, pca_reorder=False)
    ctx = TokenSparseContext(cfg, num_layers=1)
    dev = cuda_device
    ctx.forward(0, q.to(dev), k.to(dev), v.to(dev))
    cache = ctx.caches[0]
    gi, gl = cache._cached_indices.cpu(), cache._cached_lengths.cpu()
    assert gl is not None and int(gl.min()) >= 1 and int(gl.max()) * 128 == gi.shape[-1]
    ctx.step()
    out = ctx.forward(0, q.to(dev), k.to(dev), v.to(dev)).float().cpu()
    ref, _ = gather_attn_ref(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gi, gl=gl)
    mx, mr = error_metrics(out.transpose(1, 2), ref)
    assert mx < 2e-2 and mr < 1e-2, (mx, mr)
