"""GPU parity: top-k selection kernel vs the CPU oracle — bit-exact on identical fp32 scores."""

import pytest
import torch

from oracle.select import select_topk_ref

pytestmark = pytest.mark.gpu


def _run(dev, scores, k_total, sink_ranges):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import select_topk_with_sinks
    return select_topk_with_sinks(scores.to(dev), k_total, sink_ranges).cpu()


@pytest.mark.parametrize("L,k_total", [(1000, 128), (4096, 512), (32760, 2048), (70000, 4096)])
def test_random_scores_exact(cuda_device, L, k_total):
    g = torch.Generator().manual_seed(L)
    scores = torch.rand(3, 2, L, generator=g) ** 8          # mass-like: many tiny values
    out = _run(cuda_device, scores, k_total, [(0, 4)])
    ref = select_topk_ref(scores, k_total, sinks=range(4))
    assert torch.equal(out, ref)


def test_ties_go_to_lowest_index(cuda_device):
    L = 5000
    g = torch.Generator().manual_seed(1)
    scores = torch.randint(0, 6, (4, L), generator=g).float() / 8        # only 6 distinct values
    scores[1] = 0.0                                                      # fully tied row
    scores[2, ::2] = -0.0                                                # -0 and +0 tie
    out = _run(cuda_device, scores, 640, [(0, 4), (100, 103)])
    ref = select_topk_ref(scores, 640, sinks=[0, 1, 2, 3, 100, 101, 102])
    assert torch.equal(out, ref)


def test_negative_and_no_sinks_and_full_row(cuda_device):
    g = torch.Generator().manual_seed(2)
    scores = torch.randn(5, 777, generator=g)
    assert torch.equal(_run(cuda_device, scores, 256, None), select_topk_ref(scores, 256))
    assert torch.equal(_run(cuda_device, scores, 777, [(0, 4)]), select_topk_ref(scores, 777, range(4)))
    assert torch.equal(_run(cuda_device, scores, 4, [(0, 4)]), select_topk_ref(scores, 4, range(4)))


def test_reference_shaped_wrapper(cuda_device):
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import _select_topk_tokens
    g = torch.Generator().manual_seed(3)
    tp = torch.rand(1, 2, 3, 1024, generator=g)
    gi, gl = _select_topk_tokens(tp.to(cuda_device), 0.125, sink_ranges=[(0, 4)])
    assert tuple(gi.shape) == (1, 2, 3, 128) and gl is not None and int(gl.min()) == 1 == int(gl.max())
    assert torch.equal(gi.cpu(), select_topk_ref(tp, 128, range(4)))
    gi2, gl2 = _select_topk_tokens(tp.to(cuda_device), 0.25)
    assert tuple(gi2.shape) == (1, 2, 3, 256) and gl2 is None
    assert torch.equal(gi2.cpu(), select_topk_ref(tp, 256))


@pytest.mark.parametrize("L", [32768, 32761, 4100])
def test_register_path_structured_rows(cuda_device, L):
    """Rows that defeat the sampled lower bound of the register-resident kernel (it must only cost time):
    ramps, the winners hidden between the sampled positions, NaN-heavy and constant rows, a few NaNs."""
    g = torch.Generator().manual_seed(L)
    k_total = 2048 if L > 5000 else 512
    rows = []
    rows.append(torch.arange(L).float())                                   # winners at the end
    rows.append(torch.arange(L, 0, -1).float())                            # winners at the start
    hidden = torch.zeros(L)
    pos = torch.arange(1, L, 4)[: k_total + 100]                           # never a sampled position (those are multiples of 4)
    hidden[pos] = 1.0 + torch.rand(pos.numel(), generator=g)
    rows.append(hidden)
    nan_row = torch.rand(L, generator=g)
    nan_row[torch.randperm(L, generator=g)[: L - 500]] = float("nan")      # NaN ranks highest (torch.topk): a huge tie at the top
    rows.append(nan_row)
    rows.append(torch.full((L,), 0.25))                                    # constant row
    rows.append(torch.rand(L, generator=g) ** 16)                          # mass-like
    few = torch.rand(L, generator=g)
    few[torch.randperm(L, generator=g)[:37]] = float("nan")
    rows.append(few)
    scores = torch.stack(rows)
    out = _run(cuda_device, scores, k_total, [(0, 4)])
    ref = select_topk_ref(scores, k_total, sinks=range(4))
    assert torch.equal(out, ref)
