"""CPU logic tests of the preserved boundary: step modes, dispatch counters, eligibility, layer clock
(modelled on the reference's tests/test_token_sparse_logic.py sections: schedule, mode, counters, eligibility)."""

import pytest
import torch

from mcsparse_b200.h3 import token_sparse_dispatch as tsd
from mcsparse_b200.kernels.flash_mcsa.token_sparse import (TokenSparseCache, TokenSparseConfig, _select_topk_tokens,
                                                           _sink_indices)


def test_mode_schedule():
    c = TokenSparseConfig(topk=0.1, calibrate_steps=[0, 5], full_steps=[0, 2], update_steps=[3])
    cache = TokenSparseCache(c)
    seen = []
    for _ in range(7):
        seen.append(cache.mode)
        if "calibrate" in cache.mode:
            cache._cached_indices = object()
        cache.step()
    assert seen == ["full_calibrate", "reuse", "full", "update", "reuse", "calibrate", "reuse"]
    assert TokenSparseCache(TokenSparseConfig()).mode == "calibrate"        # no cache -> calibrate


def test_config_guards():
    with pytest.raises(AssertionError):
        TokenSparseConfig(topk=0.0)
    with pytest.raises(AssertionError):
        TokenSparseConfig(BLKQ=64)
    with pytest.raises(AssertionError):
        TokenSparseConfig(sink_ranges=[(4, 4)])
    with pytest.raises(AssertionError):
        TokenSparseConfig(pca_reorder=True, share_lse=True)
    with pytest.raises(NotImplementedError):
        TokenSparseConfig(selection_mode="topp", topp=0.9)


def test_residual_dropped_when_permutation_is_newer():
    c = TokenSparseConfig(pca_reorder=True, bias_correction=True)
    cache = TokenSparseCache(c)
    cache._cached_residual, cache._residual_perm_gen, cache._perm_generation = object(), 1, 1
    assert cache.residual_if_valid() is not None
    cache._perm_generation = 2
    assert cache.residual_if_valid() is None and cache._cached_residual is None


def test_sink_arithmetic():
    assert _sink_indices([(0, 4), (10, 12)], 100) == [0, 1, 2, 3, 10, 11]
    assert _sink_indices([(98, 200)], 100) == [98, 99]
    assert _sink_indices(None, 100) == []


class FakeCache:
    def __init__(self):
        self.mode = "calibrate"


class FakeCtx:
    def __init__(self, n):
        self.caches = [FakeCache() for _ in range(n)]
        self.forwards, self.steps, self.resets = [], 0, 0

    def forward(self, li, q, k, v, scale):
        self.forwards.append(li)
        self.caches[li].mode = "reuse"
        return torch.zeros(q.shape, dtype=q.dtype)

    def step(self):
        self.steps += 1

    def reset(self):
        self.resets += 1


class FakeTensor:
    """Just enough of a CUDA bf16 BTHD tensor for the eligibility checks."""
    def __init__(self, shape, cuda=True, dtype=torch.bfloat16):
        self.shape, self.ndim, self.is_cuda, self.dtype = torch.Size(shape), len(shape), cuda, dtype
        self._t = torch.zeros(shape, dtype=dtype)

    def transpose(self, a, b):
        return self._t.transpose(a, b)


def test_dispatch_counters_and_layer_clock():
    ctx = FakeCtx(3)
    calls = []

    def original(q, k, v, *a, **kw):
        calls.append(q.shape[1])
        return "dense"

    d = tsd.make_mcsa_token_dispatch(original, num_layers=3, topk=0.15, full_layers=[2], min_seq_len=1024, context=ctx,
                                     sink_ranges=[(0, 4)])
    long_ = FakeTensor((1, 2048, 2, 128))
    short = FakeTensor((1, 77, 2, 128))
    for step in range(2):
        tsd.mcsa_token_begin_forward()
        for li in range(3):
            assert d(short, short, short) == "dense"              # interleaved short attention: fallback
            out = d(long_, long_, long_)
            assert (out == "dense") == (li == 2)
    s = tsd.get_mcsa_token_stats()
    assert s["dispatch_calls"] == 12 and s["fallback_calls"] == 6
    assert s["dense_guard_calls"] == 2 and s["kernel_calls"] == 4
    assert s["dispatch_calls"] == s["fallback_calls"] + s["dense_guard_calls"] + s["kernel_calls"]
    assert s["calibrate_calls"] == 2 and s["steps_ticked"] == 2 and s["layers_per_step"] == 3
    assert ctx.forwards == [0, 1, 0, 1] and ctx.steps == 1
    assert s["seen_seq_lens"] == {77: 6, 2048: 6} and s["seq_len"] == 2048
    assert abs(s["effective_density"] - (4 + 0.15 * 2048) / 2048) < 1e-9
    # ineligible variants
    assert d(long_, long_, long_, attn_mask=object()) == "dense"
    assert d(long_, long_, long_, is_causal=True) == "dense"
    assert d(FakeTensor((1, 2048, 2, 128), cuda=False), long_, long_) == "dense"
    assert d(FakeTensor((1, 2048, 2, 96)), FakeTensor((1, 2048, 2, 96)), FakeTensor((1, 2048, 2, 96))) == "dense"
    assert tsd.get_mcsa_token_stats()["fallback_calls"] == 10


def test_dispatch_guards():
    with pytest.raises(RuntimeError):
        tsd.make_mcsa_token_dispatch(lambda *a, **k: None, num_layers=2, topk=1.5, context=FakeCtx(2))
    ctx = FakeCtx(1)
    d = tsd.make_mcsa_token_dispatch(lambda *a, **k: "dense", num_layers=1, context=ctx)
    t = FakeTensor((1, 2048, 2, 128))
    tsd.mcsa_token_begin_forward()
    d(t, t, t)
    with pytest.raises(RuntimeError):
        d(t, t, t)                         # a second sparse layer without a new step: numbering would drift
    tsd.reset_mcsa_token_state()
    assert tsd.get_mcsa_token_stats()["dispatch_calls"] == 0 and ctx.resets >= 1
