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
    c2 = TokenSparseConfig(topk=0.1, calibrate_steps=[0], approx_steps=[2])
    cache = TokenSparseCache(c2)
    cache._cached_indices = object()
    cache._step_count = 2
    assert cache.mode == "approx"
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
    with pytest.raises(AssertionError):
        TokenSparseConfig(selection_mode="topp")                      # topp modes need topp
    assert TokenSparseConfig(selection_mode="topk_topp", topp=0.9).topp == 0.9
    with pytest.raises(NotImplementedError):
        TokenSparseConfig(cal_downsample=2)
    with pytest.raises(NotImplementedError):
        TokenSparseConfig(pca_proj_dim=32)
    with pytest.raises(NotImplementedError):
        TokenSparseConfig(share_lse=True)                             # accepted by the reference, not built here: say so


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

    def contiguous(self):
        return self


# the factory's defaults are the reference's (10 dense steps, dense layers 0-1, anchor at step 9, sink required, floor
# 4096); the dispatch tests below want every step sparse from step 0
_PLAIN = dict(allow_no_sink=True, dense_steps=0, dense_layers="", calibrate_steps=(0,), min_seq_len=1024)


def test_dispatch_counters_and_layer_clock():
    ctx = FakeCtx(3)
    calls = []

    def original(q, k, v, *a, **kw):
        calls.append(q.shape[1])
        return "dense"

    d = tsd.make_mcsa_token_dispatch(original, num_layers=3, topk=0.15, full_layers=[2], context=ctx,
                                     sink_ranges=[(0, 4)], **_PLAIN)
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
    assert d(FakeTensor((1, 2048, 2, 100)), FakeTensor((1, 2048, 2, 100)), FakeTensor((1, 2048, 2, 100))) == "dense"
    assert tsd.get_mcsa_token_stats()["fallback_calls"] == 10


def test_dispatch_guards():
    with pytest.raises(RuntimeError):
        tsd.make_mcsa_token_dispatch(lambda *a, **k: None, num_layers=2, topk=1.5, context=FakeCtx(2), **_PLAIN)
    ctx = FakeCtx(1)
    d = tsd.make_mcsa_token_dispatch(lambda *a, **k: "dense", num_layers=1, context=ctx, **_PLAIN)
    t = FakeTensor((1, 2048, 2, 128))
    tsd.mcsa_token_begin_forward()
    d(t, t, t)
    with pytest.raises(RuntimeError):
        d(t, t, t)                         # a second sparse layer without a new step: numbering would drift
    tsd.reset_mcsa_token_state()
    assert tsd.get_mcsa_token_stats()["dispatch_calls"] == 0 and ctx.resets >= 1


def test_schedule_translation():
    """dense_steps / dense_layers / calibrate_every -> step and layer sets (reference :561-632)."""
    s = tsd.build_schedule(num_steps=50, dense_steps=10, dense_layers="0-1", calibrate_every=10, calibrate_steps=(9, 25))
    assert s == {"full_steps": list(range(10)), "full_layers": [0, 1], "calibrate_steps": [9, 25], "free_calibrate_step": 9}
    s = tsd.build_schedule(num_steps=50, dense_steps=10, dense_layers="0,3-4", calibrate_every=10)
    assert s["calibrate_steps"] == [9, 19, 29, 39] and s["full_layers"] == [0, 3, 4]       # 49 = last step: dropped
    s = tsd.build_schedule(num_steps=20, dense_steps=0, dense_layers="", calibrate_every=7)
    assert s["full_steps"] is None and s["calibrate_steps"] == [0, 7, 14] and s["free_calibrate_step"] is None
    s = tsd.build_schedule(num_steps=1, dense_steps=0, dense_layers="", calibrate_every=5)
    assert s["calibrate_steps"] == [0]
    for bad in (dict(num_steps=0, dense_steps=0), dict(num_steps=5, dense_steps=-1), dict(num_steps=5, dense_steps=0, calibrate_every=0)):
        kw = dict(dense_layers="", calibrate_every=10)
        kw.update(bad)
        with pytest.raises(ValueError):
            tsd.build_schedule(**kw)
    with pytest.raises(ValueError):
        tsd.build_schedule(num_steps=5, dense_steps=0, dense_layers="", calibrate_every=1, calibrate_steps=())
    tsd.validate_schedule(num_steps=10, calibrate_steps=[0, 5], update_steps=[3], approx_steps=None)
    with pytest.raises(ValueError):
        tsd.validate_schedule(num_steps=10, calibrate_steps=[0, 5], update_steps=[5], approx_steps=None)
    with pytest.raises(ValueError):
        tsd.validate_schedule(num_steps=10, calibrate_steps=[0], update_steps=[12], approx_steps=None)
    assert tsd.effective_density(sink_tokens=300, seq_len=38011, topk=0.25) == (9600 + 300) / 38011
    assert tsd.effective_density(sink_tokens=0, seq_len=0, topk=0.25) == 0.0


def test_eligibility_table():
    base = dict(ndim=4, is_cuda=True, dtype_ok=True, shapes_match=True, head_dim=128, seq_len_q=8192, seq_len_k=8192,
                has_attn_mask=False, is_causal=False, dropout_p=0.0, enable_gqa=False, scale=None, min_seq_len=4096,
                sparse_seq_len=None, has_parallel_config=False, sink_tokens=0)
    assert tsd.check_eligibility(**base) == (True, "", "")
    for change in (dict(has_parallel_config=True), dict(has_attn_mask=True), dict(is_causal=True), dict(dropout_p=0.1),
                   dict(enable_gqa=True), dict(ndim=3), dict(is_cuda=False), dict(dtype_ok=False), dict(shapes_match=False),
                   dict(seq_len_k=4096), dict(head_dim=100), dict(seq_len_q=301, seq_len_k=301), dict(sparse_seq_len=16384)):
        ok, reason, severity = tsd.check_eligibility(**{**base, **change})
        assert not ok and reason and severity == "fallback", change
    ok, _, severity = tsd.check_eligibility(**{**base, "sink_tokens": 8192})
    assert not ok and severity == "raise"


class _Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def test_parallel_config_falls_back_and_sink_splice():
    ctx = FakeCtx(1)
    seen = []

    def original(q, k, v, *a, **kw):
        seen.append((tuple(q.shape), kw.get("parallel_config")))
        return torch.ones(q.shape, dtype=torch.bfloat16)

    d = tsd.make_mcsa_token_dispatch(original, num_layers=1, topk=0.15, sink_tokens=8, context=ctx, **_PLAIN)
    t = FakeTensor((1, 2048, 2, 128))
    tsd.mcsa_token_begin_forward()
    pc = _Cfg(context_parallel_config=_Cfg(ulysses_degree=2, ring_degree=1))
    out = d(t, t, t, parallel_config=pc)                      # sequence shard: never sparsified here
    assert seen[-1] == ((1, 2048, 2, 128), pc) and tsd.get_mcsa_token_stats()["fallback_calls"] == 1
    assert ctx.forwards == []
    # eligible call: sparse path, then the first 8 query rows are recomputed densely and spliced in
    q = torch.zeros(1, 2048, 2, 128, dtype=torch.bfloat16)
    q.is_cuda_fake = True

    class Cuda(torch.Tensor):
        is_cuda = True
    qc = q.as_subclass(Cuda)
    out = d(qc, qc, qc)
    s = tsd.get_mcsa_token_stats()
    assert s["kernel_calls"] == 1 and s["splice_calls"] == 1 and s["sink_tokens"] == 8
    assert seen[-1][0] == (1, 8, 2, 128)
    assert tuple(out.shape) == (1, 2048, 2, 128) and bool((out[:, :8] == 1).all()) and bool((out[:, 8:] == 0).all())
    with pytest.raises(ValueError):
        tsd.make_mcsa_token_dispatch(original, num_layers=1, sink_tokens=0, allow_no_sink=False, context=FakeCtx(1))
    with pytest.raises(ValueError):
        tsd.make_mcsa_token_dispatch(original, num_layers=1, sink_tokens=4, use_chunk_selector=True, context=FakeCtx(1), **_PLAIN)
    with pytest.raises(ValueError):
        tsd.make_mcsa_token_dispatch(original, num_layers=1, cache_offload="residual", bias_correction=False, context=FakeCtx(1), **_PLAIN)


def test_kernel_problem_is_counted_and_served_densely():
    from mcsparse_b200 import _lib

    class Failing(FakeCtx):
        def forward(self, li, q, k, v, scale):
            raise _lib.KernelStatusError("kernel status 30")

    d = tsd.make_mcsa_token_dispatch(lambda *a, **k: "dense", num_layers=1, context=Failing(1), **_PLAIN)
    t = FakeTensor((1, 2048, 2, 128))
    tsd.mcsa_token_begin_forward()
    assert d(t, t, t) == "dense"
    s = tsd.get_mcsa_token_stats()
    assert s["kernel_error_calls"] == 1 and s["fallback_calls"] == 1 and s["kernel_calls"] == 0
    assert s["dispatch_calls"] == s["fallback_calls"] + s["dense_guard_calls"] + s["kernel_calls"]


def test_ticks_per_step():
    ctx = FakeCtx(1)
    tsd.make_mcsa_token_dispatch(lambda *a, **k: "dense", num_layers=1, context=ctx, ticks_per_step=2, **_PLAIN)
    for _ in range(6):
        tsd.mcsa_token_begin_forward()
    assert ctx.steps == 2 and tsd.get_mcsa_token_stats()["steps_ticked"] == 3


def test_with_ulysses_sparse_truth_table():
    """The branches of the reference wrapper (context_parallel.py:183-229) with fake tensors and configurations."""
    from mcsparse_b200.h3 import context_parallel as cp
    calls = []

    def inner(q, k, v, *a, **kw):
        calls.append(("kernel", kw.get("parallel_config")))
        return "sparse"

    def original(q, k, v, *a, **kw):
        calls.append(("original", kw.get("parallel_config")))
        return "dense"

    cp.reset_cp_stats()
    d = cp.with_ulysses_sparse(original, kind="mcsa_token", _inner_dispatch=inner, topk=0.15)
    t = FakeTensor((1, 2048, 2, 128))
    assert d(t, t, t) == "sparse" and cp.get_cp_stats() == {"cp_calls": 0, "local_calls": 1}
    assert d(t, t, t, parallel_config=_Cfg(context_parallel_config=None)) == "sparse"
    assert d(t, t, t, parallel_config=_Cfg(context_parallel_config=_Cfg(ulysses_degree=1, ring_degree=1))) == "sparse"
    assert cp.get_cp_stats() == {"cp_calls": 0, "local_calls": 3}
    assert all(c == ("kernel", None) for c in calls)            # past the wrapper the kernel never sees a parallel_config
    # unsupported arguments go to the original dispatch untouched, uncounted
    pc = _Cfg(context_parallel_config=_Cfg(ulysses_degree=2, ring_degree=1))
    for kw in (dict(attn_mask=object()), dict(is_causal=True), dict(dropout_p=0.1), dict(enable_gqa=True), dict(scale=0.5)):
        assert d(t, t, t, parallel_config=pc, **kw) == "dense"
    assert d(FakeTensor((1, 2048, 2, 128), cuda=False), t, t) == "dense"
    assert d(t, FakeTensor((1, 1024, 2, 128)), t) == "dense"
    assert calls[-1] == ("original", None) and cp.get_cp_stats() == {"cp_calls": 0, "local_calls": 3}
    with pytest.raises(ValueError, match="ring_degree"):
        d(t, t, t, parallel_config=_Cfg(context_parallel_config=_Cfg(ulysses_degree=2, ring_degree=2)))
    with pytest.raises(ValueError):
        cp.with_ulysses_sparse(original, kind="block_sparse")
    with pytest.raises(ValueError, match="LSE"):
        d.forward_op(None, t, t, t, return_lse=True)
    cp.reset_cp_stats()
    assert cp.get_cp_stats() == {"cp_calls": 0, "local_calls": 0}


def test_cfg_slots_give_each_forward_of_a_step_its_own_cache_slot():
    """Serial classifier-free guidance: two forwards per step, each with its own cache slot (reference :306-309, :840-851)."""
    class SlotCtx(FakeCtx):
        def __init__(self, n):
            super().__init__(n)
            self.slots = []

        def use_slot(self, name):
            self.slots.append(name)

    ctx = SlotCtx(1)
    tsd.make_mcsa_token_dispatch(lambda *a, **k: "dense", num_layers=1, context=ctx, ticks_per_step=2,
                                 cfg_slots=("cond", "uncond"), **_PLAIN)
    for _ in range(5):
        tsd.mcsa_token_begin_forward()
    assert ctx.slots == ["cond", "uncond", "cond", "uncond", "cond"] and ctx.steps == 2
    with pytest.raises(ValueError):
        tsd.make_mcsa_token_dispatch(lambda *a, **k: "dense", num_layers=1, context=SlotCtx(1), ticks_per_step=3,
                                     cfg_slots=("cond", "uncond"), **_PLAIN)


def test_discovery_window_lets_a_longer_sequence_replace_the_first_one():
    """Until the first sparse call has run, a strictly longer eligible call replaces the committed length (the
    reference's _maybe_upgrade_seq_len, :338-380); afterwards a second long length is left dense."""
    ctx = FakeCtx(2)
    ctx.caches[0].mode = "full"                   # the first layer is a dense-guard layer: no sparse call yet
    d = tsd.make_mcsa_token_dispatch(lambda *a, **k: "dense", num_layers=2, context=ctx, **_PLAIN)
    tsd.mcsa_token_begin_forward()
    refiner, packed, longer = FakeTensor((1, 2048, 2, 128)), FakeTensor((1, 8192, 2, 128)), FakeTensor((1, 16384, 2, 128))
    assert d(refiner, refiner, refiner) == "dense"                # eligible, dense guard: commits to 2048 provisionally
    assert tsd.get_mcsa_token_stats()["seq_len"] == 2048 and tsd.get_mcsa_token_stats()["kernel_calls"] == 0
    assert d(packed, packed, packed) == "dense"                   # longer, still discovering: replaces it, layer 0 again
    s = tsd.get_mcsa_token_stats()
    assert s["seq_len"] == 8192 and s["dense_guard_calls"] == 2 and s["fallback_calls"] == 0
    out = d(packed, packed, packed)                               # layer 1: the first sparse call
    assert torch.is_tensor(out) and tsd.get_mcsa_token_stats()["kernel_calls"] == 1
    assert d(refiner, refiner, refiner) == "dense"                # the shorter length now falls back ...
    assert d(longer, longer, longer) == "dense"                   # ... and so does a longer one: the window is closed
    s = tsd.get_mcsa_token_stats()
    assert s["fallback_calls"] == 2 and s["seq_len"] == 8192
    ok, reason, sev = tsd.check_eligibility(ndim=4, is_cuda=True, dtype_is_bf16=True, shapes_match=True, head_dim=128,
                                            seq_len_q=9000, seq_len_k=9000, has_attn_mask=False, is_causal=False,
                                            dropout_p=0.0, enable_gqa=False, has_parallel_config=False, scale=None,
                                            sink_tokens=0, sparse_seq_len=8192, min_seq_len=4096, discovering=True)
    assert ok and not reason


def test_context_cache_slots_share_the_step_clock():
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
    ctx = TokenSparseContext(TokenSparseConfig(topk=0.1, calibrate_steps=[0, 4]), num_layers=2)
    default = list(ctx.caches)
    ctx.step(); ctx.step(); ctx.step()
    with ctx.cache_context("uncond"):
        assert len(ctx.caches) == 2 and all(a is not b for a, b in zip(ctx.caches, default))
        assert [c._step_count for c in ctx.caches] == [3, 3]          # a slot that shows up later joins the clock
        uncond = list(ctx.caches)
    assert ctx.caches == default and ctx._active_slot == "_default"
    ctx.step()
    assert [c._step_count for c in default + uncond] == [4, 4, 4, 4]
    assert uncond[0].mode == "calibrate"                               # step 4 is an anchor step in every slot
    ctx.use_slot("uncond")
    assert ctx.caches == uncond
    ctx.reset()
    assert ctx.caches == default and [c._step_count for c in default + uncond] == [0, 0, 0, 0]
