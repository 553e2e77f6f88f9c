"""Attention-dispatch adapter for the token-sparse path (B200 build).

Keeps the contract of the reference's ``mcsparse/h3/token_sparse_dispatch.py``: a factory
``make_mcsa_token_dispatch`` (:778) returns a ``dispatch(query, key, value, attn_mask=None, dropout_p=0.0,
is_causal=False, scale=None, enable_gqa=False, attention_kwargs=None, *, backend=None, parallel_config=None)``
(:1126-1139) that takes BTHD tensors and returns a contiguous BTHD tensor in ``query.dtype`` (:1245).
Every call increments ``dispatch_calls`` and exactly one of ``fallback_calls`` (ineligible call routed to
the original dispatch, :1179-1186), ``dense_guard_calls`` (full layer / full step, :1225-1230) or
``kernel_calls`` (:1248); anchor steps also count ``calibrate_calls`` / ``full_calibrate_calls``
(:1232-1236).  Layers are numbered by counting eligible calls; a forward pre-hook on the model ticks the
step clock through ``mcsa_token_begin_forward`` (:274).

Mirrored host logic: the schedule translation of ``dense_steps`` / ``dense_layers`` / ``calibrate_every``
(:561-632) and its validation (:635-666), the effective density (:669-689), the eligibility table with its
two severities (:696-772; a call under context parallelism is ineligible here and belongs to
``mcsparse_b200.h3.context_parallel.with_ulysses_sparse``), the query-side prefix splice for
``sink_tokens > 0`` (:1086-1124) and ``ticks_per_step`` (:274-309).  The index / residual offload knobs work as in
the reference but default to off: on a 180 GB part the metadata normally stays in HBM.

One addition: a kernel problem (a negative return code of the C ABI, or a non-zero device status word) is
counted in ``kernel_error_calls`` and ``fallback_calls`` and the call is served by the original dispatch.
"""

from __future__ import annotations

import math
import sys
from typing import Callable, Optional, Sequence

BLKQ = 128
TILE_N = 128
# the reference's dispatch lists (128, 144); here every stage also exists for the other sizes of its kernel table and for 64
SUPPORTED_HEAD_DIMS = (64, 96, 128, 144, 160, 192, 256)
DEFAULT_TOPK = 0.25
DEFAULT_NUM_STEPS = 50
DEFAULT_DENSE_STEPS = 10
DEFAULT_DENSE_LAYERS = "0-1"
DEFAULT_CALIBRATE_EVERY = 10
DEFAULT_CALIBRATE_STEPS = (9,)
DEFAULT_MIN_SEQ_LEN = 4096

_STATS = {
    "dispatch_calls": 0, "kernel_calls": 0, "dense_guard_calls": 0, "fallback_calls": 0, "kernel_error_calls": 0,
    "steps_ticked": 0, "layers_per_step": 0, "calibrate_calls": 0, "full_calibrate_calls": 0, "splice_calls": 0,
    "sink_tokens": 0, "seq_len": 0, "batch": 0, "nominal_density": 0.0, "effective_density": 0.0,
}
_CONFIG_STATS = ("sink_tokens", "nominal_density")
_CTX = {"ctx": None, "layer_cursor": 0, "sparse_seq_len": None, "seen_seq_lens": {}, "tick": 0, "ticks_per_step": 1,
        "cfg_slots": ()}


def get_mcsa_token_stats() -> dict:
    out = dict(_STATS)
    out["seen_seq_lens"] = dict(sorted(_CTX["seen_seq_lens"].items()))
    return out


def reset_mcsa_token_state() -> None:
    """Per-sample reset: counters, layer/step clocks and every layer cache (configuration facts stay)."""
    for k, v in list(_STATS.items()):
        if k not in _CONFIG_STATS:
            _STATS[k] = 0.0 if isinstance(v, float) else 0
    _CTX.update(layer_cursor=0, sparse_seq_len=None, seen_seq_lens={}, tick=0)
    if _CTX["ctx"] is not None:
        _CTX["ctx"].reset()


def mcsa_token_begin_forward() -> None:
    """Call once per model forward, before its first attention call.  ``ticks_per_step`` forwards make one
    denoising step (two under serial classifier-free guidance, :274-309)."""
    if _CTX["ctx"] is None:
        raise RuntimeError("[mcsa-token] begin_forward called before make_mcsa_token_dispatch")
    if _CTX["tick"] > 0:
        if _STATS["layers_per_step"] and _CTX["layer_cursor"] != _STATS["layers_per_step"]:
            raise RuntimeError(
                f"[mcsa-token] step saw {_CTX['layer_cursor']} sparse layers, earlier steps saw "
                f"{_STATS['layers_per_step']}: the layer numbering would drift")
        _STATS["layers_per_step"] = _CTX["layer_cursor"]
    _CTX["tick"] += 1
    if _CTX["tick"] > 1 and (_CTX["tick"] - 1) % _CTX["ticks_per_step"] == 0:
        _CTX["ctx"].step()
    _CTX["layer_cursor"] = 0
    _STATS["steps_ticked"] = (_CTX["tick"] - 1) // _CTX["ticks_per_step"] + 1
    # forwards that alternate within a step (serial classifier-free guidance) each get their own cache slot (:306-309)
    slots = _CTX["cfg_slots"]
    if slots and hasattr(_CTX["ctx"], "use_slot"):
        _CTX["ctx"].use_slot(slots[(_CTX["tick"] - 1) % len(slots)])


# ------------------------------------------------------------------------------------------------ schedule
def _parse_layer_ranges(spec) -> frozenset:
    """"0-1,5" -> {0, 1, 5} (:542-558)."""
    layers = set()
    for item in str(spec or "").split(","):
        item = item.strip()
        if not item:
            continue
        if "-" in item:
            lo, hi = item.split("-", 1)
            layers.update(range(int(lo), int(hi) + 1))
        else:
            layers.add(int(item))
    return frozenset(layers)


def build_schedule(*, num_steps: int, dense_steps: int, dense_layers, calibrate_every: int, calibrate_steps=None) -> dict:
    """``dense_steps`` leading full steps and ``dense_layers`` full layers as step / layer sets (:561-632).

    The first anchor step defaults to the last dense step: a step in both sets runs ``full_calibrate``, which
    yields output, LSE, selection and residual from the one dense pass that step pays for anyway.  Without
    explicit ``calibrate_steps`` the anchor steps repeat every ``calibrate_every`` steps, and one that would
    fall on the very last step (nothing left to reuse it) is dropped unless it is the only one."""
    if num_steps <= 0:
        raise ValueError(f"num_steps must be positive, got {num_steps}")
    if dense_steps < 0:
        raise ValueError(f"dense_steps must be >= 0, got {dense_steps}")
    if calibrate_every <= 0:
        raise ValueError(f"calibrate_every must be positive, got {calibrate_every}")
    full_steps = list(range(min(dense_steps, num_steps)))
    if calibrate_steps is not None:
        cal = sorted({int(s) for s in calibrate_steps})
        if not cal:
            raise ValueError("calibrate_steps was given but is empty")
    else:
        cal = list(range(max(0, dense_steps - 1), num_steps, calibrate_every))
        if len(cal) > 1 and cal[-1] == num_steps - 1:
            cal.pop()
        cal = cal or [0]
    return {"full_steps": full_steps or None, "full_layers": sorted(_parse_layer_ranges(dense_layers)),
            "calibrate_steps": cal, "free_calibrate_step": cal[0] if cal[0] in full_steps else None}


def validate_schedule(*, num_steps, calibrate_steps, update_steps, approx_steps) -> None:
    """A step may be in only one of the calibrate / update / approx lists and must lie in [0, num_steps)
    (:635-666); full steps may overlap calibrate steps (that is ``full_calibrate``)."""
    named = [("calibrate_steps", set(calibrate_steps or [])), ("update_steps", set(update_steps or [])),
             ("approx_steps", set(approx_steps or []))]
    for i, (na, a) in enumerate(named):
        for nb, b in named[i + 1:]:
            if a & b:
                raise ValueError(f"{na} and {nb} overlap at {sorted(a & b)}")
    for name, steps in named:
        bad = sorted(s for s in steps if not (0 <= s < num_steps))
        if bad:
            raise ValueError(f"{name} contains {bad}, outside [0, {num_steps})")


def effective_density(*, sink_tokens: int, seq_len: int, topk: float, tile_n: int = TILE_N) -> float:
    """Fraction of the keys attended: the sink adds to the tile-aligned top-k budget (:669-689)."""
    if seq_len <= 0:
        return 0.0
    budget = max(1, int(topk * seq_len))
    budget = ((budget + tile_n - 1) // tile_n) * tile_n
    return min(seq_len, budget + max(0, sink_tokens)) / seq_len


# --------------------------------------------------------------------------------------------- eligibility
def check_eligibility(*, ndim, is_cuda, dtype_is_bf16=None, shapes_match, head_dim, seq_len_q, seq_len_k, has_attn_mask,
                      is_causal, dropout_p, enable_gqa, has_parallel_config=False, scale=None, sink_tokens=0,
                      sparse_seq_len=None, min_seq_len=DEFAULT_MIN_SEQ_LEN, discovering=False, dtype_ok=None):
    """(ok, reason, severity).  "fallback": the kernel cannot express the call, the original dispatch serves it;
    "raise": the configuration itself is wrong (:696-772).  Parameter names as the reference's; ``dtype_is_bf16`` says
    whether the dtype is one the kernels take (bf16, and here also fp16; ``dtype_ok`` is a synonym).  Any softmax
    scale is supported by the kernels, so ``scale`` never disqualifies a call.  ``discovering``: no sparse call has
    run yet, so a strictly longer sequence length may still replace the one committed to (:747-761)."""
    if dtype_ok is None:
        dtype_ok = bool(dtype_is_bf16)
    if has_parallel_config:
        # sequence shards: neither a global selection nor a [0, P) sink range means anything on 1/N of the tokens
        return False, "parallel_config is not None (context parallelism)", "fallback"
    if has_attn_mask or is_causal or (dropout_p or 0.0) != 0.0 or enable_gqa:
        return False, "mask / causal / dropout / gqa are not supported", "fallback"
    if ndim != 4:
        return False, "query is not 4-D (B, T, H, D)", "fallback"
    if not is_cuda:
        return False, "tensors are not on a CUDA device", "fallback"
    if not dtype_ok:
        return False, "dtype is not bf16/fp16", "fallback"
    if not shapes_match:
        return False, "q/k/v shapes differ (cross-attention or GQA)", "fallback"
    if seq_len_q != seq_len_k:
        return False, f"L_q={seq_len_q} != L_k={seq_len_k} (cross-attention)", "fallback"
    if head_dim not in SUPPORTED_HEAD_DIMS:
        return False, f"head_dim {head_dim} not supported by the kernel", "fallback"
    if seq_len_q < max(min_seq_len, BLKQ):
        return False, f"sequence length {seq_len_q} below the sparse floor {max(min_seq_len, BLKQ)}", "fallback"
    if sparse_seq_len is not None and seq_len_q != sparse_seq_len:
        if not (discovering and seq_len_q > sparse_seq_len):
            return False, (f"L={seq_len_q} is a second long sequence length (already committed to {sparse_seq_len}): "
                           "only one length is sparsified"), "fallback"
    if sink_tokens >= seq_len_k:
        return False, f"sink_tokens={sink_tokens} >= L_k={seq_len_k}: nothing would be sparse", "raise"
    return True, "", ""


# ------------------------------------------------------------------------------------------------- factory
def make_mcsa_token_dispatch(original_dispatch: Callable, *, sink_tokens: int = 0, num_layers: Optional[int] = None,
                             num_steps: int = DEFAULT_NUM_STEPS, topk: float = DEFAULT_TOPK,
                             dense_steps: int = DEFAULT_DENSE_STEPS, dense_layers=DEFAULT_DENSE_LAYERS,
                             calibrate_every: int = DEFAULT_CALIBRATE_EVERY,
                             calibrate_steps: Optional[Sequence[int]] = DEFAULT_CALIBRATE_STEPS, pca_reorder: bool = True,
                             pca_pow_iters: int = 4, pca_proj_dim=None, bias_correction: bool = True,
                             selection_mode: str = "topk", topp: Optional[float] = None, adaptive_layers: bool = False,
                             use_chunk_selector: bool = False, chunk_selector_size: int = 16384,
                             offload_indices: bool = False, cache_offload: str = "none", offload_prefetch_ahead: int = 1,
                             update_steps: Optional[Sequence[int]] = None, approx_steps: Optional[Sequence[int]] = None,
                             full_attn_impl: str = "native", allow_no_sink: bool = False,
                             min_seq_len: int = DEFAULT_MIN_SEQ_LEN, ticks_per_step: int = 1, cfg_slots=(),
                             full_steps: Optional[Sequence[int]] = None, full_layers: Sequence[int] = (),
                             sink_ranges=None, context=None) -> Callable:
    """Build the dispatch function (argument names and meaning as the reference's factory, :778-808).

    ``sink_tokens`` is the length of the exact prefix: its keys are always attended (``sink_ranges = [(0, P)]``)
    and its query rows are recomputed densely by the original dispatch and spliced in.  ``dense_steps`` /
    ``dense_layers`` / ``calibrate_every`` / ``calibrate_steps`` go through :func:`build_schedule`;
    ``full_steps`` / ``full_layers`` / ``sink_ranges`` may instead be given directly.  ``context`` may inject a
    ready TokenSparseContext-like object (``forward(li, q, k, v, scale)``, ``caches[li].mode``, ``step()``,
    ``reset()``), which the CPU tests use.  ``offload_indices`` / ``cache_offload`` / ``offload_prefetch_ahead`` park
    indices / residual in pinned host memory between uses (default off, where the reference's factory defaults to on:
    a 180 GB part keeps them resident); ``full_attn_impl`` is accepted for call compatibility and has no effect: there
    is one dense implementation.  ``ticks_per_step`` forwards make one denoising step, and ``cfg_slots`` (e.g.
    ``("cond", "uncond")``) gives each of them its own cache slot (:840-851).  The other defaults are the reference's
    (``DEFAULT_*``; ``sink_tokens`` is required there and 0 is refused without ``allow_no_sink=True``, as here).
    """
    sink_tokens = int(sink_tokens)
    if sink_tokens < 0:
        raise ValueError(f"sink_tokens must be >= 0, got {sink_tokens}")
    if sink_tokens == 0 and not allow_no_sink:
        raise ValueError("sink_tokens=0 without allow_no_sink=True: the conditioning prefix could be dropped by top-k")
    if not (0.0 < topk <= 1.0):
        raise RuntimeError(f"[mcsa-token] topk must be in (0, 1], got {topk}")
    if num_layers is not None and num_layers < 1:
        raise RuntimeError("[mcsa-token] num_layers must be positive")
    if adaptive_layers and num_layers is None:
        raise ValueError("adaptive_layers=True requires num_layers")
    if bias_correction and pca_reorder and approx_steps:
        raise ValueError("bias_correction + pca_reorder + approx_steps is incoherent: an approx step renews the "
                         "permutation, which invalidates the residual from then on")
    if sink_tokens and use_chunk_selector:
        raise ValueError("sink_tokens>0 cannot be combined with use_chunk_selector=True")
    if chunk_selector_size <= 0 or (use_chunk_selector and chunk_selector_size % TILE_N):
        raise ValueError(f"chunk_selector_size must be a positive multiple of {TILE_N}, got {chunk_selector_size}")
    if cache_offload not in ("none", "residual"):
        raise ValueError(f"cache_offload must be 'none' or 'residual', got {cache_offload!r}")
    if offload_prefetch_ahead not in (0, 1):
        raise ValueError(f"offload_prefetch_ahead only supports 0 or 1, got {offload_prefetch_ahead}")
    if cache_offload == "residual" and not bias_correction:
        raise ValueError("cache_offload='residual' requires bias_correction=True")
    sched = build_schedule(num_steps=num_steps, dense_steps=dense_steps, dense_layers=dense_layers,
                           calibrate_every=calibrate_every, calibrate_steps=calibrate_steps)
    validate_schedule(num_steps=num_steps, calibrate_steps=sched["calibrate_steps"], update_steps=update_steps,
                      approx_steps=approx_steps)
    full_steps = sorted(set(full_steps or []) | set(sched["full_steps"] or [])) or None
    full_layers_set = frozenset(full_layers) | frozenset(sched["full_layers"])
    if sink_ranges is None and sink_tokens > 0:
        sink_ranges = [(0, sink_tokens)]
    n_sink = sum(e - s for s, e in (sink_ranges or []))
    if context is None:
        from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
        cfg = TokenSparseConfig(topk=topk, topp=topp, selection_mode=selection_mode,
                                calibrate_steps=sched["calibrate_steps"],
                                update_steps=list(update_steps) if update_steps else None,
                                approx_steps=list(approx_steps) if approx_steps else None,
                                full_steps=full_steps, full_layers=sorted(full_layers_set), sink_ranges=sink_ranges,
                                bias_correction=bias_correction, pca_reorder=pca_reorder, pca_pow_iters=pca_pow_iters,
                                pca_proj_dim=pca_proj_dim, adaptive_layers=adaptive_layers,
                                use_chunk_selector=use_chunk_selector, chunk_selector_size=chunk_selector_size,
                                offload_indices=offload_indices, cache_offload=cache_offload,
                                offload_prefetch_ahead=offload_prefetch_ahead)
        context = TokenSparseContext(cfg, num_layers)
    if _CTX["ctx"] is not None and hasattr(_CTX["ctx"], "reset"):
        _CTX["ctx"].reset()                                       # release the previous context's caches first
    _CTX["ctx"] = context
    _CTX["ticks_per_step"] = max(1, int(ticks_per_step))
    _CTX["cfg_slots"] = tuple(cfg_slots)
    if _CTX["cfg_slots"] and _CTX["ticks_per_step"] % len(_CTX["cfg_slots"]):
        raise ValueError(f"cfg_slots={cfg_slots!r} needs ticks_per_step to be a multiple of {len(_CTX['cfg_slots'])}")
    reset_mcsa_token_state()
    _STATS["nominal_density"] = float(topk)
    _STATS["sink_tokens"] = sink_tokens

    def _splice_prefix_dense(out, query, key, value):
        """Query side of the sink (:1086-1124): the first ``sink_tokens`` query rows attend the whole sequence
        exactly; they are recomputed by the original dispatch and replace the sparse rows."""
        if sink_tokens <= 0:
            return out
        import torch
        dense_prefix = original_dispatch(query[:, :sink_tokens].contiguous(), key, value, None, 0.0, False, None, False,
                                         None, backend=None, parallel_config=None)
        if tuple(dense_prefix.shape[:2]) != (query.shape[0], sink_tokens):
            raise RuntimeError(f"dense prefix attention returned {tuple(dense_prefix.shape)}, expected batch="
                               f"{query.shape[0]} rows={sink_tokens}: the original dispatch does not accept L_q != L_k")
        _STATS["splice_calls"] += 1
        return torch.cat([dense_prefix.to(out.dtype), out[:, sink_tokens:]], dim=1)

    def dispatch(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
                 attention_kwargs=None, *, backend=None, parallel_config=None, out_peers=None):
        """``out_peers`` (not part of the reference signature) is handed down by the Ulysses wrapper: when the
        call ends in the sparse kernel its epilogue stores the rows into the owners' sequence shards and the
        function returns None; in every other case the tensor is returned and the wrapper reshards it."""
        _STATS["dispatch_calls"] += 1

        def _dense():
            return original_dispatch(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa,
                                     attention_kwargs, backend=backend, parallel_config=parallel_config)

        is_4d = getattr(query, "ndim", 0) == 4
        if is_4d:
            T = query.shape[1]
            _CTX["seen_seq_lens"][T] = _CTX["seen_seq_lens"].get(T, 0) + 1
        dt = str(getattr(query, "dtype", ""))
        ok, reason, severity = check_eligibility(
            ndim=getattr(query, "ndim", 0), is_cuda=bool(getattr(query, "is_cuda", False)),
            dtype_ok=dt in ("torch.bfloat16", "torch.float16"),
            shapes_match=(tuple(query.shape) == tuple(key.shape) == tuple(value.shape)),
            head_dim=query.shape[-1] if is_4d else -1, seq_len_q=query.shape[1] if is_4d else -1,
            seq_len_k=key.shape[1] if getattr(key, "ndim", 0) == 4 else -1, has_attn_mask=attn_mask is not None,
            is_causal=bool(is_causal), dropout_p=float(dropout_p or 0.0), enable_gqa=bool(enable_gqa), scale=scale,
            min_seq_len=min_seq_len, sparse_seq_len=_CTX["sparse_seq_len"],
            has_parallel_config=parallel_config is not None, sink_tokens=sink_tokens,
            discovering=_STATS["kernel_calls"] == 0)
        if not ok:
            if severity == "raise":
                raise RuntimeError(f"[mcsa-token] {reason}")
            _STATS["fallback_calls"] += 1                         # consumes no layer index
            return _dense()
        B, T, H, D = query.shape
        if _CTX["sparse_seq_len"] is not None and T > _CTX["sparse_seq_len"]:
            # a longer eligible call inside the discovery window (no sparse call has run, so no cache exists): it
            # replaces the provisional length, and the layer numbering of this forward starts over (:350-380)
            print(f"[mcsa-token] sparse length {_CTX['sparse_seq_len']} -> {T}: a longer eligible call appeared before the "
                  "first sparse call", file=sys.stderr, flush=True)
            _CTX["sparse_seq_len"] = None
            _CTX["layer_cursor"] = 0
        if _CTX["sparse_seq_len"] is None:
            _CTX["sparse_seq_len"] = T
            _STATS["seq_len"], _STATS["batch"] = T, B
            _STATS["effective_density"] = (effective_density(sink_tokens=n_sink, seq_len=T, topk=topk)
                                           if sink_tokens else min(1.0, (n_sink + topk * T) / T))
        li = _CTX["layer_cursor"]
        _CTX["layer_cursor"] += 1
        n_layers = num_layers if num_layers is not None else (_STATS["layers_per_step"] or None)
        if n_layers is not None and li >= n_layers:
            raise RuntimeError(f"[mcsa-token] layer index {li} >= num_layers {n_layers}: "
                               "mcsa_token_begin_forward was not called at the start of the step")
        mode = context.caches[li].mode if li < len(context.caches) else context.cache(li).mode
        if li in full_layers_set or mode == "full":
            _STATS["dense_guard_calls"] += 1
            return _dense()
        if mode == "calibrate":
            _STATS["calibrate_calls"] += 1
        elif mode == "full_calibrate":
            _STATS["full_calibrate_calls"] += 1
        from mcsparse_b200 import _lib
        peers = out_peers if (out_peers is not None and sink_tokens <= 0) else None
        try:
            # BTHD -> BHSD views; the kernel takes the strides, nothing is copied on the way in
            if peers is not None:
                out = context.forward(li, query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), scale,
                                      out_peers=peers)
            else:
                out = context.forward(li, query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), scale)
        except (_lib.KernelLaunchError, _lib.KernelStatusError) as e:
            _STATS["kernel_error_calls"] += 1
            _STATS["fallback_calls"] += 1
            print(f"[mcsa-token] layer {li}: kernel problem ({e}); this call is served by the original dispatch",
                  file=sys.stderr, flush=True)
            if li < len(context.caches) and hasattr(context.caches[li], "reset"):
                context.caches[li].reset()                        # nothing half-built survives
            return _dense()
        _STATS["kernel_calls"] += 1
        if out is None:
            return None                                           # rows already stored into the peers' shards
        # the state machine hands back (B, H, T, D) storage written through a (B, T, H, D) view when it can;
        # otherwise this is the one copy on the way out
        out = out.transpose(1, 2)
        if not out.is_contiguous():
            out = out.contiguous()
        if out.dtype != query.dtype:
            out = out.to(query.dtype)
        return _splice_prefix_dense(out, query, key, value)

    return dispatch


__all__ = ["get_mcsa_token_stats", "make_mcsa_token_dispatch", "mcsa_token_begin_forward", "reset_mcsa_token_state",
           "build_schedule", "validate_schedule", "effective_density", "check_eligibility"]
