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

Only the parts that touch the accelerated path are mirrored; prefix splicing for ``sink_tokens > 0``
(:1086-1124) is not (the reference's CLI default is 0).
"""

from __future__ import annotations

from typing import Callable, Optional, Sequence

_STATS = {
    "dispatch_calls": 0, "kernel_calls": 0, "dense_guard_calls": 0, "fallback_calls": 0,
    "steps_ticked": 0, "layers_per_step": 0, "calibrate_calls": 0, "full_calibrate_calls": 0,
    "seq_len": 0, "batch": 0, "nominal_density": 0.0, "effective_density": 0.0,
}
_CTX = {"ctx": None, "layer_cursor": 0, "sparse_seq_len": None, "seen_seq_lens": {}, "first_step": True}


def get_mcsa_token_stats() -> dict:
    out = dict(_STATS)
    out["seen_seq_lens"] = dict(sorted(_CTX["seen_seq_lens"].items()))
    return out


def reset_mcsa_token_state() -> None:
    """Per-sample reset: counters, layer/step clocks and every layer cache."""
    for k, v in list(_STATS.items()):
        _STATS[k] = 0.0 if isinstance(v, float) else 0
    _CTX.update(layer_cursor=0, sparse_seq_len=None, seen_seq_lens={}, first_step=True)
    if _CTX["ctx"] is not None:
        _CTX["ctx"].reset()


def mcsa_token_begin_forward() -> None:
    """Call once per model forward (denoising step), before its first attention call."""
    if _CTX["ctx"] is None:
        raise RuntimeError("[mcsa-token] begin_forward called before make_mcsa_token_dispatch")
    if not _CTX["first_step"]:
        if _STATS["layers_per_step"] and _CTX["layer_cursor"] != _STATS["layers_per_step"]:
            raise RuntimeError(
                f"[mcsa-token] step saw {_CTX['layer_cursor']} sparse layers, earlier steps saw "
                f"{_STATS['layers_per_step']}: the layer numbering would drift")
        _STATS["layers_per_step"] = _CTX["layer_cursor"]
        _CTX["ctx"].step()
    _CTX["first_step"] = False
    _CTX["layer_cursor"] = 0
    _STATS["steps_ticked"] += 1


def check_eligibility(*, ndim, is_cuda, dtype_ok, shapes_match, head_dim, seq_len_q, seq_len_k, has_attn_mask, is_causal,
                      dropout_p, enable_gqa, scale, min_seq_len, sparse_seq_len):
    """(ok, reason).  Ineligible calls fall back to the original dispatch (reference :696-772)."""
    if ndim != 4:
        return False, "query is not 4-D (B, T, H, D)"
    if not is_cuda:
        return False, "tensors are not on a CUDA device"
    if not dtype_ok:
        return False, "dtype is not bf16/fp16"
    if not shapes_match:
        return False, "q/k/v shapes differ (cross-attention or GQA)"
    if head_dim not in (64, 128):
        return False, f"head_dim {head_dim} not supported by the kernel"
    if has_attn_mask or is_causal or (dropout_p or 0.0) != 0.0 or enable_gqa:
        return False, "mask / causal / dropout / gqa are not supported"
    if seq_len_q < min_seq_len or seq_len_q != seq_len_k:
        return False, f"sequence length {seq_len_q} below the floor {min_seq_len} or not self-attention"
    if sparse_seq_len is not None and seq_len_q != sparse_seq_len:
        return False, "a second long sequence length: only the first one is sparsified"
    return True, ""


def make_mcsa_token_dispatch(original_dispatch: Callable, *, num_layers: int, topk: float = 0.15,
                             calibrate_steps: Optional[Sequence[int]] = (0,), update_steps: Optional[Sequence[int]] = None,
                             full_steps: Optional[Sequence[int]] = None, full_layers: Sequence[int] = (),
                             sink_ranges=None, bias_correction: bool = True, pca_reorder: bool = True,
                             pca_pow_iters: int = 4, min_seq_len: int = 1024, context=None) -> Callable:
    """Build the dispatch function.  ``context`` may inject a ready TokenSparseContext-like object
    (``forward(li, q, k, v, scale)``, ``caches[li].mode``, ``step()``, ``reset()``), which the CPU tests use."""
    if not (0.0 < topk <= 1.0):
        raise RuntimeError(f"[mcsa-token] topk must be in (0, 1], got {topk}")
    if num_layers < 1:
        raise RuntimeError("[mcsa-token] num_layers must be positive")
    if context is None:
        from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig, TokenSparseContext
        cfg = TokenSparseConfig(topk=topk, calibrate_steps=list(calibrate_steps) if calibrate_steps else None,
                                update_steps=list(update_steps) if update_steps else None,
                                full_steps=list(full_steps) if full_steps else None, full_layers=list(full_layers),
                                sink_ranges=sink_ranges, bias_correction=bias_correction, pca_reorder=pca_reorder,
                                pca_pow_iters=pca_pow_iters)
        context = TokenSparseContext(cfg, num_layers)
    if _CTX["ctx"] is not None and hasattr(_CTX["ctx"], "reset"):
        _CTX["ctx"].reset()                                       # release the previous context's caches first
    _CTX["ctx"] = context
    reset_mcsa_token_state()
    _STATS["nominal_density"] = float(topk)
    full_layers_set = set(full_layers)
    n_sink = sum(e - s for s, e in (sink_ranges or []))

    def dispatch(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
                 attention_kwargs=None, *, backend=None, parallel_config=None):
        _STATS["dispatch_calls"] += 1

        def _dense():
            return original_dispatch(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa,
                                     attention_kwargs, backend=backend, parallel_config=parallel_config)

        is_4d = getattr(query, "ndim", 0) == 4
        if is_4d:
            T = query.shape[1]
            _CTX["seen_seq_lens"][T] = _CTX["seen_seq_lens"].get(T, 0) + 1
        dt = str(getattr(query, "dtype", ""))
        ok, _reason = check_eligibility(
            ndim=getattr(query, "ndim", 0), is_cuda=bool(getattr(query, "is_cuda", False)),
            dtype_ok=dt in ("torch.bfloat16", "torch.float16"),
            shapes_match=(tuple(query.shape) == tuple(key.shape) == tuple(value.shape)),
            head_dim=query.shape[-1] if is_4d else -1, seq_len_q=query.shape[1] if is_4d else -1,
            seq_len_k=key.shape[1] if getattr(key, "ndim", 0) == 4 else -1, has_attn_mask=attn_mask is not None,
            is_causal=bool(is_causal), dropout_p=float(dropout_p or 0.0), enable_gqa=bool(enable_gqa), scale=scale,
            min_seq_len=min_seq_len, sparse_seq_len=_CTX["sparse_seq_len"])
        if not ok:
            _STATS["fallback_calls"] += 1                         # consumes no layer index
            return _dense()
        B, T, H, D = query.shape
        if _CTX["sparse_seq_len"] is None:
            _CTX["sparse_seq_len"] = T
            _STATS["seq_len"], _STATS["batch"] = T, B
            _STATS["effective_density"] = min(1.0, (n_sink + topk * T) / T)
        li = _CTX["layer_cursor"]
        _CTX["layer_cursor"] += 1
        if li >= num_layers:
            raise RuntimeError(f"[mcsa-token] layer index {li} >= num_layers {num_layers}: "
                               "mcsa_token_begin_forward was not called at the start of the step")
        mode = context.caches[li].mode
        if li in full_layers_set or mode == "full":
            _STATS["dense_guard_calls"] += 1
            return _dense()
        if mode == "calibrate":
            _STATS["calibrate_calls"] += 1
        elif mode == "full_calibrate":
            _STATS["full_calibrate_calls"] += 1
        # BTHD -> BHSD views; the kernel takes the strides, nothing is copied on the way in
        out = context.forward(li, query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), scale)
        out = out.transpose(1, 2).contiguous()
        if out.dtype != query.dtype:
            out = out.to(query.dtype)
        _STATS["kernel_calls"] += 1
        return out

    return dispatch
