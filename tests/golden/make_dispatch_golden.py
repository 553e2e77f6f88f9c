"""Writes ``dispatch_logic.json``: outputs of the reference's pure dispatch-side functions over grids of arguments
(``build_schedule``, ``validate_schedule``, ``effective_density``, ``check_eligibility`` of
mcsparse/h3/token_sparse_dispatch.py and the per-step mode of ``TokenSparseCache``,
mcsparse/kernels/flash_mcsa/token_sparse.py:233-247), produced by importing the reference on the CPU.
Usage: ``python tests/golden/make_dispatch_golden.py <reference root>``; ``tests/test_dispatch_golden.py`` replays
the same calls on this package."""

from __future__ import annotations

import itertools
import json
import sys
from pathlib import Path


def _jsonable(x):
    if isinstance(x, dict):
        return {str(k): _jsonable(v) for k, v in x.items()}
    if isinstance(x, (set, frozenset)):
        return sorted(_jsonable(v) for v in x)
    if isinstance(x, (list, tuple)):
        return [_jsonable(v) for v in x]
    return x


def _call(fn, kwargs):
    try:
        return {"ok": _jsonable(fn(**kwargs))}
    except Exception as e:                                   # the error type is part of the contract
        return {"error": type(e).__name__}


ELIGIBLE = dict(ndim=4, is_cuda=True, dtype_is_bf16=True, shapes_match=True, head_dim=128, seq_len_q=8192, seq_len_k=8192,
                has_attn_mask=False, is_causal=False, dropout_p=0.0, enable_gqa=False, has_parallel_config=False,
                scale=None, sink_tokens=0, sparse_seq_len=None, min_seq_len=4096, discovering=False)
ELIGIBILITY_CHANGES = [
    {}, {"ndim": 3}, {"is_cuda": False}, {"dtype_is_bf16": False}, {"shapes_match": False}, {"head_dim": 64}, {"head_dim": 96},
    {"head_dim": 256}, {"seq_len_k": 4096}, {"has_attn_mask": True}, {"is_causal": True}, {"dropout_p": 0.1}, {"enable_gqa": True},
    {"has_parallel_config": True}, {"sink_tokens": 64}, {"sink_tokens": 8192}, {"sink_tokens": 9000},
    {"seq_len_q": 301, "seq_len_k": 301}, {"seq_len_q": 100, "seq_len_k": 100, "min_seq_len": 0},
    {"seq_len_q": 4095, "seq_len_k": 4095}, {"seq_len_q": 4096, "seq_len_k": 4096}, {"sparse_seq_len": 8192},
    {"sparse_seq_len": 16384}, {"sparse_seq_len": 4096}, {"sparse_seq_len": 4096, "discovering": True},
    {"sparse_seq_len": 16384, "discovering": True}, {"min_seq_len": 16384}, {"has_attn_mask": True, "sink_tokens": 9000},
]


def main(root: str) -> None:
    sys.path.insert(0, root)
    from mcsparse.h3 import token_sparse_dispatch as tsd
    from mcsparse.kernels.flash_mcsa.token_sparse import TokenSparseCache, TokenSparseConfig

    out = {"build_schedule": [], "validate_schedule": [], "effective_density": [], "check_eligibility": [], "modes": []}
    for ns, ds, dl, ce, cs in itertools.product((1, 20, 50), (0, 1, 10, 60), ("", "0-1", "0,3-4"), (7, 10),
                                                (None, (9,), (0, 25), ())):
        kw = dict(num_steps=ns, dense_steps=ds, dense_layers=dl, calibrate_every=ce, calibrate_steps=cs)
        out["build_schedule"].append({"kwargs": _jsonable(kw), "result": _call(tsd.build_schedule, kw)})
    for kw in (dict(num_steps=0, dense_steps=0, dense_layers="", calibrate_every=10),
               dict(num_steps=10, dense_steps=-1, dense_layers="", calibrate_every=10),
               dict(num_steps=10, dense_steps=0, dense_layers="", calibrate_every=0),
               dict(num_steps=10, dense_steps=0, dense_layers="1-", calibrate_every=5),
               dict(num_steps=10, dense_steps=0, dense_layers="a", calibrate_every=5)):
        out["build_schedule"].append({"kwargs": _jsonable(kw), "result": _call(tsd.build_schedule, kw)})
    for ns, cs, us, as_ in itertools.product((10, 50), ((0,), (9, 25), (60,), (-1,)), (None, (5,), (9,), (70,)), (None, (7,), (25,), (5,))):
        kw = dict(num_steps=ns, calibrate_steps=list(cs), update_steps=us, approx_steps=as_)
        out["validate_schedule"].append({"kwargs": _jsonable(kw), "result": _call(tsd.validate_schedule, kw)})
    for st, sl, tk in itertools.product((0, 64, 300, 1000), (4096, 32760, 98280, 301), (0.05, 0.0625, 0.15, 0.25, 1.0)):
        kw = dict(sink_tokens=st, seq_len=sl, topk=tk)
        out["effective_density"].append({"kwargs": kw, "result": _call(tsd.effective_density, kw)})
    for ch in ELIGIBILITY_CHANGES:
        kw = dict(ELIGIBLE, **ch)
        r = _call(tsd.check_eligibility, kw)
        if "ok" in r:                                          # (ok, reason, severity): the wording is not part of the contract
            r = {"ok": [r["ok"][0], r["ok"][2]]}
        out["check_eligibility"].append({"kwargs": kw, "result": r})
    for cfg in (dict(calibrate_steps=[0, 5], full_steps=[0, 2], update_steps=[3]), dict(calibrate_steps=[0], approx_steps=[2]),
                dict(calibrate_steps=[9, 25], full_steps=list(range(10))), dict(calibrate_steps=[1], update_steps=[1], approx_steps=[1]),
                dict()):
        for has_cache in (False, True):
            c = TokenSparseCache(TokenSparseConfig(topk=0.1, **cfg))
            modes = []
            for step in range(12):
                c._step_count = step
                if has_cache:
                    c._cached_indices = object()
                modes.append(c.mode)
            out["modes"].append({"config": cfg, "has_cache": has_cache, "modes": modes})
    path = Path(__file__).with_name("dispatch_logic.json")
    path.write_text(json.dumps(out, sort_keys=True, separators=(",", ":")) + "\n")
    print(f"wrote {path}: " + ", ".join(f"{k} {len(v)}" for k, v in out.items()))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
