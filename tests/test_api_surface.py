"""The callables this package keeps from the reference accept the reference's own calls: same parameter names in the
same order, same kinds, same literal defaults, nothing newly required.  The reference's signatures are the committed
``tests/golden/api_surface.json`` (``tests/golden/make_api_surface.py`` reads them from the reference's source text).
Deliberate differences are listed in ``DIFFERENT`` with the reason."""

import ast
import importlib
import inspect
import json
from pathlib import Path

import pytest

SURFACE = json.loads((Path(__file__).parent / "golden" / "api_surface.json").read_text())

MODULES = {
    "mcsparse/kernels/flash_mcsa/ops/flash_sparse_attn/cute/interface.py": "mcsparse_b200.kernels.flash_mcsa.ops.flash_sparse_attn.cute.interface",
    "mcsparse/kernels/flash_mcsa/token_sparse.py": "mcsparse_b200.kernels.flash_mcsa.token_sparse",
    "mcsparse/kernels/flash_mcsa/pca_group.py": "mcsparse_b200.kernels.flash_mcsa.pca_group",
    "mcsparse/kernels/flash_mcsa/ops/full_attn.py": "mcsparse_b200.kernels.flash_mcsa.ops.full_attn",
    "mcsparse/h3/token_sparse_dispatch.py": "mcsparse_b200.h3.token_sparse_dispatch",
    "mcsparse/h3/context_parallel.py": "mcsparse_b200.h3.context_parallel",
}

# (function, parameter) -> why this package's default differs from the reference's
DIFFERENT = {
    ("make_mcsa_token_dispatch", "offload_indices"): "indices stay resident by default on a 180 GB part; offload is opt-in",
    ("make_mcsa_token_dispatch", "cache_offload"): "the residual stays resident by default; offload is opt-in",
    ("make_mcsa_token_dispatch", "full_attn_impl"): "one dense implementation (the kernel's dense mode); the name is accepted and ignored",
}
# TokenSparseConfig fields whose default differs, same reasons
DIFFERENT_FIELDS = {
    "offload_indices": "resident by default", "cache_offload": "resident by default", "full_attn_impl": "single dense implementation",
}


def _literal(src):
    if src is None:
        return False, None
    try:
        return True, ast.literal_eval(src)
    except (ValueError, SyntaxError):
        return False, None          # a module constant: compared by name below


@pytest.mark.parametrize("key", sorted(SURFACE["functions"]))
def test_function_signature_accepts_reference_calls(key):
    rel, name = key.split("::")
    mod = importlib.import_module(MODULES[rel])
    fn = getattr(mod, name)
    ours = inspect.signature(fn).parameters
    ref = SURFACE["functions"][key]
    ref_names = {p["name"] for p in ref}
    our_pos = [n for n, p in ours.items() if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    ref_pos = [p["name"] for p in ref if p["kind"] == "positional"]
    assert our_pos[:len(ref_pos)] == ref_pos, f"{name}: positional parameters {our_pos} do not start with the reference's {ref_pos}"
    has_var_kw = any(p.kind == p.VAR_KEYWORD for p in ours.values())
    for p in ref:
        if p["kind"] in ("var_positional", "var_keyword"):
            continue
        if p["name"] not in ours:
            assert has_var_kw, f"{name}: reference parameter {p['name']} is not accepted"
            continue
        o = ours[p["name"]]
        if p["kind"] == "keyword_only":
            assert o.kind in (o.KEYWORD_ONLY, o.POSITIONAL_OR_KEYWORD), f"{name}.{p['name']} cannot be passed by keyword"
        if not p["required"]:
            assert o.default is not inspect.Parameter.empty, f"{name}.{p['name']} is optional in the reference, required here"
            is_lit, val = _literal(p["default"])
            if is_lit and (name, p["name"]) not in DIFFERENT:
                assert o.default == val, f"{name}.{p['name']}: default {o.default!r}, reference {val!r}"
            elif not is_lit and (name, p["name"]) not in DIFFERENT:
                # default given by a module constant of the same name in both packages
                const = getattr(mod, p["default"], None)
                assert const is not None and o.default == const, f"{name}.{p['name']}: default should be the module constant {p['default']}"
    # nothing beyond the reference's parameters is required
    for n, o in ours.items():
        if n not in ref_names and o.kind not in (o.VAR_POSITIONAL, o.VAR_KEYWORD):
            assert o.default is not inspect.Parameter.empty, f"{name}: extra parameter {n} has no default"


def test_token_sparse_config_fields():
    import dataclasses
    from mcsparse_b200.kernels.flash_mcsa.token_sparse import TokenSparseConfig
    ref = SURFACE["dataclasses"]["mcsparse/kernels/flash_mcsa/token_sparse.py::TokenSparseConfig"]
    ours = {f.name: f for f in dataclasses.fields(TokenSparseConfig)}
    for f in ref:
        assert f["name"] in ours, f"TokenSparseConfig.{f['name']} is missing"
        is_lit, val = _literal(f["default"])
        if is_lit and f["name"] not in DIFFERENT_FIELDS:
            assert ours[f["name"]].default == val, f"TokenSparseConfig.{f['name']}: default {ours[f['name']].default!r}, reference {val!r}"
    # the reference's positional construction order is kept for the fields it has
    ref_order = [f["name"] for f in ref]
    our_order = [n for n in ours if n in set(ref_order)]
    assert our_order == ref_order
