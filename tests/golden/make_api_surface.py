"""Writes ``api_surface.json``: the signatures of the reference's callables that this package keeps (names, order,
kinds and defaults of their parameters; the fields of ``TokenSparseConfig``), read from the reference's source text
with ``ast`` (nothing of it is imported or run).  Usage: ``python tests/golden/make_api_surface.py <reference root>``.
``tests/test_api_surface.py`` compares this package's callables with the file."""

from __future__ import annotations

import ast
import json
import sys
from pathlib import Path

# reference file -> names kept by this package (functions, or Class.method)
KEPT = {
    "mcsparse/kernels/flash_mcsa/ops/flash_sparse_attn/cute/interface.py": [
        "flash_attn_gather_kv_func", "flash_attn_gather_kv_fp8_func", "flash_attn_func"],
    "mcsparse/kernels/flash_mcsa/token_sparse.py": [
        "_compute_token_probs", "_select_topk_tokens", "_compute_adaptive_topk_token", "_chunked_online_topk"],
    "mcsparse/kernels/flash_mcsa/pca_group.py": [
        "pca_group_perm", "apply_perm", "invert_perm", "apply_perm_bhld", "invert_perm_bhld", "identity_perm", "leaf_inertia"],
    "mcsparse/kernels/flash_mcsa/ops/full_attn.py": ["full_attention", "full_attention_with_lse"],
    "mcsparse/h3/token_sparse_dispatch.py": [
        "make_mcsa_token_dispatch", "mcsa_token_begin_forward", "get_mcsa_token_stats", "reset_mcsa_token_state",
        "build_schedule", "validate_schedule", "effective_density", "check_eligibility"],
    "mcsparse/h3/context_parallel.py": ["with_ulysses_sparse", "get_cp_stats", "reset_cp_stats"],
}
DATACLASSES = {"mcsparse/kernels/flash_mcsa/token_sparse.py": ["TokenSparseConfig"]}


def _src(node) -> str | None:
    return None if node is None else ast.unparse(node)


def signature(fn: ast.FunctionDef) -> list[dict]:
    a = fn.args
    out = []
    pos = list(a.posonlyargs) + list(a.args)
    defaults = [None] * (len(pos) - len(a.defaults)) + list(a.defaults)
    for arg, d in zip(pos, defaults):
        out.append({"name": arg.arg, "kind": "positional", "default": _src(d), "required": d is None})
    if a.vararg is not None:
        out.append({"name": a.vararg.arg, "kind": "var_positional", "default": None, "required": False})
    for arg, d in zip(a.kwonlyargs, a.kw_defaults):
        out.append({"name": arg.arg, "kind": "keyword_only", "default": _src(d), "required": d is None})
    if a.kwarg is not None:
        out.append({"name": a.kwarg.arg, "kind": "var_keyword", "default": None, "required": False})
    return out


def main(root: str) -> None:
    rootp = Path(root)
    result = {"functions": {}, "dataclasses": {}}
    for rel, names in KEPT.items():
        tree = ast.parse((rootp / rel).read_text())
        found = {n.name: n for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef))}
        for name in names:
            if name not in found:
                raise SystemExit(f"{rel}: no function {name}")
            result["functions"][f"{rel}::{name}"] = signature(found[name])
    for rel, names in DATACLASSES.items():
        tree = ast.parse((rootp / rel).read_text())
        for node in ast.walk(tree):
            if isinstance(node, ast.ClassDef) and node.name in names:
                fields = []
                for st in node.body:
                    if isinstance(st, ast.AnnAssign) and isinstance(st.target, ast.Name):
                        fields.append({"name": st.target.id, "default": _src(st.value)})
                result["dataclasses"][f"{rel}::{node.name}"] = fields
    out = Path(__file__).with_name("api_surface.json")
    out.write_text(json.dumps(result, indent=1, sort_keys=True) + "\n")
    print(f"wrote {out} ({len(result['functions'])} functions, {len(result['dataclasses'])} dataclasses)")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
