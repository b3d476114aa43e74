#!/usr/bin/env python
"""Writes ``codebase-map.json``: every source file of the package with its classes (first docstring line, public
methods) and functions, the native kernels (exported C entry points per ``.cu`` file), the scripts with the tests that
exercise them, the tests (test counts per file, GPU-marked or not), fixtures and registry entries.

    python scripts/build_codebase_map.py            # rewrite codebase-map.json at the repository root
    python scripts/build_codebase_map.py --check    # exit 1 when the file on disk is out of date

The map is derived from the source with ``ast`` (nothing is imported), so it cannot drift from the code the way a
hand-kept index does; ``tests/test_runtime_units.py`` runs the ``--check`` form.
"""

from __future__ import annotations

import argparse
import ast
import json
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = "kempnerforge_b200"


def first_line(doc: str | None) -> str:
    if not doc:
        return ""
    return " ".join(doc.strip().split("\n\n")[0].split())[:240]


def signature(fn: ast.FunctionDef | ast.AsyncFunctionDef) -> str:
    args = [a.arg for a in fn.args.posonlyargs + fn.args.args if a.arg not in ("self", "cls")]
    if fn.args.vararg:
        args.append("*" + fn.args.vararg.arg)
    args += [a.arg for a in fn.args.kwonlyargs]
    if fn.args.kwarg:
        args.append("**" + fn.args.kwarg.arg)
    return f"{fn.name}({', '.join(args)})"


def describe_python(path: Path) -> dict:
    tree = ast.parse(path.read_text())
    entry: dict = {"purpose": first_line(ast.get_docstring(tree))}
    classes, functions = {}, []
    for node in tree.body:
        if isinstance(node, ast.ClassDef):
            methods = [signature(n) for n in node.body
                       if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)) and not n.name.startswith("_")]
            classes[node.name] = {"purpose": first_line(ast.get_docstring(node)), "methods": methods}
        elif isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)) and not node.name.startswith("_"):
            functions.append(signature(node))
    if classes:
        entry["classes"] = classes
    if functions:
        entry["functions"] = functions
    return entry


def registry_entries() -> dict[str, list[str]]:
    out: dict[str, set[str]] = {}
    pat = re.compile(r"registry\.register\(\s*[\"'](\w+)[\"']\s*,\s*[\"']([\w\-]+)[\"']")
    for path in sorted((ROOT / PKG).rglob("*.py")):
        for cat, name in pat.findall(path.read_text()):
            out.setdefault(cat, set()).add(name)
    return {k: sorted(v) for k, v in sorted(out.items())}


def kernels() -> dict:
    out = {}
    sym = re.compile(r"^(?:extern \"C\" )?(?:int|void|void\*)\s+(kf_\w+)\s*\(", re.M)
    for path in sorted((ROOT / "csrc").glob("*.cu")):
        text = path.read_text()
        head = []
        for line in text.splitlines():
            if not line.startswith("//"):
                break
            head.append(line[2:].strip())
        out[f"csrc/{path.name}"] = {"purpose": " ".join(head)[:300], "entry_points": sorted(set(sym.findall(text)))}
    return out


def tests() -> tuple[dict, dict]:
    files, fixtures = {}, {}
    for path in sorted((ROOT / "tests").glob("*.py")):
        text = path.read_text()
        tree = ast.parse(text)
        names = [n.name for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)) and n.name.startswith("test_")]
        fx = []
        for n in ast.walk(tree):
            if isinstance(n, ast.FunctionDef):
                for d in n.decorator_list:
                    src = ast.unparse(d)
                    if src.startswith("pytest.fixture"):
                        fx.append(n.name)
        if fx:
            fixtures[f"tests/{path.name}"] = sorted(fx)
        if names:
            files[f"tests/{path.name}"] = {"purpose": first_line(ast.get_docstring(tree)), "tests": len(names),
                                            "gpu": "pytest.mark.gpu" in text}
    return files, fixtures


def scripts(test_files: dict) -> dict:
    out = {}
    for path in sorted((ROOT / "scripts").glob("*.py")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]:
        rel = str(path.relative_to(ROOT))
        stem = path.stem
        used_by = sorted(t for t in test_files if stem in (ROOT / t).read_text())
        out[rel] = {"purpose": first_line(ast.get_docstring(ast.parse(path.read_text()))), "tested_by": used_by}
    return out


def build() -> dict:
    source = {str(p.relative_to(ROOT)): describe_python(p) for p in sorted((ROOT / PKG).rglob("*.py"))
              if p.name != "__init__.py" or p.stat().st_size > 200}
    test_files, fixtures = tests()
    return {
        "meta": {"description": f"{PKG} codebase map: files, classes, functions, kernels, tests and registry entries",
                 "generated_by": "scripts/build_codebase_map.py (derived from the source; do not edit by hand)"},
        "source": source,
        "kernels": kernels(),
        "scripts": scripts(test_files),
        "benchmarks": {str(p.relative_to(ROOT)): first_line(ast.get_docstring(ast.parse(p.read_text())))
                       for p in sorted((ROOT / "benchmarks").glob("*.py")) if p.name != "__init__.py"},
        "tests": test_files,
        "fixtures": fixtures,
        "registry_entries": registry_entries(),
    }


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args()
    text = json.dumps(build(), indent=1, sort_keys=False) + "\n"
    target = ROOT / "codebase-map.json"
    if args.check:
        if not target.exists() or target.read_text() != text:
            print("codebase-map.json is out of date: run python scripts/build_codebase_map.py", file=sys.stderr)
            return 1
        return 0
    target.write_text(text)
    print(f"wrote {target} ({len(text) // 1024} KB)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
