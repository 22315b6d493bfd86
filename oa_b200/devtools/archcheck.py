"""Architecture gate: the dependency direction between the packages of `oa_b200` is a checked contract
(Tools/Architecture/oacheck.py and its modules.json / dependency_baseline.json in the reference).

`modules.json` names, for every top-level package, the packages it may import.  `dependency_baseline.json` holds the
accepted count of each edge that is outside the policy today; a count may fall, never rise, and an edge that is neither
allowed nor in the baseline fails the check.  Imports are read from the syntax tree (no module is executed); an import
inside a function counts like one at module level, because it is the same dependency.

    python -m oa_b200.devtools.archcheck              check, exit 1 on a violation
    python -m oa_b200.devtools.archcheck --edges      print the edge table (module -> module: imports)
    python -m oa_b200.devtools.archcheck --write-baseline   rewrite the baseline from the tree (for the commit that REMOVES edges)
"""
from __future__ import annotations

import argparse
import ast
import json
import sys
from collections import Counter
from pathlib import Path
from typing import Dict, Iterable, List, Tuple

HERE = Path(__file__).resolve().parent
PACKAGE = HERE.parent                      # .../oa_b200
POLICY = HERE / "modules.json"
BASELINE = HERE / "dependency_baseline.json"


def module_of(path: Path, root: Path = PACKAGE) -> str:
    """Top-level package of a file under the root; files directly in the root form the module "_root"."""
    rel = path.resolve().relative_to(root.resolve())
    return rel.parts[0] if len(rel.parts) > 1 else "_root"


def _resolve(node: ast.ImportFrom, file: Path, root: Path) -> str:
    """Absolute dotted name (below the root package) that a relative or absolute `from x import y` refers to, or ""."""
    pkg = root.name
    if node.level == 0:
        name = node.module or ""
        if name == pkg:
            return "."
        return name[len(pkg) + 1:] if name.startswith(pkg + ".") else ""
    parts = list(file.resolve().relative_to(root.resolve()).parts[:-1])
    up = node.level - 1
    if up > len(parts):
        return ""
    base = parts[:len(parts) - up]
    if node.module:
        base += node.module.split(".")
    return ".".join(base) if base else "."


def imports_of(file: Path, root: Path = PACKAGE) -> List[Tuple[str, int]]:
    """(target top-level module, line) for every import of a sibling package made by `file`."""
    tree = ast.parse(file.read_text(), filename=str(file))
    pkg = root.name
    out: List[Tuple[str, int]] = []
    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            for a in node.names:
                if a.name.startswith(pkg + "."):
                    out.append((a.name.split(".")[1], node.lineno))
        elif isinstance(node, ast.ImportFrom):
            target = _resolve(node, file, root)
            if not target:
                continue
            if target == ".":                          # `from .. import x, y`: each name is a module of the root
                for a in node.names:
                    out.append((a.name, node.lineno))
            else:
                out.append((target.split(".")[0], node.lineno))
    known = {p.name for p in root.iterdir() if p.is_dir() and (p / "__init__.py").exists()}
    res = []
    for t, line in out:
        res.append((t if t in known else "_root", line))
    return res


def edges(root: Path = PACKAGE) -> Dict[Tuple[str, str], List[str]]:
    table: Dict[Tuple[str, str], List[str]] = {}
    for file in sorted(root.rglob("*.py")):
        if "__pycache__" in file.parts:
            continue
        src = module_of(file, root)
        for dst, line in imports_of(file, root):
            if dst != src:
                table.setdefault((src, dst), []).append(f"{file.relative_to(root)}:{line}")
    return table


def check(root: Path = PACKAGE, policy_path: Path = POLICY, baseline_path: Path = BASELINE) -> List[str]:
    """Messages of every violation (empty list: the tree agrees with the policy)."""
    policy = json.loads(policy_path.read_text())
    baseline = json.loads(baseline_path.read_text()).get("edges", {}) if baseline_path.exists() else {}
    mods = policy["modules"]
    problems: List[str] = []
    found = edges(root)
    present = {m for e in found for m in e} | {p.name for p in root.iterdir() if p.is_dir() and (p / "__init__.py").exists()}
    for m in sorted(present):
        if m not in mods:
            problems.append(f"package '{m}' has no entry in {policy_path.name}")
    for m, spec in mods.items():
        for a in spec.get("allows", []):
            if a not in mods:
                problems.append(f"{policy_path.name}: '{m}' allows unknown module '{a}'")
    seen = Counter()
    for (src, dst), sites in sorted(found.items()):
        if src not in mods or dst in mods.get(src, {}).get("allows", []):
            continue
        key = f"{src}->{dst}"
        seen[key] = len(sites)
        accepted = int(baseline.get(key, 0))
        if len(sites) > accepted:
            what = "new forbidden dependency" if accepted == 0 else f"{len(sites)} imports, the baseline accepts {accepted}"
            problems.append(f"{key}: {what}: " + ", ".join(sites[:6]) + (" ..." if len(sites) > 6 else ""))
    for key, accepted in sorted(baseline.items()):
        if seen.get(key, 0) < int(accepted):
            problems.append(f"{key}: the tree has {seen.get(key, 0)} imports, the baseline still says {accepted}: lower or delete the entry")
    return problems


def write_baseline(root: Path = PACKAGE, policy_path: Path = POLICY, baseline_path: Path = BASELINE) -> Dict[str, int]:
    mods = json.loads(policy_path.read_text())["modules"]
    out = {}
    for (src, dst), sites in sorted(edges(root).items()):
        if src in mods and dst not in mods[src].get("allows", []):
            out[f"{src}->{dst}"] = len(sites)
    baseline_path.write_text(json.dumps({"version": 1, "edges": out}, indent=1, sort_keys=True) + "\n")
    return out


def main(argv: Iterable[str] = None) -> int:
    ap = argparse.ArgumentParser(description="dependency-direction gate of the oa_b200 packages")
    ap.add_argument("--edges", action="store_true")
    ap.add_argument("--write-baseline", action="store_true")
    a = ap.parse_args(list(argv) if argv is not None else None)
    if a.edges:
        for (src, dst), sites in sorted(edges().items()):
            print(f"{src} -> {dst}: {len(sites)}")
        return 0
    if a.write_baseline:
        for k, v in write_baseline().items():
            print(f"{k}: {v}")
        return 0
    problems = check()
    for p in problems:
        print("ARCH:", p)
    print("architecture check:", "FAILED" if problems else "ok")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
