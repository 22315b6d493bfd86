"""Reader of the kernel library's C header: entry points with the section they stand under, and enum constants.
Standard library only; used by the operation registry and by the table generator."""
from __future__ import annotations

import re
from typing import Dict, List, Tuple


def _const_expr(text: str) -> int:
    """Value of an integer constant expression of a C enum (literals, + - * << >> | & and parentheses)."""
    import ast
    import operator as op
    ops = {ast.Add: op.add, ast.Sub: op.sub, ast.Mult: op.mul, ast.LShift: op.lshift, ast.RShift: op.rshift, ast.BitOr: op.or_,
           ast.BitAnd: op.and_}

    def ev(n):
        if isinstance(n, ast.Constant) and isinstance(n.value, int):
            return n.value
        if isinstance(n, ast.BinOp) and type(n.op) in ops:
            return ops[type(n.op)](ev(n.left), ev(n.right))
        if isinstance(n, ast.UnaryOp) and isinstance(n.op, ast.USub):
            return -ev(n.operand)
        raise ValueError(f"unsupported constant expression: {text!r}")

    return ev(ast.parse(re.sub(r"(?<=[0-9a-fA-F])[uUlL]+\b", "", text), mode="eval").body)


def fnv1a32(s: str) -> int:
    h = 0x811C9DC5
    for b in s.encode():
        h = ((h ^ b) * 0x01000193) & 0xFFFFFFFF
    return h


def parse_api(text: str) -> Tuple[List[dict], Dict[str, int]]:
    """Entry points (in header order, with the section comment they stand under) and enum constants of api.h."""
    consts: Dict[str, int] = {}
    for body in re.findall(r"enum\s*\{(.*?)\}\s*;", text, flags=re.S):
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        body = re.sub(r"//.*", "", body)
        val = -1
        for item in body.split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, v = item.split("=")
                val = _const_expr(v.strip())
                consts[name.strip()] = val
            else:
                val += 1
                consts[item] = val
    rows: List[dict] = []
    section, provider = "core", "api.h"
    # walk the header so that every prototype keeps the section it stands under
    pos = 0
    # a section comment is `// ---- name (file.cu) ...` or `// ---- file.cu: name`
    pattern = re.compile(r"//[ \t]*-+[ \t]*([^\n(]+?)[ \t]*\(([\w.]+\.cu)[^)\n]*\)|//[ \t]*-+[ \t]*()([\w.]+\.cu):[^\n]*"
                         r"|\b(int|size_t|void)\s+(oa_\w+)\s*\(([^)]*)\)\s*;", flags=re.S)
    clean = re.sub(r"/\*.*?\*/", lambda m: " " * len(m.group(0)), text, flags=re.S)
    for m in pattern.finditer(clean, pos):
        if m.group(2):
            section, provider = m.group(1).strip(), m.group(2)
            continue
        if m.group(4):
            section, provider = m.group(4)[:-3], m.group(4)
            continue
        line_start = clean.rfind("\n", 0, m.start(5)) + 1
        if "//" in clean[line_start:m.start(5)]:
            continue                                   # a prototype quoted inside a comment
        args = []
        for a in re.sub(r"//.*", "", m.group(7)).split(","):
            a = " ".join(a.split())
            if not a or a == "void":
                continue
            args.append("ptr" if "*" in a else " ".join(a.replace("const ", "").split(" ")[:-1]))
        rows.append({"name": m.group(6), "section": section, "file": provider, "id": fnv1a32(m.group(6)), "returns": m.group(5), "args": args})
    return rows, consts
