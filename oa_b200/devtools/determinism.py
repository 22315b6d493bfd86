"""Replay determinism: run a workload several times in fresh processes and compare the traces it prints
(Tools/Diagnostics/oadeterminism.py of the reference: selected output traces across fresh workload processes).

    python -m oa_b200.devtools.determinism --name nlp-transformer --runs 3 --trace 'loss=(?P<value>[-0-9.e]+)' \\
        --output var/report/determinism -- python -m oa_b200.apps.train --config ... --steps 20

The trace is every match of `--trace` in the run's standard output (no capture: the whole match; one capture or a capture
named `value`: that text), in order.  Runs agree when their traces are equal element by element; `--tolerance` makes the
comparison numeric (|a - b| <= tol * max(1, |a|, |b|)) for workloads whose reductions use floating-point atomics.  The
report names the first step at which two runs part.  In-process helpers: `tensor_digest` / `model_digest` hash parameter
bytes (sha256 over dtype, shape and contents in name order), the digest a training script prints to be compared here.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import re
import subprocess
import sys
import time
from pathlib import Path
from typing import Dict, List, Optional, Sequence

SCHEMA = "oa_b200.determinism.v1"
ANSI = re.compile(r"\x1b\[[0-?]*[ -/]*[@-~]")


def extract_trace(pattern: "re.Pattern[str]", text: str) -> List[str]:
    out: List[str] = []
    for m in pattern.finditer(ANSI.sub("", text)):
        if "value" in m.groupdict() and m.group("value") is not None:
            out.append(m.group("value"))
        elif m.lastindex is None:
            out.append(m.group(0))
        elif m.lastindex == 1:
            out.append(m.group(1))
        else:
            raise ValueError("the trace pattern must have no capture, one capture, or a capture named 'value'")
    return out


def first_difference(a: Sequence[str], b: Sequence[str], tolerance: float = 0.0) -> Optional[int]:
    """Index of the first element at which two traces differ (a missing element differs), or None."""
    for i in range(max(len(a), len(b))):
        if i >= len(a) or i >= len(b):
            return i
        if a[i] == b[i]:
            continue
        if tolerance > 0.0:
            try:
                x, y = float(a[i]), float(b[i])
                if abs(x - y) <= tolerance * max(1.0, abs(x), abs(y)):
                    continue
            except ValueError:
                pass
        return i
    return None


def compare(traces: Sequence[Sequence[str]], tolerance: float = 0.0) -> Dict[str, object]:
    """Every run against the first.  {"deterministic": bool, "lengths": [...], "differences": [{run, index, first, other}]}"""
    diffs = []
    for r in range(1, len(traces)):
        i = first_difference(traces[0], traces[r], tolerance)
        if i is not None:
            diffs.append({"run": r, "index": i, "first": traces[0][i] if i < len(traces[0]) else None,
                          "other": traces[r][i] if i < len(traces[r]) else None})
    empty = any(len(t) == 0 for t in traces)
    return {"deterministic": not diffs and not empty, "empty_trace": empty, "lengths": [len(t) for t in traces], "differences": diffs}


def run_workload(command: Sequence[str], runs: int, pattern: "re.Pattern[str]", output: Optional[Path] = None, timeout: float = 3600.0,
                 env: Optional[Dict[str, str]] = None, tolerance: float = 0.0, name: str = "workload") -> Dict[str, object]:
    traces, records = [], []
    for r in range(runs):
        t0 = time.time()
        p = subprocess.run(list(command), capture_output=True, text=True, timeout=timeout, env={**os.environ, **(env or {})})
        trace = extract_trace(pattern, p.stdout)
        traces.append(trace)
        records.append({"run": r, "exit_status": p.returncode, "duration_s": round(time.time() - t0, 3), "trace_length": len(trace),
                        "trace_sha256": hashlib.sha256("\n".join(trace).encode()).hexdigest()})
        if output is not None:
            output.mkdir(parents=True, exist_ok=True)
            (output / f"run{r}.stdout.log").write_text(p.stdout)
            (output / f"run{r}.stderr.log").write_text(p.stderr)
    report = {"schema": SCHEMA, "name": name, "command": list(command), "pattern": pattern.pattern, "tolerance": tolerance, "runs": records}
    report.update(compare(traces, tolerance))
    report["ok"] = bool(report["deterministic"]) and all(x["exit_status"] == 0 for x in records)
    if output is not None:
        (output / "determinism.json").write_text(json.dumps(report, indent=1, sort_keys=True) + "\n")
    return report


# ---- digests a workload can print
def tensor_digest(t) -> str:
    import torch
    c = t.detach().contiguous().cpu()
    h = hashlib.sha256(f"{c.dtype}{tuple(c.shape)}".encode())
    h.update(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")
    return h.hexdigest()


def model_digest(model) -> str:
    """sha256 over every named parameter of an OaModule (names sorted), 16 hex digits."""
    h = hashlib.sha256()
    for n in sorted(model.AllNamedParameterPtrs(), key=lambda q: q.Name):
        h.update(n.Name.encode())
        h.update(tensor_digest(n.Param.Tensor()).encode())
    return h.hexdigest()[:16]


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="compare output traces of a workload across fresh processes")
    ap.add_argument("--name", required=True)
    ap.add_argument("--runs", type=int, default=2)
    ap.add_argument("--trace", required=True, help="regular expression whose matches form the trace")
    ap.add_argument("--tolerance", type=float, default=0.0)
    ap.add_argument("--output", type=Path, default=None)
    ap.add_argument("--timeout", type=float, default=3600.0)
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(list(argv) if argv is not None else None)
    cmd = a.command[1:] if a.command[:1] == ["--"] else a.command
    if not cmd or a.runs < 2:
        ap.error("a command and at least two runs are needed")
    rep = run_workload(cmd, a.runs, re.compile(a.trace), a.output, a.timeout, tolerance=a.tolerance, name=a.name)
    for d in rep["differences"]:
        print(f"DETERMINISM: run {d['run']} parts from run 0 at trace element {d['index']}: {d['first']!r} vs {d['other']!r}")
    if rep["empty_trace"]:
        print("DETERMINISM: a run printed nothing that matches the trace pattern")
    print(f"determinism {a.name}: {'ok' if rep['ok'] else 'FAILED'} ({a.runs} runs, trace lengths {rep['lengths']})")
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
