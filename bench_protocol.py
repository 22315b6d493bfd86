"""Benchmark protocol: run a benchmark command in fresh processes, summarise with median and MAD, and compare against
an accepted baseline, refusing to compare runs that are not comparable.

    python bench_protocol.py run --runs 7 --out result.json -- python bench.py --steps 5 --warmup 3
    python bench_protocol.py compare --baseline accepted.json --candidate result.json [--tolerance 0.03]
    python bench_protocol.py accept --candidate result.json --baseline accepted.json

Protocol of the reference's Tools/Diagnostics/oabench.py (fresh process per run, at least 7 runs, median / median
absolute deviation, fail-closed comparability: metric, unit, configuration, GPU count and data type must all match or
the comparison is refused with exit code 3, a regression beyond the tolerance exits 2).  Every run must print one JSON
line holding "metric" and "value"; the last such line of a run is taken.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import time
from typing import List, Optional

SCHEMA = "oa_b200.benchmark_result.v1"
MIN_RUNS = 7
COMPARABLE_KEYS = ("metric", "unit", "n_gpus", "dtype", "config", "higher_is_better")


def ParseRun(stdout: str) -> Optional[dict]:
    """The last line of `stdout` that is a JSON object with "metric" and "value"."""
    for line in reversed(stdout.splitlines()):
        line = line.strip()
        if not line.startswith("{"):
            continue
        try:
            obj = json.loads(line)
        except json.JSONDecodeError:
            continue
        if isinstance(obj, dict) and "metric" in obj and "value" in obj:
            return obj
    return None


def Mad(values: List[float]) -> float:
    med = statistics.median(values)
    return statistics.median(abs(v - med) for v in values)


def Summarise(runs: List[dict], command: List[str]) -> dict:
    first = runs[0]
    for r in runs[1:]:
        for k in COMPARABLE_KEYS:
            if r.get(k) != first.get(k):
                raise ValueError(f"runs disagree on '{k}': {first.get(k)!r} vs {r.get(k)!r}")
    values = [float(r["value"]) for r in runs]
    med = statistics.median(values)
    out = {"schema": SCHEMA, "command": command, "runs": len(runs), "values": values, "median": med, "mad": Mad(values),
           "min": min(values), "max": max(values), "relative_mad": (Mad(values) / med) if med else 0.0, "created": time.time()}
    for k in COMPARABLE_KEYS:
        out[k] = first.get(k)
    return out


def Run(command: List[str], runs: int, timeout: Optional[float] = None, log=print) -> dict:
    if runs < MIN_RUNS:
        raise ValueError(f"the protocol needs at least {MIN_RUNS} runs")
    results = []
    for i in range(runs):
        p = subprocess.run(command, capture_output=True, text=True, timeout=timeout)       # a fresh process every time
        if p.returncode != 0:
            raise RuntimeError(f"run {i + 1} exited with {p.returncode}: {p.stderr.strip()[-400:]}")
        r = ParseRun(p.stdout)
        if r is None:
            raise RuntimeError(f"run {i + 1} printed no result line")
        log(f"  run {i + 1}/{runs}: {r['value']:.6g} {r.get('unit', '')}")
        results.append(r)
    return Summarise(results, command)


def Compare(baseline: dict, candidate: dict, tolerance: float = 0.03) -> dict:
    """{"comparable", "reasons", "ratio", "verdict"}: verdict is improved / unchanged / regressed / not-comparable."""
    reasons = [f"{k}: {baseline.get(k)!r} vs {candidate.get(k)!r}" for k in COMPARABLE_KEYS if baseline.get(k) != candidate.get(k)]
    for side, r in (("baseline", baseline), ("candidate", candidate)):
        if r.get("schema") != SCHEMA:
            reasons.append(f"{side} is not a {SCHEMA} record")
        elif r.get("runs", 0) < MIN_RUNS:
            reasons.append(f"{side} has fewer than {MIN_RUNS} runs")
    if reasons:
        return {"comparable": False, "reasons": reasons, "ratio": None, "verdict": "not-comparable"}
    ratio = candidate["median"] / baseline["median"] if baseline["median"] else float("inf")
    gain = ratio - 1.0 if baseline.get("higher_is_better", True) else 1.0 - ratio
    noise = max(tolerance, 3.0 * max(baseline.get("relative_mad", 0.0), candidate.get("relative_mad", 0.0)))
    verdict = "improved" if gain > noise else "regressed" if gain < -noise else "unchanged"
    return {"comparable": True, "reasons": [], "ratio": ratio, "verdict": verdict, "noise_band": noise}


def main(argv=None, out=print) -> int:
    ap = argparse.ArgumentParser(prog="bench_protocol")
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run")
    r.add_argument("--runs", type=int, default=MIN_RUNS); r.add_argument("--out", required=True); r.add_argument("--timeout", type=float, default=None)
    r.add_argument("command", nargs=argparse.REMAINDER)
    c = sub.add_parser("compare")
    c.add_argument("--baseline", required=True); c.add_argument("--candidate", required=True); c.add_argument("--tolerance", type=float, default=0.03)
    a = sub.add_parser("accept")
    a.add_argument("--baseline", required=True); a.add_argument("--candidate", required=True)
    args = ap.parse_args(argv)
    if args.cmd == "run":
        cmd = [x for x in args.command if x != "--"] if args.command[:1] == ["--"] else args.command
        if not cmd:
            out("Error: no command after --")
            return 1
        try:
            res = Run(cmd, args.runs, args.timeout, out)
        except (ValueError, RuntimeError, subprocess.TimeoutExpired) as e:
            out(f"Error: {e}")
            return 1
        with open(args.out, "w") as f:
            json.dump(res, f, indent=1)
        out(f"  median {res['median']:.6g} {res.get('unit') or ''} (MAD {res['mad']:.3g}, {100 * res['relative_mad']:.2f} %) over {res['runs']} runs -> {args.out}")
        return 0
    with open(args.candidate) as f:
        cand = json.load(f)
    if args.cmd == "accept":
        if cand.get("schema") != SCHEMA or cand.get("runs", 0) < MIN_RUNS:
            out(f"Error: only a {SCHEMA} record of at least {MIN_RUNS} runs can become a baseline")
            return 1
        with open(args.baseline, "w") as f:
            json.dump(cand, f, indent=1)
        out(f"  accepted {args.candidate} as {args.baseline}")
        return 0
    with open(args.baseline) as f:
        base = json.load(f)
    res = Compare(base, cand, args.tolerance)
    if not res["comparable"]:
        out("  not comparable: " + "; ".join(res["reasons"]))
        return 3
    out(f"  {res['verdict']}: candidate / baseline = {res['ratio']:.4f} (noise band {100 * res['noise_band']:.2f} %)")
    return 2 if res["verdict"] == "regressed" else 0


if __name__ == "__main__":
    sys.exit(main())
