"""Evidence bundles: one checksummed directory with what is needed to reproduce a result
(Tools/Diagnostics/oaevidence.py and run_validation.py of the reference, which snapshot the checkout and the Vulkan device,
wrap a workload, request validation and attach graph / benchmark artifacts under a manifest).

    python -m oa_b200.devtools.evidence --output var/report/snapshot
    python -m oa_b200.devtools.evidence --validation sync --output var/report/flagship -- python bench.py --steps 3 --warmup 3
    python -m oa_b200.devtools.evidence --attach var/report/flagship.json --attach profiles/flagship_step_launch_shares.md

The manifest records: git commit, branch and dirty state; platform, Python, torch and CUDA versions; the devices as
`nvidia-smi --query-gpu` reports them (read only; absent on a CPU box); an allowlist of environment variables
(OA_*, NCCL_*, CUDA_VISIBLE_DEVICES, WORLD_SIZE, RANK, LOCAL_RANK); checksums of the kernel library, of the C header
and of the measured-peaks file; the workload's command, duration, exit status and logs; the validation request and the
errors the layer reported (`--validation MODE` runs the workload with OA_VALIDATION=1 and fails the bundle when the log
holds a validation error); every attached artifact with its SHA-256; and the bench JSON line when the workload printed one.
`verify()` re-checks every checksum of a bundle.
"""
from __future__ import annotations

import argparse
import datetime as dt
import hashlib
import json
import os
import platform
import re
import shutil
import subprocess
import sys
import time
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence

SCHEMA = "oa_b200.evidence.v1"
REPO = Path(__file__).resolve().parents[2]
ENV_ALLOW = re.compile(r"^(OA_|NCCL_|TORCH_NCCL_)|^(CUDA_VISIBLE_DEVICES|WORLD_SIZE|RANK|LOCAL_RANK|MASTER_ADDR|MASTER_PORT)$")
VALIDATION_ERROR = re.compile(r"\[validation:(ERROR|FATAL)\]")
GPU_QUERY = "index,name,memory.total,driver_version,clocks.max.sm,clocks.max.memory,power.limit"


def sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _git(repo: Path, *args: str) -> str:
    try:
        r = subprocess.run(["git", "-C", str(repo), *args], capture_output=True, text=True, timeout=30)
        return r.stdout.strip() if r.returncode == 0 else ""
    except (OSError, subprocess.TimeoutExpired):
        return ""


def git_state(repo: Path = REPO) -> Dict[str, object]:
    status = _git(repo, "status", "--porcelain")
    return {"commit": _git(repo, "rev-parse", "HEAD"), "branch": _git(repo, "rev-parse", "--abbrev-ref", "HEAD"),
            "dirty": bool(status), "dirty_files": len(status.splitlines()) if status else 0}


def devices() -> List[Dict[str, str]]:
    """What the driver reports about the GPUs (a read-only query); [] where there is no nvidia-smi or no device."""
    exe = shutil.which("nvidia-smi")
    if not exe:
        return []
    try:
        r = subprocess.run([exe, f"--query-gpu={GPU_QUERY}", "--format=csv,noheader"], capture_output=True, text=True, timeout=30)
    except (OSError, subprocess.TimeoutExpired):
        return []
    if r.returncode != 0:
        return []
    keys = GPU_QUERY.split(",")
    return [dict(zip(keys, [c.strip() for c in line.split(",")])) for line in r.stdout.splitlines() if line.strip()]


def software() -> Dict[str, str]:
    out = {"python": platform.python_version(), "platform": platform.platform()}
    try:
        import torch
        out["torch"] = torch.__version__
        out["torch_cuda"] = str(torch.version.cuda)
        out["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else ""
    except Exception:          # torch missing or broken: the bundle still says what it can
        pass
    nvcc = shutil.which("nvcc")
    if nvcc:
        r = subprocess.run([nvcc, "--version"], capture_output=True, text=True)
        m = re.search(r"release ([\d.]+), V([\d.]+)", r.stdout)
        out["nvcc"] = m.group(2) if m else ""
    return out


def tracked_files(repo: Path = REPO) -> Dict[str, Optional[str]]:
    files = {"kernel_library": repo / "oa_b200" / "_lib" / "liboa_kernels.so", "runtime_library": repo / "oa_b200" / "_lib" / "liboa_runtime.so",
             "kernel_header": repo / "oa_b200" / "csrc" / "kernels" / "api.h", "measured_peaks": repo / "MEASURED_PEAKS.json"}
    return {k: (sha256_file(p) if p.exists() else None) for k, p in files.items()}


def last_json_line(text: str) -> Optional[dict]:
    for line in reversed(text.splitlines()):
        line = line.strip()
        if line.startswith("{") and line.endswith("}"):
            try:
                return json.loads(line)
            except ValueError:
                continue
    return None


def collect(output: Path, command: Sequence[str] = (), validation: str = "", attach: Iterable[Path] = (), timeout: float = 3600.0,
            repo: Path = REPO) -> Dict[str, object]:
    """Writes the bundle and returns its manifest.  manifest["ok"] is False when the workload failed, timed out, or ran
    under validation and the layer reported an error."""
    output.mkdir(parents=True, exist_ok=True)
    manifest: Dict[str, object] = {"schema": SCHEMA, "created_utc": dt.datetime.now(dt.timezone.utc).isoformat(timespec="seconds"),
                                   "git": git_state(repo), "software": software(), "devices": devices(), "files": tracked_files(repo),
                                   "environment": {k: v for k, v in sorted(os.environ.items()) if ENV_ALLOW.search(k)}}
    ok = True
    if command:
        env = dict(os.environ)
        if validation:
            env.update({"OA_VALIDATION": "1", "OA_VALIDATION_MODE": validation})
        t0 = time.time()
        try:
            r = subprocess.run(list(command), capture_output=True, text=True, timeout=timeout, env=env, cwd=str(repo))
            rc, out, err, timed_out = r.returncode, r.stdout, r.stderr, False
        except subprocess.TimeoutExpired as e:
            rc, out, err, timed_out = -1, (e.stdout or b"").decode(errors="replace") if isinstance(e.stdout, bytes) else (e.stdout or ""), \
                (e.stderr or b"").decode(errors="replace") if isinstance(e.stderr, bytes) else (e.stderr or ""), True
        (output / "stdout.log").write_text(out)
        (output / "stderr.log").write_text(err)
        errors = [line for line in (out + "\n" + err).splitlines() if VALIDATION_ERROR.search(line)]
        manifest["workload"] = {"command": list(command), "exit_status": rc, "timed_out": timed_out, "duration_s": round(time.time() - t0, 3),
                                "result": last_json_line(out)}
        manifest["validation"] = {"requested": validation or None, "errors": len(errors), "first_errors": errors[:10]}
        ok = rc == 0 and not timed_out and not (validation and errors)
    artifacts = []
    for src in attach:
        src = Path(src)
        if not src.exists():
            raise FileNotFoundError(f"artifact to attach does not exist: {src}")
        dst = output / "artifacts" / src.name
        dst.parent.mkdir(exist_ok=True)
        shutil.copyfile(src, dst)
        artifacts.append({"name": src.name, "source": str(src), "bytes": dst.stat().st_size})
    manifest["artifacts"] = artifacts
    manifest["ok"] = ok
    sums = {}
    for p in sorted(output.rglob("*")):
        if p.is_file() and p.name not in ("manifest.json",):
            sums[str(p.relative_to(output))] = sha256_file(p)
    manifest["checksums"] = sums
    (output / "manifest.json").write_text(json.dumps(manifest, indent=1, sort_keys=True) + "\n")
    return manifest


def verify(bundle: Path) -> List[str]:
    """Problems of a bundle: files that are missing or whose checksum changed, files the manifest does not know."""
    manifest = json.loads((bundle / "manifest.json").read_text())
    problems = []
    if manifest.get("schema") != SCHEMA:
        problems.append(f"unknown schema {manifest.get('schema')!r}")
    sums = manifest.get("checksums", {})
    for rel, want in sums.items():
        p = bundle / rel
        if not p.exists():
            problems.append(f"missing: {rel}")
        elif sha256_file(p) != want:
            problems.append(f"checksum differs: {rel}")
    for p in bundle.rglob("*"):
        if p.is_file() and p.name != "manifest.json" and str(p.relative_to(bundle)) not in sums:
            problems.append(f"not in the manifest: {p.relative_to(bundle)}")
    return problems


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="checksummed evidence bundle of a workload")
    ap.add_argument("--output", type=Path, default=Path("var/report/evidence"))
    ap.add_argument("--validation", choices=["core", "sync", "nan"], default="")
    ap.add_argument("--attach", type=Path, action="append", default=[])
    ap.add_argument("--timeout", type=float, default=3600.0)
    ap.add_argument("--verify", type=Path, help="check the checksums of an existing bundle instead of writing one")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(list(argv) if argv is not None else None)
    if a.verify:
        problems = verify(a.verify)
        for p in problems:
            print("EVIDENCE:", p)
        print("evidence bundle:", "FAILED" if problems else "ok")
        return 1 if problems else 0
    cmd = a.command[1:] if a.command[:1] == ["--"] else a.command
    m = collect(a.output, cmd, a.validation, a.attach, a.timeout)
    print(f"evidence: {a.output / 'manifest.json'} ok={m['ok']}")
    return 0 if m["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
