"""Builds the native libraries in-tree with nvcc / g++ (sm_100a only).

`python -m oa_b200.build` compiles every `.cu` under `csrc/kernels` into `oa_b200/_lib/liboa_kernels.so`
and the host-side C++ runtime under `csrc/runtime` into `oa_b200/_lib/liboa_runtime.so`.  Objects are
rebuilt only when their source (or a header) is newer.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
KERNEL_DIR = ROOT / "csrc" / "kernels"
RUNTIME_DIR = ROOT / "csrc" / "runtime"
LIB_DIR = ROOT / "_lib"
OBJ_DIR = ROOT / "_lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _newest_header(d: Path) -> float:
    hs = [p.stat().st_mtime for p in list(d.glob("*.cuh")) + list(d.glob("*.h")) + list(d.glob("*.hpp"))]
    return max(hs) if hs else 0.0


def _compile_one(cmd: list[str], log: Path) -> tuple[int, str]:
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(r.stdout + r.stderr)
    return r.returncode, r.stdout + r.stderr


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    out = LIB_DIR / "liboa_kernels.so"
    hdr = _newest_header(KERNEL_DIR)
    srcs = sorted(KERNEL_DIR.glob("*.cu"))
    jobs = []
    objs = []
    for src in srcs:
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr):
            jobs.append(([_nvcc(), *NVCC_FLAGS, *os.environ.get("OA_NVCC_EXTRA", "").split(), "-I", str(KERNEL_DIR), "-c", str(src), "-o", str(obj)],
                         OBJ_DIR / (src.stem + ".log")))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            results = list(ex.map(lambda j: _compile_one(*j), jobs))
        for (cmd, _), (rc, text) in zip(jobs, results):
            if verbose or rc != 0:
                sys.stderr.write(text)
            if rc != 0:
                raise RuntimeError(f"nvcc failed: {' '.join(cmd)}")
    if jobs or not out.exists():
        # link beside the target and rename: a reader (or a copy of the tree) never sees a half-written library
        tmp = out.with_suffix(".so.tmp")
        cmd = [_nvcc(), "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of liboa_kernels.so failed")
        os.replace(tmp, out)
    return out


def build_runtime(force: bool = False) -> Path | None:
    srcs = sorted(RUNTIME_DIR.glob("*.cpp"))
    if not srcs:
        return None
    LIB_DIR.mkdir(exist_ok=True)
    out = LIB_DIR / "liboa_runtime.so"
    newest = max([s.stat().st_mtime for s in srcs] + [_newest_header(RUNTIME_DIR)])
    if force or not out.exists() or out.stat().st_mtime < newest:
        tmp = out.with_suffix(".so.tmp")
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-I", str(RUNTIME_DIR), "-o", str(tmp),
               *map(str, srcs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("build of liboa_runtime.so failed")
        os.replace(tmp, out)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_runtime(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", *[p.name for p in LIB_DIR.glob("*.so")])
