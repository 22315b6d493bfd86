"""GEMM launch-plan tuner: the consumer of the native OaGemmPlanCache (csrc/runtime/plan_cache.cpp).

The reference keeps tuner samples per (M, N, K, layout, epilogue, role, world) and persists the winning launch plan
(Source/Private/Oa/Runtime/GemmPlanCache.cpp); its GEMM dispatch consults the cache before it picks a kernel.  Here the
plan is the N tile of the tcgen05 kernel family (0 = the library's own choice, which includes the 256 x 256 CTA-pair
kernel; 128 or 256 = the single-CTA kernel with that tile).  `Install()` hooks the tuner into `ops.kernels.gemm`:

  * a shape that the cache knows runs with its recorded plan;
  * an unknown shape is timed once, outside stream capture, on the caller's own operands (`reps` launches per candidate,
    CUDA events, median), every sample is recorded, the fastest plan is kept;
  * under stream capture, or with tuning off, an unknown shape runs with the library's choice and nothing is recorded.

OA_GEMM_TUNE=1 installs the tuner when the engine starts; OA_GEMM_PLANS=<file> loads the plans of an earlier run at start
and `Save()` (also at interpreter exit) writes them back, so a tuned job pays the timing runs once.
"""
from __future__ import annotations

import atexit
import os
from typing import Callable, Optional

import torch

from ..ops import kernels as K
from .graph import OaGemmPlanCache

CANDIDATES = (0, 128, 256)


class OaGemmTuner:
    def __init__(self, path: Optional[str] = None, tune: bool = True, reps: int = 5,
                 timer: Optional[Callable[[Callable[[], None], int], float]] = None):
        self.Cache = OaGemmPlanCache()
        self.Path = path
        self.Tune = bool(tune)
        self.Reps = int(reps)
        self.Tuned = 0
        self._timer = timer or self._time_cuda
        if path and os.path.exists(path):
            st = self.Cache.Load(path)
            if not st.IsOk():
                raise RuntimeError(st.message)

    @staticmethod
    def _time_cuda(run: Callable[[], None], reps: int) -> float:
        """Median microseconds of `reps` launches after one warm-up launch."""
        run()
        times = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            run()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        times.sort()
        return times[len(times) // 2]

    def Plan(self, M: int, N: int, Kd: int, layout: int, epilogue: int, run: Callable[[int], None]) -> int:
        """The N tile to launch with (0 = library's choice).  `run(bn)` launches the caller's GEMM with that tile."""
        hit = self.Cache.Lookup(M, N, Kd, layout, epilogue)
        if hit is not None:
            return hit[0]
        if not self.Tune or (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()):
            return 0
        best, best_us = 0, float("inf")
        for bn in CANDIDATES:
            if bn and N < bn:
                continue
            us = self._timer(lambda bn=bn: run(bn), self.Reps)
            self.Cache.Record(M, N, Kd, bn, 1, us, layout, epilogue)
            if us < best_us:
                best, best_us = bn, us
        self.Tuned += 1                   # the cache has re-elected the key's plan by median at every Record
        return best

    def Install(self) -> "OaGemmTuner":
        K.set_gemm_planner(self.Plan)
        if self.Path:
            atexit.register(self.Save)
        return self

    def Uninstall(self) -> None:
        K.set_gemm_planner(None)

    def Save(self) -> None:
        if self.Path and self.Cache.Size():
            self.Cache.Save(self.Path)


_installed: Optional[OaGemmTuner] = None


def InstallFromEnv() -> Optional[OaGemmTuner]:
    """Called when the engine starts: OA_GEMM_TUNE=1 and / or OA_GEMM_PLANS=<file>."""
    global _installed
    tune = os.environ.get("OA_GEMM_TUNE", "0") == "1"
    path = os.environ.get("OA_GEMM_PLANS") or None
    if _installed is None and (tune or path):
        _installed = OaGemmTuner(path, tune=tune).Install()
    return _installed
