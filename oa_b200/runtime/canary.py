"""OaDeviceCanary: a deterministic known-answer admission test of a GPU before a run
(Source/Public/Oa/Runtime/Canary.h:14-47, Source/Private/Oa/Runtime/Canary.cpp; exit codes 0 pass, 2 wrong answer,
3 device or runtime error).  Every probe has an exact expected result (small-integer operands make the bf16 tensor-core
GEMM exact), so a mismatch is a hardware or driver fault, not noise.  `python -m oa_b200.runtime.canary [--device N] [--json PATH]`.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from dataclasses import asdict, dataclass, field

import torch

EXIT_OK, EXIT_MISMATCH, EXIT_ERROR = 0, 2, 3


@dataclass
class OaCanaryProbe:
    Name: str
    Passed: bool
    Detail: str = ""
    Ms: float = 0.0


@dataclass
class OaCanaryReport:
    Device: int = 0
    DeviceName: str = ""
    Passed: bool = False
    ExitCode: int = EXIT_ERROR
    Probes: list = field(default_factory=list)
    Error: str = ""

    def ToJson(self) -> str:
        return json.dumps(asdict(self), indent=1)


def _probes(dev):
    from ..ops import kernels as K
    g = torch.Generator().manual_seed(7)

    def gemm():
        a = torch.randint(-3, 4, (256, 192), generator=g).to(torch.bfloat16).to(dev)
        b = torch.randint(-3, 4, (128, 192), generator=g).to(torch.bfloat16).to(dev)
        want = (a.float().cpu() @ b.float().cpu().t())
        got = K.gemm(a, b, out_dtype=torch.float32)
        return torch.equal(got.cpu(), want), f"max |diff| {(got.cpu() - want).abs().max().item()}"

    def elementwise():
        x = torch.arange(-512, 512, dtype=torch.float32, device=dev)
        y = K.binary("add", K.unary("scale", x, 2.0), x)
        return torch.equal(y.cpu(), (3 * torch.arange(-512, 512)).float()), ""

    def reduction():
        x = torch.ones(1024, 333, dtype=torch.float32, device=dev)
        s = K.col_sum(x)
        return torch.equal(s.cpu(), torch.full((333,), 1024.0)), ""

    def memory():
        n = 64 << 20
        x = torch.empty(n, dtype=torch.uint8, device=dev)
        pat = torch.arange(256, dtype=torch.uint8, device=dev).repeat(n // 256)
        x.copy_(pat)
        ok = bool((x.view(torch.int64) == pat.view(torch.int64)).all().item())
        return ok, f"{n >> 20} MiB pattern"

    def softmax():
        x = torch.zeros(64, 1000, dtype=torch.float32, device=dev)
        y = K.softmax(x)
        return bool(((y - 1e-3).abs() < 1e-9).all().item()), ""

    return [("gemm_bf16_exact", gemm), ("elementwise_exact", elementwise), ("column_sum_exact", reduction), ("memory_pattern", memory),
            ("softmax_uniform", softmax)]


def OaRunDeviceCanary(device: int = 0) -> OaCanaryReport:
    rep = OaCanaryReport(Device=device)
    try:
        if not torch.cuda.is_available() or device >= torch.cuda.device_count():
            raise RuntimeError(f"CUDA device {device} is not present")
        dev = torch.device("cuda", device)
        torch.cuda.set_device(dev)
        rep.DeviceName = torch.cuda.get_device_name(dev)
        from ..ops import kernels as K
        for name, fn in _probes(dev):
            t0 = time.perf_counter()
            ok, detail = fn()
            torch.cuda.synchronize(dev)
            K.check_status(dev)
            rep.Probes.append(OaCanaryProbe(name, bool(ok), detail, (time.perf_counter() - t0) * 1e3))
        rep.Passed = all(p.Passed for p in rep.Probes)
        rep.ExitCode = EXIT_OK if rep.Passed else EXIT_MISMATCH
    except Exception as e:          # noqa: BLE001 - any runtime failure is the "device error" verdict
        rep.Error, rep.ExitCode = f"{type(e).__name__}: {e}", EXIT_ERROR
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="GPU admission canary")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    rep = OaRunDeviceCanary(a.device)
    if a.json:
        with open(a.json, "w") as f:
            f.write(rep.ToJson())
    print(rep.ToJson())
    return rep.ExitCode


if __name__ == "__main__":
    sys.exit(main())
