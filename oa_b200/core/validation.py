"""OaValidation: the debug layer of the framework (Source/Public/Oa/Core/Validation.h:1-190 of the reference).

The reference compiles `OA_VALIDATE(cond, severity, component, fmt, ...)` into debug builds and gates it at run time in
release builds; a failed Error / Fatal check returns an error status from the function that made it.  Here the layer is
always present and off by default (one boolean test per check when off):

    OA_VALIDATION=1                 enable (also `OaValidation.Enable()`)
    OA_VALIDATION_SEVERITY=warning  lowest severity that is reported (verbose | info | warning | error | fatal)
    OA_VALIDATION_MODE=core         what the kernel wrappers check when the layer is on:
        core   arguments of every launch: device, dtype, contiguity, 16-byte alignment of pointers, extents
        sync   core + a stream synchronisation and a read of the kernel status word after EVERY launch, so that a bounded
               wait that ran out, or a CUDA error, is reported against the launch that caused it and not a later one
        nan    sync + a finite check of the floating-point outputs that the wrappers declare

Counters (`IncrCounter`) count launches per entry point and reports per severity while the layer is on; `DumpCounters`
logs the non-zero ones.  The device-side checks (index bounds in the gather / scatter / routing kernels, bounded waits)
are always compiled in and report through the status word, which `sync` mode reads after every launch.
"""
from __future__ import annotations

import enum
import os
import threading
from typing import Callable, Dict, Optional

from .types import OaError, OaStatus, OaStatusCode


class OaValidationSeverity(enum.IntEnum):
    Verbose = 0     # internal state dumps, opt-in
    Info = 1        # routing decisions, kernel selection, shape reports
    Warning = 2     # performance issues (fallback paths, misaligned tiles)
    Error = 3       # contract violations that produce wrong results
    Fatal = 4       # invariant broken, cannot continue safely


def OaValidationSeverityName(sev: OaValidationSeverity) -> str:
    return {0: "VERBOSE", 1: "INFO", 2: "WARNING", 3: "ERROR", 4: "FATAL"}.get(int(sev), "?")


_MODES = ("core", "sync", "nan")


class OaValidation:
    """Global validation controller (all members static, as in the reference)."""
    _enabled = False
    _min = OaValidationSeverity.Warning
    _mode = "core"
    _callback: Optional[Callable[[OaValidationSeverity, str, str], None]] = None
    _counters: Dict[str, int] = {}
    _lock = threading.Lock()
    _errors = 0

    # ---- switches
    @staticmethod
    def Enable(enable: bool = True) -> None:
        OaValidation._enabled = bool(enable)

    @staticmethod
    def IsEnabled() -> bool:
        return OaValidation._enabled

    @staticmethod
    def InitFromEnv() -> None:
        """Applies OA_VALIDATION, OA_VALIDATION_SEVERITY and OA_VALIDATION_MODE.  Unknown values are an error: a validation
        run that silently ran with the layer off proves nothing."""
        on = os.environ.get("OA_VALIDATION", os.environ.get("OA_VALIDATE", ""))
        if on not in ("", "0", "1"):
            raise OaError(OaStatus.Error(OaStatusCode.InvalidArgument, f"OA_VALIDATION must be 0 or 1, got {on!r}"))
        OaValidation._enabled = on == "1"
        sev = os.environ.get("OA_VALIDATION_SEVERITY", "")
        if sev:
            names = {s.name.lower(): s for s in OaValidationSeverity}
            if sev.lower() not in names:
                raise OaError(OaStatus.Error(OaStatusCode.InvalidArgument, f"OA_VALIDATION_SEVERITY: unknown severity {sev!r}"))
            OaValidation._min = names[sev.lower()]
        mode = os.environ.get("OA_VALIDATION_MODE", "")
        if mode:
            if mode not in _MODES:
                raise OaError(OaStatus.Error(OaStatusCode.InvalidArgument, f"OA_VALIDATION_MODE must be one of {_MODES}, got {mode!r}"))
            OaValidation._mode = mode

    @staticmethod
    def SetMode(mode: str) -> None:
        if mode not in _MODES:
            raise ValueError(f"validation mode must be one of {_MODES}")
        OaValidation._mode = mode

    @staticmethod
    def Mode() -> str:
        return OaValidation._mode

    @staticmethod
    def SetMinSeverity(sev: OaValidationSeverity) -> None:
        OaValidation._min = OaValidationSeverity(sev)

    @staticmethod
    def GetMinSeverity() -> OaValidationSeverity:
        return OaValidation._min

    @staticmethod
    def SetCallback(cb: Optional[Callable[[OaValidationSeverity, str, str], None]]) -> None:
        """cb(severity, component, message); None restores the default (the framework log)."""
        OaValidation._callback = cb

    # ---- reporting
    @staticmethod
    def Report(sev: OaValidationSeverity, component: str, fmt: str, *args) -> OaStatus:
        """Formats and delivers one message.  Returns an error status for Error / Fatal, Ok below."""
        sev = OaValidationSeverity(sev)
        msg = (fmt % args) if args else fmt
        OaValidation.IncrCounter("validation." + OaValidationSeverityName(sev).lower())
        if sev >= OaValidationSeverity.Error:
            OaValidation._errors += 1
        if sev >= OaValidation._min:
            cb = OaValidation._callback
            if cb is not None:
                cb(sev, component, msg)
            else:
                from ..utils import log as L
                comp = getattr(L.OaLogComponent, component, L.OaLogComponent.Core)
                emit = L.OA_LOG_ERROR if sev >= OaValidationSeverity.Error else L.OA_LOG_WARN if sev == OaValidationSeverity.Warning else L.OA_LOG_INFO
                emit(comp, "%s", f"[validation:{OaValidationSeverityName(sev)}] {component}: {msg}")
        if sev >= OaValidationSeverity.Error:
            return OaStatus.Error(OaStatusCode.FailedPrecondition if sev == OaValidationSeverity.Error else OaStatusCode.Internal, msg)
        return OaStatus.Ok()

    @staticmethod
    def ErrorCount() -> int:
        """Reports of severity Error or Fatal since the last ResetCounters (whatever the severity filter shows)."""
        return OaValidation._errors

    # ---- counters
    @staticmethod
    def IncrCounter(name: str, n: int = 1) -> None:
        if not OaValidation._enabled:
            return
        with OaValidation._lock:
            OaValidation._counters[name] = OaValidation._counters.get(name, 0) + n

    IncrCounterNamed = IncrCounter

    @staticmethod
    def GetCounter(name: str) -> int:
        return OaValidation._counters.get(name, 0)

    @staticmethod
    def Counters() -> Dict[str, int]:
        with OaValidation._lock:
            return dict(OaValidation._counters)

    @staticmethod
    def ResetCounters() -> None:
        with OaValidation._lock:
            OaValidation._counters.clear()
        OaValidation._errors = 0

    @staticmethod
    def DumpCounters(component: str = "Core") -> None:
        from ..utils import log as L
        comp = getattr(L.OaLogComponent, component, L.OaLogComponent.Core)
        for k, v in sorted(OaValidation.Counters().items()):
            if v:
                L.OA_LOG_INFO(comp, "%s", f"[validation:counter] {k} = {v}")


def OA_VALIDATE(cond, sev: OaValidationSeverity, component: str, fmt: str, *args) -> None:
    """`cond` false while the layer is on: report; Error and Fatal raise OaError with the report's status (the Python form
    of "return the error status from the calling function").  `cond` may be a callable, evaluated only when the layer is
    on, for checks that cost something."""
    if not OaValidation._enabled:
        return
    ok = cond() if callable(cond) else cond
    if ok:
        return
    st = OaValidation.Report(sev, component, fmt, *args)
    if not st.IsOk():
        raise OaError(st)


# --------------------------------------------------------------------------------------------- checks used by wrappers
def ValidateTensor(what: str, t, *, dtype=None, cuda: Optional[bool] = None, contiguous: bool = True, align: int = 16,
                   rank: Optional[int] = None) -> None:
    """Argument check of one tensor of a kernel launch (no-op while the layer is off, and for None)."""
    if not OaValidation._enabled or t is None:
        return
    E = OaValidationSeverity.Error
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list, set)) else t.dtype == dtype
        OA_VALIDATE(ok, E, "Kernel", "%s: dtype %s, expected %s", what, t.dtype, dtype)
    if cuda is not None:
        OA_VALIDATE(t.is_cuda == cuda, E, "Kernel", "%s: tensor on %s", what, t.device)
    if contiguous:
        OA_VALIDATE(t.is_contiguous(), E, "Kernel", "%s: not contiguous (shape %s, strides %s)", what, tuple(t.shape), tuple(t.stride()))
    if align and t.numel():
        OA_VALIDATE(t.data_ptr() % align == 0, E, "Kernel", "%s: pointer 0x%x is not %d-byte aligned", what, t.data_ptr(), align)
    if rank is not None:
        OA_VALIDATE(t.dim() == rank, E, "Kernel", "%s: rank %d, expected %d", what, t.dim(), rank)


def AfterLaunch(what: str, outputs=()) -> None:
    """Called by the launch wrapper after every kernel launch while the layer is on."""
    if not OaValidation._enabled:
        return
    OaValidation.IncrCounter("launch." + what.split("(")[0].split(" ")[0])
    mode = OaValidation._mode
    if mode == "core":
        return
    import torch
    if not torch.cuda.is_available():
        return
    torch.cuda.synchronize()
    from ..ops import kernels as K
    code = K.peek_status()
    OA_VALIDATE(code == 0, OaValidationSeverity.Error, "Kernel", "%s: kernel status word %d (%s)", what, code, K.status_name(code))
    if mode == "nan":
        for o in outputs:
            if o is not None and o.is_floating_point() and o.numel():
                OA_VALIDATE(bool(torch.isfinite(o).all()), OaValidationSeverity.Error, "Kernel", "%s: non-finite values in an output of shape %s",
                            what, tuple(o.shape))


OaValidation.InitFromEnv()
