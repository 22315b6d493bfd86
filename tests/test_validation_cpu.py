"""OaValidation layer: switches from the environment, severity filter, callback, counters, OA_VALIDATE raising on Error,
argument checks of tensors (Source/Public/Oa/Core/Validation.h:45-140 of the reference; its tests drive the same surface
through Test/Core/Misc/TestValidation.cpp)."""
import os
import subprocess
import sys

import pytest
import torch

from oa_b200.core.types import OaError
from oa_b200.core.validation import OA_VALIDATE, OaValidation, OaValidationSeverity, OaValidationSeverityName, ValidateTensor


@pytest.fixture
def layer():
    seen = []
    OaValidation.Enable(True)
    OaValidation.ResetCounters()
    OaValidation.SetMinSeverity(OaValidationSeverity.Verbose)
    OaValidation.SetCallback(lambda sev, comp, msg: seen.append((sev, comp, msg)))
    yield seen
    OaValidation.SetCallback(None)
    OaValidation.SetMinSeverity(OaValidationSeverity.Warning)
    OaValidation.ResetCounters()
    OaValidation.SetMode("core")
    OaValidation.Enable(False)


def test_off_by_default_and_free_when_off():
    assert not OaValidation.IsEnabled()
    OA_VALIDATE(False, OaValidationSeverity.Fatal, "Core", "never evaluated %d", 1)       # no raise while off
    OA_VALIDATE(lambda: 1 / 0, OaValidationSeverity.Error, "Core", "the callable is not called while off")
    OaValidation.IncrCounter("x")
    assert OaValidation.GetCounter("x") == 0


def test_report_severity_filter_callback_and_counters(layer):
    assert OaValidation.Report(OaValidationSeverity.Info, "Core", "kernel %s chosen", "pair").IsOk()
    st = OaValidation.Report(OaValidationSeverity.Error, "Kernel", "M must be > 0, got %d", 0)
    assert not st.IsOk() and "got 0" in st.message
    assert [s for s, _, _ in layer] == [OaValidationSeverity.Info, OaValidationSeverity.Error]
    assert OaValidation.GetCounter("validation.info") == 1 and OaValidation.GetCounter("validation.error") == 1
    assert OaValidation.ErrorCount() == 1
    OaValidation.SetMinSeverity(OaValidationSeverity.Error)
    OaValidation.Report(OaValidationSeverity.Warning, "Core", "filtered")
    assert len(layer) == 2 and OaValidation.GetCounter("validation.warning") == 1      # counted, not delivered
    OaValidation.ResetCounters()
    assert OaValidation.GetCounter("validation.info") == 0 and OaValidation.ErrorCount() == 0
    assert OaValidationSeverityName(OaValidationSeverity.Fatal) == "FATAL"


def test_validate_macro_raises_from_error_upwards(layer):
    OA_VALIDATE(True, OaValidationSeverity.Error, "Core", "fine")
    OA_VALIDATE(False, OaValidationSeverity.Warning, "Core", "slow path for %s", "x")        # reported, no raise
    with pytest.raises(OaError) as e:
        OA_VALIDATE(lambda: False, OaValidationSeverity.Error, "Core", "rows %d exceed %d", 9, 8)
    assert "rows 9 exceed 8" in str(e.value)
    assert len(layer) == 2


def test_tensor_argument_checks(layer):
    t = torch.zeros(8, 16)
    ValidateTensor("ok", t, dtype=torch.float32, cuda=False, rank=2)
    with pytest.raises(OaError, match="dtype"):
        ValidateTensor("a", t, dtype=torch.bfloat16)
    with pytest.raises(OaError, match="not contiguous"):
        ValidateTensor("b", t.t())
    with pytest.raises(OaError, match="aligned"):
        ValidateTensor("c", torch.zeros(33)[1:])
    with pytest.raises(OaError, match="rank"):
        ValidateTensor("d", t, rank=3)
    ValidateTensor("none", None)


def test_launch_wrapper_counts_by_entry_point(layer):
    from oa_b200.core import validation as V
    V.AfterLaunch("oa_gemm_bf16 M=128 N=128 K=64")
    V.AfterLaunch("oa_peer_push(counts)")
    V.AfterLaunch("oa_peer_push(stats)")
    assert OaValidation.GetCounter("launch.oa_gemm_bf16") == 1 and OaValidation.GetCounter("launch.oa_peer_push") == 2


def _child(env):
    code = ("from oa_b200.core.validation import OaValidation as V;"
            "print(V.IsEnabled(), V.Mode(), int(V.GetMinSeverity()))")
    e = dict(os.environ)
    e.update(env)
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=e,
                          cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_environment_switches():
    r = _child({"OA_VALIDATION": "1", "OA_VALIDATION_MODE": "sync", "OA_VALIDATION_SEVERITY": "info"})
    assert r.returncode == 0 and r.stdout.split() == ["True", "sync", "1"], r.stderr[-2000:]
    r = _child({"OA_VALIDATION": "0"})
    assert r.stdout.split()[0] == "False"
    r = _child({"OA_VALIDATION": "1", "OA_VALIDATION_MODE": "everything"})
    assert r.returncode != 0 and "OA_VALIDATION_MODE" in r.stderr
