"""Device records, feature gates, scoring and selection against stand-in devices."""
import json

from oa_b200.core.types import OaStatusCode
from oa_b200.runtime.device import (DescribeDevice, GateFeatures, LoadMeasuredPeaks, OaDeviceBuilder, OaDeviceHardwareInfo, OaDeviceInfo,
                                    OaDevicePerformance, OaDevicePreference, OaDeviceType, OaFeatureModule, ScoreDevice, _find)


def _gpu(ordinal, major=10, sms=148, mem=180 << 30, peers=True, lib=True, name="B200"):
    hw = OaDeviceHardwareInfo(ordinal, name, OaDeviceType.DiscreteGpu, major, 0, sms, mem)
    return OaDeviceInfo(hw, GateFeatures(hw, lib, peers), OaDevicePerformance(1500.0, 6600.0, "measured"))


def test_feature_gates():
    b200 = _gpu(0)
    assert b200.Supports(OaFeatureModule.Ml) and b200.Supports(OaFeatureModule.Collective) and not b200.Supports(OaFeatureModule.Render)
    assert b200.Software.Reasons == {"Render": "no graphics stack"} and b200.Hardware.IsBlackwellDataCenter()
    alone = _gpu(0, peers=False)
    assert alone.Supports(OaFeatureModule.Ml) and not alone.Supports(OaFeatureModule.Collective) and "peer" in alone.Software.Reasons["Collective"]
    hopper = _gpu(1, major=9, name="H100")
    assert not hopper.Supports(OaFeatureModule.Core) and "sm_100a only" in hopper.Software.Reasons["Ml"] and ScoreDevice(hopper) == 0
    assert "not loaded" in _gpu(0, lib=False).Software.Reasons["Ml"]
    cpu = DescribeDevice(-1)
    assert cpu.Hardware.Type == OaDeviceType.Cpu and cpu.Supports(OaFeatureModule.Ml) and not cpu.Supports(OaFeatureModule.Collective)
    d = b200.ToDict()
    assert d["compute_capability"] == "10.0" and "Collective" in d["features"] and d["performance_source"] == "measured" and json.dumps(d)


def test_scoring_and_builder():
    devices = {0: _gpu(0, sms=100), 1: _gpu(1, sms=148), 2: _gpu(2, major=9, name="H100")}
    describe = lambda i: devices[i] if i in devices else DescribeDevice(-1)
    b = OaDeviceBuilder(describe, lambda: 3)
    chosen, st = b.Build()
    assert st.IsOk() and chosen.Hardware.Ordinal == 1 and len(b.Candidates()) == 3
    low, _ = OaDeviceBuilder(describe, lambda: 3).SetPreference(OaDevicePreference.LowPower).Build()
    assert low.Hardware.Ordinal == 0
    spec, st = OaDeviceBuilder(describe, lambda: 3).SetPreference(OaDevicePreference.Specific, 2).Require(OaFeatureModule.Ml).Build()
    assert spec is None and st.code == OaStatusCode.FailedPrecondition and "sm_100a" in st.message
    assert OaDeviceBuilder(describe, lambda: 3).SetPreference(OaDevicePreference.Specific, 7).Build()[1].code == OaStatusCode.NotFound
    host, st = OaDeviceBuilder(describe, lambda: 0).Build()
    assert st.IsOk() and host.Hardware.Type == OaDeviceType.Cpu
    none, st = OaDeviceBuilder(describe, lambda: 0).Require(OaFeatureModule.Collective).Build()
    assert none is None and "process group" in st.message
    assert ScoreDevice(_gpu(0)) > ScoreDevice(_gpu(0, peers=False)) > ScoreDevice(_gpu(0, sms=10, peers=False))


def test_measured_peaks_lookup(tmp_path):
    p = tmp_path / "peaks.json"
    p.write_text(json.dumps({"gpu": {"copy": {"hbm_gbs": 6650.0}, "gemm": {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}}}))
    peaks = LoadMeasuredPeaks(str(p))
    assert _find(peaks, "hbm_gbs") == 6650.0 and _find(peaks, "bf16_tflops") == 1590.0 and _find(peaks, "nope") is None
    (tmp_path / "bad.json").write_text("{")
    assert LoadMeasuredPeaks(str(tmp_path / "bad.json")) is None and LoadMeasuredPeaks(str(tmp_path / "missing.json")) is None
