"""Logging, scalar-metric stream, rolling statistics, the performance store and profiler ranges."""
import io
import json
import os

import numpy as np
import pytest

from oa_b200.core.types import OaStatusCode
from oa_b200.utils.log import (OA_LOG_DEBUG, OA_LOG_INFO, OA_LOG_WARN, OaGetComponentName, OaLog, OaLogComponent, OaLogLevel, OaLogSummary,
                               OaMetricsWriter)
from oa_b200.utils.perf import OaNvtxRange, OaPerfRecord, OaPerfStat, OaPerfStore


def test_log_levels_components_and_file(tmp_path):
    log = OaLog.Instance()
    assert log is OaLog.Instance()
    log.Init(str(tmp_path), "unit", OaLogLevel.Info, console=False)
    OA_LOG_DEBUG(OaLogComponent.Core, "hidden %d", 1)
    OA_LOG_INFO(OaLogComponent.ML, "step %d loss %.3f", 7, 0.25)
    OA_LOG_WARN(OaLogComponent.Execution, "plain text with a %% sign kept as is" if False else "plain text")
    OaLogSummary(OaLogComponent.App, "parameters", 1234567)
    log.SetLevel(OaLogLevel.Off)
    OA_LOG_WARN(OaLogComponent.Core, "silenced")
    log.Close()
    lines = open(log.Path).read().splitlines()
    assert len(lines) == 3 and "[INFO ] [ML  ] step 7 loss 0.250" in lines[0] and "[WARN ] [EXEC] plain text" in lines[1]
    assert lines[2].endswith("1,234,567") and "parameters ." in lines[2] and len(lines[2].split("] ", 2)[2]) == 60
    assert OaGetComponentName(OaLogComponent.Storage) == "STOR"
    log.Init(level=OaLogLevel.Info)


def test_metrics_writer(tmp_path):
    path = str(tmp_path / "m" / "metrics.jsonl")
    w = OaMetricsWriter(path, flush_interval=2)
    w.LogScalar("loss", 1, 0.5)
    w.LogScalars("eval", 2, {"acc": 0.9, "ppl": 3.0})
    w.Close()
    w.LogScalar("late", 3, 1.0)                      # after Close: ignored
    rows = [json.loads(l) for l in open(path)]
    assert [(r["tag"], r["step"], r["value"]) for r in rows] == [("loss", 1, 0.5), ("eval/acc", 2, 0.9), ("eval/ppl", 2, 3.0)]
    assert all(r["wall_time"] > 0 for r in rows)


def test_rolling_statistics_against_numpy():
    x = np.random.default_rng(0).random(200)
    s = OaPerfStat("step_ms")
    for v in x:
        s.Add(v)
    assert s.Count() == 200 and s.Mean() == pytest.approx(x.mean()) and s.Stddev() == pytest.approx(x.std()) and s.Min() == x.min()
    for q in (0.5, 0.95, 0.99):
        assert s.Percentile(q) == pytest.approx(np.percentile(x, 100 * q))
    w = OaPerfStat("w", window=10)
    for v in x:
        w.Add(v)
    assert w.Count() == 10 and w.TotalSamples == 200 and w.Mean() == pytest.approx(x[-10:].mean()) and w.Max() == x[-10:].max()
    w.Reset()
    assert w.Count() == 0 and w.Mean() == 0.0 and w.Percentile(0.5) == 0.0


def test_perf_store_round_trip(tmp_path):
    path = str(tmp_path / "perf" / "OaPerf.dat")
    store = OaPerfStore()
    assert store.Load(path).IsOk() and store.RecordCount() == 0
    s = OaPerfStat("gemm_tflops")
    for v in (100.0, 110.0, 120.0):
        s.Add(v)
    first = s.ToRecord("NVIDIA B200")
    assert store.Append(first).IsOk() and store.Append(OaPerfRecord(1, "other gpu", "gemm_tflops", 1, 5.0)).IsOk()
    s.Add(200.0)
    again = OaPerfStore()
    assert again.Load(path).IsOk() and again.RecordCount() == 2
    got = again.FindLatest("NVIDIA B200", "gemm_tflops")
    assert got == first and got.P50 == 110.0 and again.FindLatest("NVIDIA B200", "nope") is None
    text = again.Comparison("gemm_tflops", s.ToRecord("NVIDIA B200"), "NVIDIA B200")
    assert "132.5000 vs 110.0000 (+20.45 %)" in text
    assert "no earlier record" in again.Comparison("x", first, "NVIDIA B200")
    with open(path, "ab") as f:
        f.write(b"torn")
    assert OaPerfStore().Load(path).code == OaStatusCode.DataLoss


def test_profiler_range_is_harmless_without_a_gpu():
    with OaNvtxRange("forward"):
        with OaNvtxRange("attention"):
            pass
    with pytest.raises(ZeroDivisionError):
        with OaNvtxRange("failing"):
            1 / 0
