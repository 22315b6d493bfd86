"""Series / frames against numpy and pandas, and the persistent stores on temporary files."""
import math

import numpy as np
import pandas as pd
import pytest

from oa_b200.core.types import OaStatusCode
from oa_b200.data.dataframe import OaDataFrame, OaDataOhlcv, OaRecordOhlcv, OaSeries, OaTimeSeries
from oa_b200.data.stores import OaKeyValueStore, OaOhlcvStore, OaSqlStore, OaStoreKind


def test_series_against_pandas():
    x = np.random.default_rng(0).standard_normal(50) + 5
    s, p = OaSeries(x), pd.Series(x)
    assert s.Size() == 50 and s.Sum() == pytest.approx(p.sum()) and s.Mean() == pytest.approx(p.mean())
    assert s.Std() == pytest.approx(p.std(ddof=0)) and s.Var() == pytest.approx(p.var(ddof=0))
    assert (s.Min(), s.Max(), s.ArgMin(), s.ArgMax()) == (p.min(), p.max(), p.idxmin(), p.idxmax())
    for name, ref in (("RollingSum", p.rolling(7).sum()), ("RollingMean", p.rolling(7).mean()), ("RollingStd", p.rolling(7).std(ddof=0)),
                      ("RollingMin", p.rolling(7).min()), ("RollingMax", p.rolling(7).max())):
        np.testing.assert_allclose(getattr(s, name)(7).Data(), ref.to_numpy(), rtol=1e-9, atol=1e-9, equal_nan=True)
    np.testing.assert_allclose(s.Diff(2).Data(), p.diff(2).to_numpy(), equal_nan=True)
    np.testing.assert_allclose(s.PctChange().Data(), p.pct_change().to_numpy(), equal_nan=True)
    np.testing.assert_array_equal(s.Shift(3, -1.0).Data(), p.shift(3, fill_value=-1.0).to_numpy())
    np.testing.assert_array_equal(s.Shift(-3, 0.0).Data(), p.shift(-3, fill_value=0.0).to_numpy())
    assert s.Shift(100).Sum() == 0 and s.Head(3).ToList() == list(x[:3]) and s.Tail(2).ToList() == list(x[-2:])
    t = (s + s) * 0.5 - s
    assert abs(t.Sum()) < 1e-12
    t += 2; t /= OaSeries(np.full(50, 4.0))
    assert t.Mean() == pytest.approx(0.5)
    with pytest.raises(ValueError):
        s.Add(OaSeries(3))
    with pytest.raises(IndexError):
        s.At(50)
    e = OaSeries(); e.PushBack(1); e.PushBack(3); e.Resize(4)
    assert e.ToList() == [1, 3, 0, 0] and e.ToTensor().shape == (4,)


def test_frame_and_ohlcv():
    bars = OaDataOhlcv([OaRecordOhlcv(t, 10 + t, 12 + t, 9 + t, 11 + t, 100 * t) for t in range(6)])
    assert bars.Size() == 6 and bars.GetRecord(2).Close == 13 and bars.GetRecord(2).IsValid() and not OaRecordOhlcv(0, 5, 4, 3, 2, 1).IsValid()
    df = OaDataFrame.FromOhlcvData(bars)
    assert df.ColumnNames() == ["Time", "Open", "High", "Low", "Close", "Volume"] and df.NumRows() == 6
    df.AddColumn("Mid", (df["High"] + df["Low"]) / OaSeries(np.full(6, 2.0)))
    assert df["Mid"][3] == 13.5 and df.ToTensor(["Open", "Mid"]).shape == (6, 2) and df.Tail(2)["Time"].ToList() == [4, 5]
    with pytest.raises(ValueError):
        df.AddColumn("bad", [1, 2])
    assert df.RemoveColumn("Mid") and not df.RemoveColumn("Mid")
    ts = OaTimeSeries.FromOhlcvClose(bars)
    assert ts.HasTimeIndex() and ts.Slice(1, 3).Values().ToList() == [12, 13]
    with pytest.raises(ValueError):
        OaTimeSeries.Create(OaSeries([2, 1]), OaSeries([0, 0]))


def test_frame_csv(tmp_path):
    df = OaDataFrame(); df.AddColumn("a", [1.5, 2.5]); df.AddColumn("b", [1e-9, -3])
    df.ToCsv(str(tmp_path / "f.csv"))
    back = OaDataFrame.FromCsv(str(tmp_path / "f.csv"))
    assert back.ColumnNames() == ["a", "b"] and back["b"].ToList() == [1e-9, -3.0]


def test_kv_store(tmp_path):
    path = str(tmp_path / "kv.log")
    kv = OaKeyValueStore()
    assert kv.Open(path).IsOk() and kv.Kind() == OaStoreKind.KvOrdered and not kv.Open(path).IsOk()
    for i in range(20):
        assert kv.Put(b"k%02d" % i, b"v" * i).IsOk()
    assert kv.Put(b"k05", b"new").IsOk() and kv.Delete(b"k06").IsOk() and kv.Delete(b"zz").code == OaStatusCode.NotFound
    assert kv.Get(b"k05") == b"new" and kv.Get(b"k06") is None and kv.Get(b"k00") == b"" and kv.Count() == 19
    assert [k for k, _ in kv.Scan(b"k04", b"k08")] == [b"k04", b"k05", b"k07"]
    kv.Close()
    with open(path, "ab") as f:
        f.write(b"\x01\x02\x03torn tail of a crashed write")
    kv = OaKeyValueStore()
    assert kv.Open(path).IsOk() and kv.Count() == 19 and kv.Get(b"k05") == b"new" and kv.DeadRecords() == 3
    size_before = (tmp_path / "kv.log").stat().st_size
    assert kv.CompactStorage().IsOk() and kv.DeadRecords() == 0 and (tmp_path / "kv.log").stat().st_size < size_before
    assert kv.Get(b"k19") == b"v" * 19 and kv.Put(b"a", b"1").IsOk() and next(iter(kv.Scan()))[0] == b"a"
    kv.Close()
    ro = OaKeyValueStore()
    assert ro.Open(path, read_only=True).IsOk() and ro.Get(b"a") == b"1" and not ro.Put(b"b", b"2").IsOk()
    ro.Close()
    assert OaKeyValueStore().Open(str(tmp_path / "none"), read_only=True).code == OaStatusCode.NotFound
    (tmp_path / "junk").write_bytes(b"not a log at all")
    assert OaKeyValueStore().Open(str(tmp_path / "junk")).code == OaStatusCode.DataLoss


def test_sql_and_ohlcv_store(tmp_path):
    sql = OaSqlStore()
    assert sql.Open(":memory:").IsOk() and sql.ExecuteSQL("CREATE TABLE t (a INTEGER)").IsOk() and sql.ExecuteSQL("INSERT INTO t VALUES (3)").IsOk()
    assert sql.Query("SELECT a FROM t") == [(3,)] and not sql.ExecuteSQL("SELEKT").IsOk() and sql.CompactStorage().IsOk()
    sql.Close()
    st = OaOhlcvStore()
    assert st.Open(str(tmp_path / "bars.db")).IsOk()
    recs = [OaRecordOhlcv(float(t), 10, 12, 9, 11, 5) for t in range(10)]
    assert st.SaveRecords("BTC", "spot", "1m", recs).IsOk() and st.SaveRecords("ETH", "perp", "1h", recs[:3]).IsOk()
    assert not st.SaveRecords("BTC", "spot", "1m", [OaRecordOhlcv(1, 5, 4, 3, 2, 1)]).IsOk()
    assert st.SaveRecords("BTC", "spot", "1m", [OaRecordOhlcv(3.0, 1, 2, 1, 2, 9)]).IsOk()        # replaces the bar at t=3
    assert st.GetRecordCount("BTC", "spot", "1m") == 10 and st.LoadRecords("BTC", "spot", "1m", 3, 4)[0].Volume == 9
    assert st.LoadData("BTC", "spot", "1m", start=7).Size() == 3 and st.GetEarliestTimestamp("ETH", "perp", "1h") == 0.0
    assert st.GetLatestTimestamp("BTC", "spot", "1m") == 9.0 and st.GetAllTimestamps("ETH", "perp", "1h") == [0.0, 1.0, 2.0]
    assert [(c.Ticker, c.Interval) for c in st.GetTickerCombinations()] == [("BTC", "1m"), ("ETH", "1h")]
    assert [(s.Ticker, s.Count) for s in st.GetAvailableData()] == [("BTC", 10), ("ETH", 3)]
    assert st.DeleteData("BTC", "spot", "1m", end=4).IsOk() and st.GetRecordCount("BTC", "spot", "1m") == 5
    assert st.GetEarliestTimestamp("X", "y", "z") is None
    st.Close()
