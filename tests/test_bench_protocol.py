"""The benchmark protocol on a stand-in benchmark: fresh processes, median / MAD, fail-closed comparison."""
import json
import sys

import pytest

import bench_protocol as BP


def _fake(tmp_path, value_expr, metric="tokens/s", extra=""):
    script = tmp_path / "fake_bench.py"
    script.write_text("import json, os, sys\nprint('warming up')\n"
                      f"v = {value_expr}\n"
                      f"print(json.dumps({{'metric': '{metric}', 'value': v, 'unit': 'tokens/s', 'n_gpus': 1, 'dtype': 'bf16', "
                      f"'config': {{'model': 'tiny'{extra}}}, 'higher_is_better': True}}))\n")
    return [sys.executable, str(script)]


def test_run_summarise_compare_accept(tmp_path):
    lines = []
    base_path, cand_path = str(tmp_path / "base.json"), str(tmp_path / "cand.json")
    cmd = _fake(tmp_path, "1000.0 + (os.getpid() % 7)")
    assert BP.main(["run", "--runs", "7", "--out", cand_path, "--"] + cmd, out=lines.append) == 0
    res = json.load(open(cand_path))
    assert res["runs"] == 7 and 1000 <= res["median"] <= 1006 and res["mad"] <= 3 and res["metric"] == "tokens/s" and res["schema"] == BP.SCHEMA
    assert BP.main(["accept", "--candidate", cand_path, "--baseline", base_path], out=lines.append) == 0
    assert BP.main(["compare", "--baseline", base_path, "--candidate", cand_path], out=lines.append) == 0 and "unchanged" in lines[-1]
    slow = dict(res, median=res["median"] * 0.8, values=[v * 0.8 for v in res["values"]])
    json.dump(slow, open(cand_path, "w"))
    assert BP.main(["compare", "--baseline", base_path, "--candidate", cand_path], out=lines.append) == 2 and "regressed" in lines[-1]
    fast = dict(res, median=res["median"] * 1.5)
    assert BP.Compare(res, fast)["verdict"] == "improved"
    other = dict(res, config={"model": "other"})
    json.dump(other, open(cand_path, "w"))
    assert BP.main(["compare", "--baseline", base_path, "--candidate", cand_path], out=lines.append) == 3 and "not comparable" in lines[-1]
    few = dict(res, runs=3)
    assert not BP.Compare(res, few)["comparable"]
    lower = dict(res, higher_is_better=False)
    assert BP.Compare(lower, dict(lower, median=res["median"] * 0.5))["verdict"] == "improved"


def test_failures_are_reported(tmp_path):
    lines = []
    out = str(tmp_path / "o.json")
    assert BP.main(["run", "--runs", "3", "--out", out, "--", sys.executable, "-c", "print(1)"], out=lines.append) == 1 and "at least 7" in lines[-1]
    assert BP.main(["run", "--runs", "7", "--out", out, "--", sys.executable, "-c", "print('no json')"], out=lines.append) == 1
    assert BP.main(["run", "--runs", "7", "--out", out, "--", sys.executable, "-c", "raise SystemExit(4)"], out=lines.append) == 1
    assert BP.ParseRun('noise\n{"metric": "m", "value": 1}\n{"other": 2}\ntrailer') == {"metric": "m", "value": 1}
    assert BP.ParseRun("{broken") is None and BP.Mad([1, 2, 3, 4, 100]) == 1
    with pytest.raises(ValueError):
        BP.Summarise([{"metric": "a", "value": 1}, {"metric": "b", "value": 2}], [])
