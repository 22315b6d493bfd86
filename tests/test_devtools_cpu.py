"""Tooling layer: generated tables and their drift gate, kernel audit, architecture gate, evidence bundles, determinism
comparison (Tools/check_autogen_drift.py, Tools/audit_kernels.py, Tools/Architecture/test_oacheck.py,
Tools/Diagnostics/test_oaevidence.py and test_oadeterminism.py of the reference)."""
import json
import re
import sys
from pathlib import Path

import pytest

from oa_b200.devtools import archcheck, autogen, determinism, evidence


# ---------------------------------------------------------------------------------------------------------- autogen
def test_generated_tables_match_their_generators():
    drift = autogen.check()
    assert drift == [], f"generated files differ from the generators: {drift} (run python -m oa_b200.devtools.autogen)"


def test_kernel_table_covers_the_binding_and_ids_are_unique():
    from oa_b200 import _native as N
    from oa_b200._generated import kernel_table as KT
    assert {k[0] for k in KT.KERNELS} == {p[0] for p in N._PROTOS}
    assert len({k[3] for k in KT.KERNELS}) == len(KT.KERNELS)
    assert KT.KERNEL_ID["oa_gemm_bf16"] == autogen.fnv1a32("oa_gemm_bf16")
    assert KT.CONSTANTS["OA_BF16"] == 1 and KT.CONSTANTS == N.CONST
    by_file = {k[2] for k in KT.KERNELS}
    assert {"gemm_tcgen05.cu", "flash_attn.cu", "comm.cu", "moe.cu", "mamba3_ssd.cu"} <= by_file


def test_header_parser_sections_and_comment_forms():
    text = """
enum { A_X = 0, A_Y, A_Z = 7 };
// ---- first things (one.cu): a description (with parentheses)
int oa_one(const void* x, long long n, void* stream);
// int oa_quoted(int a);   a prototype inside a comment is not an entry point
// ---- two.cu: second form of a section comment
size_t oa_two(int rows);
void oa_three(unsigned a,
              float b);
"""
    rows, consts = autogen.parse_api(text)
    assert consts == {"A_X": 0, "A_Y": 1, "A_Z": 7}
    assert [(r["name"], r["file"], r["returns"], r["args"]) for r in rows] == [
        ("oa_one", "one.cu", "int", ["ptr", "long long", "ptr"]), ("oa_two", "two.cu", "size_t", ["int"]),
        ("oa_three", "two.cu", "void", ["unsigned", "float"])]


def test_kernel_audit_has_no_missing_definition():
    res = autogen.audit()
    assert res["MISSING"] == [], res["MISSING"]
    # (the allocation-free entry points are declared in a header of their own, which the audit reads too)
    assert res["UNDECLARED"] == [], res["UNDECLARED"]


def test_operation_contracts_name_real_kernels():
    from oa_b200._generated import kernel_table as KT
    ops = json.loads((autogen.OUT / "operation_contracts.json").read_text())["operations"]
    assert len(ops) > 150
    names = {k[0] for k in KT.KERNELS}
    for o in ops:
        assert set(o["kernels"]) <= names, o
    by = {o["name"]: o for o in ops}
    assert by["Linear"]["lowering"] == "Gemm" and by["Linear"]["differentiation"] == "Analytic"
    assert by["Dropout"]["effects"] == "Random"


# --------------------------------------------------------------------------------------------------------- archcheck
def test_package_dependencies_follow_the_policy():
    assert archcheck.check() == []


def _tree(tmp_path, files):
    root = tmp_path / "pkg"
    for rel, src in files.items():
        p = root / rel
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(src)
    return root


def test_archcheck_reports_new_edges_and_stale_baselines(tmp_path):
    root = _tree(tmp_path, {"__init__.py": "", "low/__init__.py": "", "low/a.py": "import os\n",
                            "high/__init__.py": "", "high/b.py": "from ..low import a\nfrom ..low.a import os\n",
                            "low/bad.py": "def f():\n    from ..high import b\n    return b\n"})
    policy = tmp_path / "modules.json"
    policy.write_text(json.dumps({"version": 1, "modules": {"low": {"allows": []}, "high": {"allows": ["low"]}}}))
    baseline = tmp_path / "baseline.json"
    problems = archcheck.check(root, policy, baseline)
    assert len(problems) == 1 and problems[0].startswith("low->high: new forbidden dependency") and "low/bad.py:2" in problems[0]
    baseline.write_text(json.dumps({"version": 1, "edges": {"low->high": 1}}))
    assert archcheck.check(root, policy, baseline) == []
    baseline.write_text(json.dumps({"version": 1, "edges": {"low->high": 3}}))
    assert any("lower or delete" in p for p in archcheck.check(root, policy, baseline))
    (root / "low" / "bad.py").write_text("from ..high import b\nfrom ..high.b import a\n")
    baseline.write_text(json.dumps({"version": 1, "edges": {"low->high": 1}}))
    assert any("2 imports, the baseline accepts 1" in p for p in archcheck.check(root, policy, baseline))
    policy.write_text(json.dumps({"version": 1, "modules": {"low": {"allows": []}}}))
    assert any("'high' has no entry" in p for p in archcheck.check(root, policy, baseline))


# ---------------------------------------------------------------------------------------------------------- evidence
def test_evidence_bundle_records_verifies_and_detects_tampering(tmp_path):
    art = tmp_path / "result.json"
    art.write_text('{"x": 1}\n')
    out = tmp_path / "bundle"
    cmd = [sys.executable, "-c", "print('step 1'); print('{\"metric\": \"tokens/s\", \"value\": 12.5}')"]
    m = evidence.collect(out, cmd, attach=[art])
    assert m["ok"] and m["schema"] == evidence.SCHEMA
    assert m["workload"]["exit_status"] == 0 and m["workload"]["result"] == {"metric": "tokens/s", "value": 12.5}
    assert set(m["git"]) == {"commit", "branch", "dirty", "dirty_files"}              # empty strings outside a git checkout
    assert set(m["files"]) == {"kernel_library", "runtime_library", "kernel_header", "measured_peaks"}
    assert m["artifacts"][0]["name"] == "result.json" and "artifacts/result.json" in m["checksums"]
    assert evidence.verify(out) == []
    (out / "stdout.log").write_text("edited\n")
    (out / "extra.txt").write_text("x")
    problems = evidence.verify(out)
    assert "checksum differs: stdout.log" in problems and "not in the manifest: extra.txt" in problems


def test_evidence_fails_on_validation_errors_and_bad_exit(tmp_path):
    bad = [sys.executable, "-c", "import os; print('[validation:ERROR] Kernel: gemm.a: pointer is not 16-byte aligned'); "
                                 "print(os.environ['OA_VALIDATION'], os.environ['OA_VALIDATION_MODE'])"]
    m = evidence.collect(tmp_path / "v", bad, validation="sync")
    assert not m["ok"] and m["validation"] == {"requested": "sync", "errors": 1, "first_errors": m["validation"]["first_errors"]}
    assert "1 sync" in (tmp_path / "v" / "stdout.log").read_text()
    m = evidence.collect(tmp_path / "e", [sys.executable, "-c", "raise SystemExit(3)"])
    assert not m["ok"] and m["workload"]["exit_status"] == 3
    with pytest.raises(FileNotFoundError):
        evidence.collect(tmp_path / "a", attach=[tmp_path / "nope.bin"])


# ------------------------------------------------------------------------------------------------------- determinism
def test_trace_extraction_forms():
    text = "step 1 loss=0.5000\n\x1b[31mstep 2 loss=0.2500\x1b[0m\n"
    assert determinism.extract_trace(re.compile(r"loss=(?P<value>[0-9.]+)"), text) == ["0.5000", "0.2500"]
    assert determinism.extract_trace(re.compile(r"loss=([0-9.]+)"), text) == ["0.5000", "0.2500"]
    assert determinism.extract_trace(re.compile(r"step \d"), text) == ["step 1", "step 2"]
    with pytest.raises(ValueError):
        determinism.extract_trace(re.compile(r"(step) (\d)"), text)


def test_trace_comparison():
    assert determinism.first_difference(["1", "2"], ["1", "2"]) is None
    assert determinism.first_difference(["1", "2"], ["1", "3"]) == 1
    assert determinism.first_difference(["1"], ["1", "2"]) == 1
    assert determinism.first_difference(["1.0000001"], ["1.0000002"], tolerance=1e-6) is None
    rep = determinism.compare([["a", "b"], ["a", "b"], ["a", "c"]])
    assert not rep["deterministic"] and rep["differences"] == [{"run": 2, "index": 1, "first": "b", "other": "c"}]
    assert not determinism.compare([[], []])["deterministic"]


def test_workload_runs_in_fresh_processes(tmp_path):
    same = [sys.executable, "-c", "import random; random.seed(3); [print('loss=%.6f' % random.random()) for _ in range(5)]"]
    rep = determinism.run_workload(same, 3, re.compile(r"loss=([0-9.]+)"), tmp_path / "same", name="seeded")
    assert rep["ok"] and rep["lengths"] == [5, 5, 5] and len({r["trace_sha256"] for r in rep["runs"]}) == 1
    assert json.loads((tmp_path / "same" / "determinism.json").read_text())["schema"] == determinism.SCHEMA
    differs = [sys.executable, "-c", "import os; print('loss=0.5'); print('loss=%d' % os.getpid())"]
    rep = determinism.run_workload(differs, 2, re.compile(r"loss=([0-9.]+)"), None, name="pid")
    assert not rep["ok"] and rep["differences"][0]["index"] == 1
    assert determinism.main(["--name", "cli", "--runs", "2", "--trace", r"loss=([0-9.]+)", "--"] + same) == 0


def test_model_digest_changes_with_a_weight():
    import torch
    from oa_b200.ml.nn.layers import OaLinear
    m = OaLinear(4, 3)
    a = determinism.model_digest(m)
    assert a == determinism.model_digest(m) and len(a) == 16
    m.AllParameterPtrs()[0].Tensor().view(-1)[0] += 1.0
    assert determinism.model_digest(m) != a
    assert determinism.tensor_digest(torch.zeros(3)) != determinism.tensor_digest(torch.zeros(3, dtype=torch.float64))
