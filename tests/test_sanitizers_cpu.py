"""The native runtime under the compiler's sanitizers, and the device synchronisation protocols emulated on host threads
under the race detector.

* `csrc/runtime/*.cpp` + `check/sanitize_main.cpp` built with -fsanitize=address,undefined and again with
  -fsanitize=thread: the driver walks the C API of the compute graph, plan cache, pool / channel / locks, .oam writer and
  loader (with truncated and bit-flipped files), asynchronous reader and allocation session.
* `check/protocol_emulation.cpp` built with -fsanitize=thread: the flag / epoch protocols of the data-parallel fused step
  of the tensor-parallel call sites and of the expert-parallel dispatch, several seeds; two negative controls (one ordering edge removed) must be
  REPORTED by the detector.

Reference strategy: the upstream project's host validation profile builds everything with -fsanitize=address,undefined
(CMakeLists.txt:68-96, OA_SANITIZERS); the thread-sanitizer runs and the protocol emulation have no upstream counterpart
(its collectives stage through the host)."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
RUNTIME = ROOT / "oa_b200" / "csrc" / "runtime"
CHECK = RUNTIME / "check"
COMMON = ["g++", "-O1", "-g", "-std=c++17", "-pthread", "-fno-omit-frame-pointer"]


def _have(flag: str, tmp: Path) -> bool:
    src = tmp / "probe.cpp"
    src.write_text("int main() { return 0; }\n")
    exe = tmp / ("probe" + flag.replace("=", "_").replace(",", "_"))
    r = subprocess.run(["g++", flag, str(src), "-o", str(exe)], capture_output=True)
    return r.returncode == 0 and subprocess.run([str(exe)], capture_output=True).returncode == 0


def _build(tmp: Path, name: str, flags, sources) -> Path:
    exe = tmp / name
    r = subprocess.run([*COMMON, *flags, "-I", str(RUNTIME), "-o", str(exe), *map(str, sources)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return exe


def _env(**extra):
    env = dict(os.environ)
    env.pop("LD_PRELOAD", None)
    env.update(extra)
    return env


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    return tmp_path_factory.mktemp("sanitize")


def _runtime_sources():
    return [CHECK / "sanitize_main.cpp", *sorted(RUNTIME.glob("*.cpp"))]


def test_runtime_under_address_and_undefined_behaviour_sanitizers(workdir):
    if not _have("-fsanitize=address,undefined", workdir):
        pytest.skip("ASAN/UBSAN runtime not installed")
    exe = _build(workdir, "rt_asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], _runtime_sources())
    scratch = workdir / "asan_files"
    scratch.mkdir()
    r = subprocess.run([str(exe), str(scratch)], capture_output=True, text=True, timeout=300,
                       env=_env(ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    assert "all ok" in r.stdout
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr and "LeakSanitizer" not in r.stderr


def test_runtime_under_thread_sanitizer(workdir):
    if not _have("-fsanitize=thread", workdir):
        pytest.skip("TSAN runtime not installed")
    exe = _build(workdir, "rt_tsan", ["-fsanitize=thread"], _runtime_sources())
    scratch = workdir / "tsan_files"
    scratch.mkdir()
    r = subprocess.run([str(exe), str(scratch)], capture_output=True, text=True, timeout=300, env=_env(TSAN_OPTIONS="halt_on_error=1"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    assert "all ok" in r.stdout and "ThreadSanitizer" not in r.stderr


@pytest.fixture(scope="module")
def emulation(workdir):
    if not _have("-fsanitize=thread", workdir):
        pytest.skip("TSAN runtime not installed")
    return _build(workdir, "proto_tsan", ["-fsanitize=thread"], [CHECK / "protocol_emulation.cpp"])


@pytest.mark.parametrize("what", ["dp", "tp", "ep", "timeout"])
def test_protocols_are_race_free_over_random_interleavings(emulation, what):
    for seed in (1, 2, 3, 4, 5, 6):
        r = subprocess.run([str(emulation), what, str(seed)], capture_output=True, text=True, timeout=300,
                           env=_env(TSAN_OPTIONS="halt_on_error=1"))
        assert r.returncode == 0 and "ThreadSanitizer" not in r.stderr, f"{what} seed {seed}\n" + r.stdout[-2000:] + r.stderr[-6000:]
        assert r.stdout.strip().endswith("ok")


@pytest.mark.parametrize("what", ["dp-no-ack", "tp-no-fence"])
def test_detector_reports_a_protocol_with_one_edge_removed(emulation, what):
    """Without the parameters-complete round a rank's next backward pass overwrites gradients that a peer still reads; without
    the ready/ack round between two uses of one call site a peer's push overwrites rows that are still being read."""
    r = subprocess.run([str(emulation), what, "1"], capture_output=True, text=True, timeout=300, env=_env(TSAN_OPTIONS="halt_on_error=0"))
    assert "ThreadSanitizer: data race" in r.stderr, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.returncode != 0
