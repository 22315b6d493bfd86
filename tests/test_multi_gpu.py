"""Multi-GPU checks, each run as torchrun child processes on 2 GPUs (skipped on a single-GPU box)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script: str, nproc: int = 2, timeout: int = 240) -> str:
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "multi_gpu", script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def test_expert_parallel_matches_single_device():
    assert "EP_CHECK_OK" in _run("ep_check.py")


def test_tensor_parallel_kernels_and_model():
    assert "TP_CHECK_OK" in _run("tp_check.py")


def test_tensor_parallel_decoding():
    assert "TP_DECODE_CHECK_OK" in _run("tp_decode_check.py")


def test_collective_verbs_match_nccl():
    assert "COLLECTIVE_CHECK_OK" in _run("collective_check.py")


def test_data_parallel_fused_step_clipping_and_checkpoint():
    assert "DP_CHECK_OK" in _run("dp_check.py", timeout=400)
