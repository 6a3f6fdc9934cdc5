"""Every per-operator executable validates itself on the GPU: exit code 0 and a final [SUCCESS] line, the protocol of
the reference's test+benchmark programs (AGENTS.md:42-44; CTest registration CMakeLists.txt:246-334).  The timing stage
is skipped (--correctness-only); bench.py and the executables' default mode do the timing."""
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "cudaop_b200", "bench")


def _run(args, timeout=600):
    exe = os.path.join(BENCH, args[0])
    assert os.path.exists(exe), f"{exe} is not built: python -m cudaop_b200.build"
    r = subprocess.run([exe] + args[1:], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert r.returncode == 0, r.stdout[-3000:]
    assert lines and lines[-1].startswith("[SUCCESS]"), r.stdout[-3000:]
    assert not any(l.startswith("[FAILED]") for l in lines)
    return lines


def _executables():
    return sorted(f[:-3] for f in os.listdir(BENCH) if f.endswith(".cu") and f != "nccl_mlp_test.cu")


@pytest.mark.parametrize("exe", _executables())
def test_operator_executable_passes_its_own_check(exe):
    lines = _run([exe, "--correctness-only"])
    assert any(l.startswith("[CONFIG]") for l in lines) and any(l.startswith("[STAGE]") for l in lines)


def test_nccl_mlp_test_on_one_gpu():
    _run(["nccl_mlp_test", "--correctness-only", "--case", "small", "--gpus", "1"])


@pytest.mark.parametrize("comm", ["fused", "pipelined", "nccl"])
def test_nccl_mlp_test_on_two_gpus(comm):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(["nccl_mlp_test", "--correctness-only", "--case", "small", "--gpus", "2", "--comm", comm])


def test_profile_flag_runs_the_steady_state_launch_only():
    lines = _run(["gemm_fp8_bf16", "--profile", "--case", "config"])
    assert not any(l.startswith("[BENCHMARK]") for l in lines)
