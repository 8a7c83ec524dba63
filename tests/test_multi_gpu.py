"""Multi-process tests (one process per GPU); skipped where fewer than two GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _torchrun(nproc, args, port):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "rbruck_alltoallv_b200.utils.selftest", *args]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


@pytest.mark.skipif(_ngpus() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_two_processes(nranks):
    res = _torchrun(2, ["--nranks", str(nranks)], 29611 + nranks)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert '"selftest": "ok"' in res.stdout


@pytest.mark.skipif(_ngpus() < 4, reason="needs 4 GPUs")
def test_four_processes():
    res = _torchrun(4, ["--nranks", "8"], 29631)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.skipif(_ngpus() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("extra", [[], ["--mx"]], ids=["bf16", "mxfp8"])
def test_moe_two_processes_matches_reference(extra):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29651", "-m", "rbruck_alltoallv_b200.utils.moe_bench", "--tokens", "512",
           "--hidden", "512", "--inter", "1024", "--experts-per-rank", "4", "--check", "--steps", "3"] + extra
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert '"check": "ok"' in res.stdout


@pytest.mark.skipif(_ngpus() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("pr,pc", [(2, 1), (1, 2)])
def test_fft_transposes_two_processes(pr, pc):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29661", "-m", "rbruck_alltoallv_b200.utils.fft_bench", "--size", "48", "--pr", str(pr),
           "--pc", str(pc), "--check", "--steps", "2", "--warmup", "1"]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert '"check": "ok"' in res.stdout


@pytest.mark.skipif(_ngpus() < 2 or os.environ.get("RBV_TEST_NVLS") != "1",
                    reason="needs 2 GPUs and RBV_TEST_NVLS=1 (binds memory to an NVLink multicast object)")
def test_nvls_metadata_two_processes():
    env = dict(os.environ, PYTHONPATH=ROOT, RBV_NVLS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29671", "-m", "rbruck_alltoallv_b200.utils.selftest"]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert '"selftest": "ok"' in res.stdout and '"nvls_metadata": true' in res.stdout


@pytest.mark.skipif(_ngpus() < 2 or os.environ.get("RBV_TEST_NVLS") != "1",
                    reason="needs 2 GPUs and RBV_TEST_NVLS=1 (binds memory to an NVLink multicast object)")
@pytest.mark.parametrize("module,args", [
    ("moe_bench", ["--tokens", "512", "--hidden", "512", "--inter", "1024", "--experts-per-rank", "4", "--check", "--steps", "3"]),
    ("fft_bench", ["--size", "48", "--pr", "1", "--pc", "2", "--check", "--steps", "2", "--warmup", "1"])])
def test_nvls_arrivals_of_the_auxiliary_barriers(module, args):
    """MoE dispatch / combine and the transpose report their arrival with one multimem.red when NVLS is on."""
    env = dict(os.environ, PYTHONPATH=ROOT, RBV_NVLS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29681", "-m", f"rbruck_alltoallv_b200.utils.{module}", *args]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert '"check": "ok"' in res.stdout


@pytest.mark.skipif(_ngpus() < 2, reason="needs 2 GPUs")
def test_a_process_that_does_not_join_is_a_timeout_and_the_communicator_recovers():
    """Failures are made on the host (a process skips a call, then announces a departure); no GPU is faulted.
    NVLS stays off: a process that fails while bound to a multicast object would disturb the other GPUs."""
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    env.pop("RBV_NVLS", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29691", "-m", "rbruck_alltoallv_b200.utils.fault_case"]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert '"fault_case": "ok"' in res.stdout
