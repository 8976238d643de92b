"""Tensor-parallel runs of the path on 2+ GPUs of one node (skipped with fewer).

Each case launches `tests/mp_worker.py` under torchrun, one process per GPU, and passes
when every rank exits 0.  The all-reduce is issued by the kernels themselves (NVLS
multimem when the GPUs expose multicast, plain peer loads otherwise); NCCL only
bootstraps the group and serves as an untimed cross-check.  The failure case injects its
fault on the host (a rank that does not launch), with NVLS off everywhere, and no rank
leaves before the end."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "mp_worker.py")


def _gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(nproc, *args, env=None, timeout=600):
    port = 29500 + (os.getpid() % 400)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           WORKER, *args]
    full_env = dict(os.environ)
    full_env.update(env or {})
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=full_env)
    sys.stdout.write(proc.stdout[-4000:])
    if proc.returncode != 0:
        sys.stdout.write("---- worker stderr ----\n" + proc.stderr[-8000:])
    return proc.returncode


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_layer_parity_tensor_parallel(nproc):
    if _gpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    assert _run(nproc, "--mode", "parity") == 0


def test_layer_parity_without_multicast():
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    assert _run(2, "--mode", "parity", "--no-multicast") == 0


def test_absent_peer_times_out_and_recovers():
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    assert _run(2, "--mode", "timeout", env={"NCCL_NVLS_ENABLE": "0"}) == 0
