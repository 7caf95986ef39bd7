"""Multi-GPU tests: run the torchrun scripts under tests/multi_gpu on 2 (and, when present, 4 / 8) GPUs."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import free_port

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script, nproc, extra_env=None, timeout=600):
    env = dict(os.environ)
    env.update({"MASTER_ADDR": "127.0.0.1", "NCCL_NVLS_ENABLE": env.get("NCCL_NVLS_ENABLE", "0")})
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "multi_gpu", script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    return r.returncode, r.stdout[-6000:] + r.stderr[-3000:]


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("n", [2, 4, 8])
def test_exchange_across_gpus(native_built, n):
    _need(n)
    rc, out = _torchrun("run_exchange.py", n)
    assert rc == 0, out


def test_exchange_scm_rights_transport(native_built):
    _need(2)
    rc, out = _torchrun("run_exchange.py", 2, {"HELIX_A2A_HANDLE_TRANSPORT": "scm"})
    assert rc == 0, out
