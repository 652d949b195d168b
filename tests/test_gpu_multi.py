"""Spawns tests/dist_worker.py under torchrun on 1, 2, 4 and 8 GPUs (as many as are visible):
the drop-in Manager over cudaIpc-mapped peer memory, checked against the CPU oracle."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("nproc", [1, 2, 4, 8])
def test_manager_end_to_end(native_lib, nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs, {torch.cuda.device_count()} visible")
    from ultra_ep_b200 import build

    build.build_ext()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
         "127.0.0.1", "--master-port", str(29700 + nproc), os.path.join(ROOT, "tests", "dist_worker.py")],
        env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + "\n" + res.stderr[-6000:]
    assert "all checks passed" in res.stdout
