"""Tensor-parallel MLP on real GPUs (needs at least two): sharded result vs the one-GPU result, max relative error
1e-2 (the partials are rounded to BF16 and summed in a different order)."""

import pathlib
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parent.parent


def test_tensor_parallel_mlp_matches_one_gpu():
    count = torch.cuda.device_count()
    if count < 2:
        pytest.skip("needs two GPUs")
    world = 2 if count < 4 else 4 if count < 8 else 8
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "tp_check.py")]
    done = subprocess.run(command, capture_output=True, text=True, timeout=600,
                          env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert done.returncode == 0 and "TP_CHECK_OK" in done.stdout, done.stdout[-2000:] + done.stderr[-4000:]
