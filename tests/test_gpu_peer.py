"""Peer-memory exchange (all-gather of column shards, expert-parallel routed layer) on two
GPUs of one box: the rank program runs as child processes, one per GPU."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_peer_paths_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "peer_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert done.returncode == 0, done.stdout[-4000:] + done.stderr[-4000:]
    assert "rank 0: peer paths ok" in done.stdout and "rank 1: peer paths ok" in done.stdout
