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


def test_a_wait_that_runs_out_raises_the_status_word_and_leaves_the_gpu_usable():
    """One GPU, a group of two ranks whose second flag block is a local buffer that nobody ever
    writes: the barrier's wait for rank 1 runs into its limit (shortened to 50 ms for the test),
    the kernel returns, the status word reads 3, and after a reset the library works as before."""
    import ctypes

    from gridbook_b200 import _native as nat
    from gridbook_b200 import kernels, synth
    from gridbook_b200.formats import NVFP4_LITERAL

    nat.prepare(0)
    lib = nat.load()
    dev = torch.device("cuda:0")
    assert nat.device_status(0) == 0
    mine, absent = ctypes.c_void_p(), ctypes.c_void_p()
    nat.check(lib.gb_peer_alloc(nat.PEER_FLAG_BYTES, ctypes.byref(mine)), lib)
    nat.check(lib.gb_peer_alloc(nat.PEER_FLAG_BYTES, ctypes.byref(absent)), lib)
    group = nat.GbPeerGroup(rank=0, world=2)
    group.flags[0], group.flags[1] = mine.value, absent.value
    nat.set_wait_limit_ms(50)
    try:
        nat.check(lib.gb_peer_barrier(ctypes.byref(group), ctypes.c_void_p(nat.stream_ptr(dev))), lib)
        torch.cuda.synchronize()                      # returns: the wait gave up, nothing hangs
        assert nat.device_status(0) == 3
    finally:
        nat.set_wait_limit_ms(0)
        nat.device_status_reset(0)
        lib.gb_peer_free(mine)
        lib.gb_peer_free(absent)
    assert nat.device_status(0) == 0
    d = synth.make_linear(NVFP4_LITERAL, 256, 1024, seed=0, global_scale=1.0 / 448.0)
    w = synth.to_device_weight(d, dev)
    x = synth.bf16_tensor(synth.make_activations(1, 1024, seed=0), dev)
    y = kernels.gemv(x, w, act="fp4")                 # a healthy call afterwards
    torch.cuda.synchronize()
    assert nat.device_status(0) == 0 and bool(torch.isfinite(y.float()).all())
