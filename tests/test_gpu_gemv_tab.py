"""The one-launch table GEMV (gb_gemv_tab) through the C ABI: one activation row against one
matrix or against several matrices that share the row, checked against the oracle; ragged
last K slices, ragged row counts, row counts that leave CTAs of a band without rows, several
calls in a row on one armed slot buffer, and the canary of a buffer that was never armed."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import oracle_kwargs
from tests.helpers import assert_close_bf16, f32_of, oracle_linear

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


def _literal():
    from gridbook_b200.formats import CBFormat
    return CBFormat("fp4", 8, mode="full", scale_coding="v1")


def _c_linear(x, d):
    fmt = d["fmt"]
    xq = C.act_qdq(x, fmt.grid, "recip")
    return C.linear(xq, d["qw"], d["cb"], None, N=d["N"], K=d["K"], compose=None, weight_scale=None,
                    global_scale=d.get("global_scale"), **oracle_kwargs(fmt))


@pytest.mark.parametrize("N,K", [(64, 256), (200, 1024), (264, 1280), (1000, 2816), (6144, 5120), (5120, 6144),
                                 (2048, 5120), (5120, 17408), (34816, 5120), (4096, 4096),
                                 # the shards of the same five projections over four and eight ranks
                                 (1536, 5120), (512, 5120), (1280, 6144), (8704, 5120), (1280, 17408),
                                 (768, 5120), (256, 5120), (640, 6144), (4352, 5120), (640, 17408)])
def test_one_matrix_against_oracle(dev, request, N, K):
    from gridbook_b200 import _native, kernels, synth
    _native.set_wait_limit_ms(200)           # a wait that cannot end shows as a status, not as minutes
    request.addfinalizer(lambda: _native.set_wait_limit_ms(0))
    fmt = _literal()
    d = synth.make_linear(fmt, N, K, seed=N + K, global_scale=1.0 / 448.0)
    x = synth.make_activations(1, K, seed=K)
    ref = _c_linear(x, d) if N * K > (1 << 22) else oracle_linear(x, d)
    w = synth.to_device_weight(d, dev)
    slots = kernels.new_tab_slots([w])
    xd = synth.bf16_tensor(x, dev)
    for call in range(2):                    # the second call meets the slots the first one re-armed
        (y,) = kernels.gemv_tab(xd, [w], slots)
        torch.cuda.synchronize()
        assert _native.device_status(0) == 0
        assert_close_bf16(f32_of(y), ref, f"{N}x{K} call {call}")
    assert bool((slots == 0xFF).all()), "the slot buffer must be left armed"


def test_matrices_that_share_a_row(dev):
    """q (6144), kv (2048) and a third small matrix with their own codebooks in one launch; the
    result equals the one-matrix launches bit for bit (same slices, same order of additions)."""
    from gridbook_b200 import _native, kernels, synth
    fmt = _literal()
    K = 5120
    ds = [synth.make_linear(fmt, n, K, seed=7 + i, global_scale=g) for i, (n, g) in
          enumerate(((6144, 1.0 / 448.0), (2048, 1.0 / 448.0), (192, 0.5)))]
    ws = [synth.to_device_weight(d, dev) for d in ds]
    x = synth.make_activations(1, K, seed=3)
    xd = synth.bf16_tensor(x, dev)
    slots = kernels.new_tab_slots(ws)
    outs = kernels.gemv_tab(xd, ws, slots)
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    for d, w, y in zip(ds, ws, outs):
        assert_close_bf16(f32_of(y), _c_linear(x, d), f"shared row N={d['N']}")
        (alone,) = kernels.gemv_tab(xd, [w], slots)
        assert torch.equal(alone, y)
    assert bool((slots == 0xFF).all())


def test_same_bits_as_the_two_launch_kernel_and_from_run_to_run(dev):
    from gridbook_b200 import kernels, synth
    fmt = _literal()
    d = synth.make_linear(fmt, 34816, 5120, seed=11, global_scale=1.0 / 448.0)
    w = synth.to_device_weight(d, dev)
    slots = kernels.new_tab_slots([w])
    x = synth.bf16_tensor(synth.make_activations(1, 5120, seed=4), dev)
    (y0,) = kernels.gemv_tab(x, [w], slots)
    for _ in range(5):
        (y1,) = kernels.gemv_tab(x, [w], slots)
        assert torch.equal(y0, y1)
    # no bucket: scaling the row by a power of two scales every partial sum exactly
    (a,) = kernels.gemv_tab(x, [w], slots, act=None)
    (b,) = kernels.gemv_tab((x.float() * 4.0).to(torch.bfloat16), [w], slots, act=None)
    assert torch.equal(b.float(), a.float() * 4.0)
    two = kernels.gemv(x, w, act="fp4")
    assert_close_bf16(f32_of(y0), f32_of(two), "one launch vs two launches")


def test_unarmed_buffer_raises_the_status_word(dev):
    from gridbook_b200 import _native, kernels, synth
    fmt = _literal()
    d = synth.make_linear(fmt, 256, 1024, seed=1)
    w = synth.to_device_weight(d, dev)
    slots = torch.zeros(kernels.new_tab_slots([w]).numel(), dtype=torch.uint8, device=dev)
    x = synth.bf16_tensor(synth.make_activations(1, 1024, seed=1), dev)
    kernels.gemv_tab(x, [w], slots)
    torch.cuda.synchronize()
    assert _native.device_status(0) == 24
    _native.device_status_reset(0)
    assert _native.device_status(0) == 0


def test_other_formats_are_declined(dev):
    from gridbook_b200 import kernels, synth
    from gridbook_b200.formats import NVFP4_CB_K16
    d = synth.make_linear(NVFP4_CB_K16, 256, 1024, seed=1)
    w = synth.to_device_weight(d, dev)
    lit = synth.to_device_weight(synth.make_linear(_literal(), 256, 1024, seed=1), dev)
    slots = kernels.new_tab_slots([lit])
    x = synth.bf16_tensor(synth.make_activations(1, 1024, seed=1), dev)
    assert kernels.gemv_tab(x, [w], slots) is None
