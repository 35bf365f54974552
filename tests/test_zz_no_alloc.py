"""The allocation-free entry point gb_gemv_static, called through the C ABI.

Some callers of this library cannot allocate device memory: an engine that handed all of
it to its own pools at start-up, or a binding with no argument for a scratch buffer.  For
them the library carries a fixed scratch array; this test checks that the entry point
using it returns what gb_gemv returns with a caller-owned workspace, twice in a row (the
second call meets the first call's leftovers), for a launch that needs no partial sums and
for a K-sliced one that does, and that an oversized shape is refused.

The file name sorts last on purpose: a run that stops at the first failure has then
already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from tests.helpers import assert_close_bf16, f32_of

pytestmark = pytest.mark.gpu


def _static_gemv(x, w, act):
    from gridbook_b200 import _native as nat
    lib = nat.load()
    x2 = x.reshape(-1, w.K).contiguous()
    y = torch.empty((x2.shape[0], w.rows), dtype=torch.bfloat16, device=x.device)
    nw = w.native()
    rc = lib.gb_gemv_static(ctypes.c_void_p(x2.data_ptr()), x2.shape[0], ctypes.byref(nw),
                            {"fp4": nat.ACT_FP4_GROUP16, "fp8": nat.ACT_FP8_TOKEN}[act], nat.SCALE_RULE_RECIP,
                            ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(nat.stream_ptr(x.device)))
    return rc, y, lib


@pytest.mark.parametrize("name,M,N,K", [("lit", 3, 200, 1024), ("k16v2", 16, 264, 6144), ("f8k32", 9, 136, 7168),
                                        ("lit", 1, 512, 2048), ("lit", 3, 384, 1280)])
def test_static_scratch_matches_workspace_entry(name, M, N, K):
    from gridbook_b200 import _native, kernels, synth
    from gridbook_b200.formats import CBFormat
    _native.prepare(0)
    dev = torch.device("cuda:0")
    fmt = {"lit": CBFormat("fp4", 8, mode="full", scale_coding="v1"),
           "k16v2": CBFormat("fp4", 16, n_sub=2, scale_coding="v2"),
           "f8k32": CBFormat("fp8", 32, n_sub=4)}[name]
    d = synth.make_linear(fmt, N, K, seed=21)
    w = synth.to_device_weight(d, dev)
    for call in range(2):                       # two calls in a row share the built-in array
        x = synth.bf16_tensor(synth.make_activations(M, K, seed=100 + call), dev)
        ref = kernels.gemv(x, w, act=fmt.grid)
        rc, got, lib = _static_gemv(x, w, fmt.grid)
        assert rc == 0, lib.gb_last_error().decode()
        torch.cuda.synchronize()
        assert_close_bf16(f32_of(got), f32_of(ref), f"{name} call {call}")
    assert _native.device_status(0) == 0


def test_static_scratch_table_kernels_after_a_larger_call_against_the_oracle():
    """The literal format's table kernels (one row; a few rows, one table GEMV per row) write
    every (K slice, row) slot they later add and never clear the array.  A larger call first
    leaves its partial sums behind; the smaller calls that follow must not pick them up.
    Checked against the oracle, not only against gb_gemv."""
    from gridbook_b200 import _native, synth
    from gridbook_b200.formats import CBFormat
    from tests.helpers import oracle_linear
    _native.prepare(0)
    dev = torch.device("cuda:0")
    fmt = CBFormat("fp4", 8, mode="full", scale_coding="v1")
    for M, N, K in ((4, 1024, 4096), (1, 512, 2048), (3, 256, 1024), (1, 320, 1280)):
        d = synth.make_linear(fmt, N, K, seed=N + K + M, global_scale=1.0 / 448.0)
        w = synth.to_device_weight(d, dev)
        xh = synth.make_activations(M, K, seed=M + N)
        rc, got, lib = _static_gemv(synth.bf16_tensor(xh, dev), w, "fp4")
        assert rc == 0, lib.gb_last_error().decode()
        torch.cuda.synchronize()
        assert_close_bf16(f32_of(got), oracle_linear(xh, d), f"static literal M={M} {N}x{K}")
    assert _native.device_status(0) == 0


def test_static_scratch_refuses_oversized_shapes():
    from gridbook_b200 import _native, synth
    from gridbook_b200.formats import CBFormat
    _native.prepare(0)
    dev = torch.device("cuda:0")
    fmt = CBFormat("fp8", 32, n_sub=4)
    N, K = 70000, 256                           # 16 x 70000 fp32 partial sums > 4 MiB
    d = synth.make_linear(fmt, N, K, seed=1)
    w = synth.to_device_weight(d, dev)
    x = torch.zeros(16, K, dtype=torch.bfloat16, device=dev)
    rc, _, lib = _static_gemv(x, w, "fp8")
    assert rc != 0
    msg = lib.gb_last_error().decode()
    assert "scratch" in msg and "gb_gemv" in msg
