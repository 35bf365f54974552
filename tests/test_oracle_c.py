"""The C restatement of the oracle against the reference-generated fixtures and against
the numpy restatement on synthetic layers (CPU only)."""
import numpy as np
import pytest

from gridbook_b200 import synth
from gridbook_b200.formats import CBFormat
from oracle import c_oracle as C
from oracle import oracle_kwargs
from oracle import cb_oracle as O


def f32(bits):
    return O.bf16_bits_to_f32(bits)


@pytest.mark.parametrize("k", [12, 13, 16, 20])
def test_c_fp4_v2_fixture(golden, k):
    p = f"fp4v2_k{k}_"
    kw = dict(N=6, K=512, k_bits=k, n_sub=2, type_size=4 * k + 9, grid="fp4", scale_coding="v2",
              compose=golden["compose"])
    w = C.reconstruct(golden[p + "qw"], f32(golden[p + "cb"]), golden[p + "off"], **kw)
    assert np.array_equal(O.f32_to_bf16_bits(w), golden[p + "w"])
    xq = C.act_qdq(f32(golden[p + "x"]), "fp4", "div")
    assert np.array_equal(O.f32_to_bf16_bits(xq), golden[p + "xq"])
    y = C.linear(xq, golden[p + "qw"], f32(golden[p + "cb"]), golden[p + "off"], **kw)
    ref = f32(golden[p + "y"])
    assert np.all(np.abs(y - ref) <= np.maximum(np.abs(y), np.abs(ref)) * 2.0 ** -7 + 1e-5)


@pytest.mark.parametrize("k,n_sub", [(28, 4), (30, 4), (32, 4), (37, 4), (16, 2)])
def test_c_fp8_fixture(golden, k, n_sub):
    p = f"fp8_k{k}_n{n_sub}_"
    kw = dict(N=5, K=512, k_bits=k, n_sub=n_sub, type_size=4 * k, grid="fp8", weight_scale=golden[p + "ws"])
    w = C.reconstruct(golden[p + "qw"], f32(golden[p + "cb"]), None, **kw)
    assert np.array_equal(O.f32_to_bf16_bits(w), golden[p + "w"])
    xq = C.act_qdq(f32(golden[p + "x"]), "fp8", "div")
    assert np.array_equal(O.f32_to_bf16_bits(xq), golden[p + "xq"])


def test_c_activation_fixture(golden):
    x = f32(golden["act_x"])
    assert np.array_equal(O.f32_to_bf16_bits(C.act_qdq(x, "fp4", "div")), golden["act_fp4"])
    assert np.array_equal(O.f32_to_bf16_bits(C.act_qdq(x, "fp8", "div")), golden["act_fp8"])
    for rule in ("recip", "div"):
        assert np.array_equal(C.act_qdq(x, "fp4", rule), O.fp4_group16_act_qdq(x, rule))
        assert np.array_equal(C.act_qdq(x, "fp8", rule), O.fp8_dynamic_act_qdq(x, rule))


@pytest.mark.parametrize("fmt", [
    CBFormat("fp4", 8, mode="full", scale_coding="v1"), CBFormat("fp4", 16, n_sub=2, scale_coding="v2"),
    CBFormat("fp4", 13, mode="signed", scale_coding="v1"), CBFormat("fp8", 32, n_sub=4),
    CBFormat("fp8", 16, n_sub=2), CBFormat("fp8", 45, n_sub=4)], ids=str)
def test_c_matches_numpy_on_synthetic(fmt):
    N, K = 50, 768
    d = synth.make_linear(fmt, N, K, seed=3, n_books=2, super_span=None)
    kw = dict(N=N, K=K, compose=d["compose"], weight_scale=d["weight_scale"], **oracle_kwargs(fmt))
    wn = O.reconstruct_weight(d["qw"], d["cb"], d["cb_row_offset"], **kw)
    wc = C.reconstruct(d["qw"], d["cb"], d["cb_row_offset"], **kw)
    assert np.array_equal(wn.view(np.uint32), wc.view(np.uint32))
    x = synth.make_activations(3, K, seed=1)
    yn = O.cb_linear(x, d["qw"], d["cb"], d["cb_row_offset"], global_scale=0.5, **kw)
    yc = C.linear(x, d["qw"], d["cb"], d["cb_row_offset"], global_scale=0.5, **kw)
    assert np.all(np.abs(yn - yc) <= np.maximum(np.abs(yn), np.abs(yc)) * 2.0 ** -7 + 1e-5)
