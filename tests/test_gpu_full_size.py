"""GPU parity at the full sizes of the benchmark configurations: the dense linears of
configurations 0 and 1 against the C restatement of the oracle (OpenMP, seconds per case), a
size-independent property (scaling the activations by a power of two scales the output
exactly), the routed layer of configuration 3 against the loop-chain oracle, and a prefill GEMM
with several output tiles per persistent CTA."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import oracle_kwargs
from oracle import cb_oracle as O
from tests.helpers import assert_close_bf16, f32_of

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


def _literal():
    from gridbook_b200.formats import CBFormat
    return CBFormat("fp4", 8, mode="full", scale_coding="v1")


def _c_linear(x, d, scale_rule="recip"):
    fmt = d["fmt"]
    xq = C.act_qdq(x, fmt.grid, scale_rule)
    return C.linear(xq, d["qw"], d["cb"], None, N=d["N"], K=d["K"], compose=d.get("compose"),
                    weight_scale=d.get("weight_scale"), global_scale=d.get("global_scale"), **oracle_kwargs(fmt))


@pytest.mark.parametrize("N,K,M", [(4096, 4096, 1),            # configuration 0
                                   (34816, 5120, 1), (34816, 5120, 4), (34816, 5120, 16),   # gate_up
                                   (5120, 17408, 1), (5120, 17408, 4),                      # down
                                   (2048, 5120, 2)])                                        # kv
def test_dense_linear_full_size_against_c_oracle(dev, N, K, M):
    from gridbook_b200 import _native, kernels, synth
    fmt = _literal()
    d = synth.make_linear(fmt, N, K, seed=N + K + M, global_scale=1.0 / 448.0)
    x = synth.make_activations(M, K, seed=M)
    ref = _c_linear(x, d)
    w = synth.to_device_weight(d, dev)
    y = kernels.gemv(synth.bf16_tensor(x, dev), w, act="fp4")
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    assert_close_bf16(f32_of(y), ref, f"{N}x{K} M={M}")


def test_scaling_activations_by_a_power_of_two_scales_the_output_exactly(dev):
    """No bucket: y(4 x) == 4 y(x) bit for bit (every product and partial sum scales exactly),
    on the largest projection, for the one-row table kernel and the expanding kernel."""
    from gridbook_b200 import kernels, synth
    d = synth.make_linear(_literal(), 34816, 5120, seed=5, global_scale=1.0 / 448.0)
    w = synth.to_device_weight(d, dev)
    for M in (1, 3, 9):
        x = synth.bf16_tensor(synth.make_activations(M, 5120, seed=M), dev)
        y1 = kernels.gemv(x, w).float()
        y4 = kernels.gemv((x.float() * 4.0).to(torch.bfloat16), w).float()
        assert torch.equal(y4, y1 * 4.0), M


def test_routed_layer_full_size_against_loop_chain(dev):
    """Configuration 3 (128 experts, top-8, 2048 -> 2 x 768 -> 2048) at 16 tokens through the layer
    method (per-pair table kernels) and through the grouped kernels, against the oracle."""
    from gridbook_b200 import kernels, synth
    from gridbook_b200.moe import CBMoE
    fmt = _literal()
    E, topk, hidden, inter, T = 128, 8, 2048, 768, 16
    w13d, w2d = synth.make_moe(fmt, fmt, E, hidden, inter, seed=2)
    ids, tw = synth.make_routing(T, E, topk, seed=2)
    x = synth.make_activations(T, hidden, seed=2)
    ref = O.moe_loop_chain(x, ids, tw, w13d, w2d, E=E, hidden=hidden, inter=inter, fmt13=oracle_kwargs(fmt),
                           fmt2=oracle_kwargs(fmt), scale_rule="recip")
    w13, w2 = synth.to_device_weight(w13d, dev), synth.to_device_weight(w2d, dev)
    xd, idd = synth.bf16_tensor(x, dev), torch.from_numpy(ids).to(dev)
    twd = torch.from_numpy(tw).to(dev)
    x_row = (torch.arange(T * topk, device=dev, dtype=torch.int32) // topk).contiguous()
    # per-pair path
    a = kernels.moe_gemv_pairs(xd, w13, idd, x_row=x_row, swiglu=True, act="fp4")
    y = kernels.moe_gemv_pairs(a, w2, idd, act="fp4")
    out_pairs = f32_of(kernels.moe_combine(y, twd, T, topk, topk_ids=idd, E=E, round_weights=True))
    # grouped path
    _, offsets, order, pw = kernels.moe_route(idd, E, twd)
    a2 = kernels.moe_gemv(kernels.fp4_act_qdq(xd), w13, offsets, order, x_row=x_row, swiglu=True)
    y2 = kernels.moe_gemv(kernels.fp4_act_qdq(a2), w2, offsets, order)
    out_grouped = f32_of(kernels.moe_combine(y2, pw, T, topk))
    for tag, got in (("per-pair", out_pairs), ("grouped", out_grouped)):
        rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert rel <= 1e-2, (tag, rel)
        assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max(), tag


def test_gemm_many_tiles_per_cta(dev):
    """512 output tiles over 148 persistent CTAs: both accumulator buffers are reused."""
    from gridbook_b200 import _native, kernels
    M, N, K = 1024, 16384, 1024
    g = torch.Generator(device=dev).manual_seed(3)
    a = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, generator=g, device=dev).to(torch.bfloat16)
    d = kernels.gemm_tn(a, b)
    ref = a.float() @ b.float().t()
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    err = (d.float() - ref).abs()
    assert bool((err <= ref.abs() * 2.0 ** -7 + 1e-2).all()), float(err.max())
    a8, b8 = a.to(torch.float8_e4m3fn), b.to(torch.float8_e4m3fn)
    d8 = kernels.gemm_tn(a8, b8)
    ref8 = a8.float() @ b8.float().t()
    err8 = (d8.float() - ref8).abs()
    assert bool((err8 <= ref8.abs() * 2.0 ** -7 + 1e-2).all()), float(err8.max())
