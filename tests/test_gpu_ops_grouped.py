"""The grouped prefill ops with the reference's argument lists (gridbook/ops.py:137-178,309-428):
the grouped bf16 GEMM over expert segments (allocating and in-place, a local expert slice), the
persistent-B decode-and-multiply ops (fp4 two-tier product, the literal format, fp8) and their
stand-alone decode stages, each against the oracle."""
import numpy as np
import pytest
import torch

from oracle import cb_oracle as O
from oracle import oracle_kwargs
from tests.helpers import assert_close_bf16, bits_of, f32_of

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    import gridbook_b200.ops  # noqa: F401  (registers the ops)
    _native.prepare(0)
    return torch.device("cuda:0")


def _sorted_rows(counts, K, seed):
    """Rows sorted by expert with the given per-expert counts -> (rows fp32 [P, K], ends int32 [E])."""
    from gridbook_b200 import synth
    P = int(np.sum(counts))
    return synth.make_activations(P, K, seed=seed), np.cumsum(counts).astype(np.int32)


def test_cb_bf16_grouped_mm_local_slice(dev):
    P_ = torch.ops.prismaquant
    E, N, K = 6, 256, 512
    counts = np.array([5, 0, 140, 33, 1, 60])
    a, ends = _sorted_rows(counts, K, seed=1)
    g = torch.Generator(device=dev).manual_seed(2)
    weights = torch.randn(E, N, K, generator=g, device=dev).to(torch.bfloat16)
    a_d, ends_d = torch.from_numpy(a).to(torch.bfloat16).to(dev), torch.from_numpy(ends).to(dev)
    ref = np.zeros((a.shape[0], N), np.float32)
    starts = np.concatenate([[0], ends])
    wf = weights.float().cpu().numpy()
    for e in range(E):
        ref[starts[e]:starts[e + 1]] = a[starts[e]:starts[e + 1]] @ wf[e].T
    out = P_.cb_bf16_grouped_mm(a_d, weights, ends_d, 0)
    assert_close_bf16(f32_of(out), O.bf16_round(ref), "grouped mm, whole stack")
    # a local slice of experts 2..4: the other experts' rows stay zero (allocating form) ...
    part = P_.cb_bf16_grouped_mm(a_d, weights[2:5].contiguous(), ends_d, 2)
    want = np.zeros_like(ref)
    want[starts[2]:starts[5]] = ref[starts[2]:starts[5]]
    assert_close_bf16(f32_of(part), O.bf16_round(want), "grouped mm, experts 2..4")
    # ... or untouched (in-place form)
    buf = torch.full((a.shape[0], N), 7.0, dtype=torch.bfloat16, device=dev)
    P_.cb_bf16_grouped_mm_out(buf, a_d, weights[2:5].contiguous(), ends_d, 2)
    got = f32_of(buf)
    assert np.all(got[:starts[2]] == 7.0) and np.all(got[starts[5]:] == 7.0)
    assert_close_bf16(got[starts[2]:starts[5]], O.bf16_round(ref[starts[2]:starts[5]]), "grouped mm out")


@pytest.mark.parametrize("name", ["k16v2", "lit"])
def test_cb_moe_persistent_b_prefill_fp4(dev, name):
    from gridbook_b200 import formats as F
    from gridbook_b200 import synth
    P_ = torch.ops.prismaquant
    fmt = {"k16v2": F.NVFP4_CB_K16, "lit": F.NVFP4_LITERAL}[name]
    E, N, K = 5, 256, 1024
    counts = np.array([40, 0, 7, 130, 16])
    a, ends = _sorted_rows(counts, K, seed=3)
    aq = O.fp4_group16_act_qdq(a, "recip")
    w13, _ = synth.make_moe(fmt, fmt, E, K, N // 2, seed=4)
    w = synth.to_device_weight(w13, dev)
    starts = np.concatenate([[0], ends])
    ref = np.zeros((a.shape[0], N), np.float32)
    for e in range(E):
        if counts[e]:
            ref[starts[e]:starts[e + 1]] = O.cb_linear(aq[starts[e]:starts[e + 1]], w13["qw"][e], w13["cb"],
                                                       np.zeros(N, np.int32), N=N, K=K, compose=w13["compose"],
                                                       **oracle_kwargs(fmt))
    a_d = torch.from_numpy(aq).to(torch.bfloat16).to(dev)
    ends_d = torch.from_numpy(ends).to(dev)
    if name == "lit":
        # the literal format is not one of the reference's (full mode, v1 bytes): through the method-level
        # entry of this package the same op body serves it
        from gridbook_b200 import ops
        out = torch.empty((a.shape[0], N), dtype=torch.bfloat16, device=dev)
        ops._persistent_b(out, a_d, w, ends_d)
        assert_close_bf16(f32_of(out), ref, "persistent-B literal")
        return
    compose = w.compose
    for op in (P_.cb_moe_persistent_b_prefill, P_.cb_moe_persistent_b_prefill_d2r):
        out = torch.zeros((a.shape[0], N), dtype=torch.bfloat16, device=dev)
        op(out, a_d, w.qw, w.codebook, compose, ends_d, fmt.k, fmt.type_size, 0)
        assert_close_bf16(f32_of(out), ref, f"persistent-B {name}")
    flat = w.qw.reshape(E * N, -1)
    tile = P_.cb_moe_persistent_b_decode(flat, w.codebook, compose, N + 8, 100, K, fmt.k, fmt.type_size)
    want = O.reconstruct_weight(w13["qw"][1], w13["cb"], np.zeros(N, np.int32), N=N, K=K, compose=w13["compose"],
                                **oracle_kwargs(fmt))[8:108]
    assert np.array_equal(bits_of(tile), O.f32_to_bf16_bits(want))


def test_cb_moe_persistent_b_prefill_fp8(dev):
    from gridbook_b200 import formats as F
    from gridbook_b200 import synth
    P_ = torch.ops.prismaquant
    fmt = F.FP8_CB_K32
    E, N, K = 4, 256, 768
    counts = np.array([3, 150, 0, 21])
    a, ends = _sorted_rows(counts, K, seed=5)
    aq = O.fp8_dynamic_act_qdq(a, "recip")
    w13, _ = synth.make_moe(fmt, fmt, E, K, N // 2, seed=6)
    w = synth.to_device_weight(w13, dev)
    lut_f32 = torch.from_numpy(w13["cb"]).to(dev)
    scale = torch.from_numpy(w13["scale"]).to(dev)
    starts = np.concatenate([[0], ends])
    ref = np.zeros((a.shape[0], N), np.float32)
    for e in range(E):
        if counts[e]:
            ref[starts[e]:starts[e + 1]] = O.cb_linear(aq[starts[e]:starts[e + 1]], w13["qw"][e], w13["cb"],
                                                       np.zeros(N, np.int32), N=N, K=K, weight_scale=w13["scale"][e],
                                                       **oracle_kwargs(fmt))
    out = torch.zeros((a.shape[0], N), dtype=torch.bfloat16, device=dev)
    P_.cb_moe_persistent_b_prefill_fp8(out, torch.from_numpy(aq).to(torch.bfloat16).to(dev), w.qw, lut_f32, scale,
                                       torch.from_numpy(ends).to(dev), fmt.k, fmt.type_size, 0)
    assert_close_bf16(f32_of(out), ref, "persistent-B fp8")
    tile = P_.cb_moe_persistent_b_decode_fp8(w.qw.reshape(E * N, -1), lut_f32, scale.reshape(-1), 2 * N + 5, 64, K,
                                             fmt.k, fmt.type_size)
    want = O.reconstruct_weight(w13["qw"][2], w13["cb"], np.zeros(N, np.int32), N=N, K=K,
                                weight_scale=w13["scale"][2], **oracle_kwargs(fmt))[5:69]
    assert np.array_equal(bits_of(tile), O.f32_to_bf16_bits(want))
