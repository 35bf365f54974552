"""GPU parity of the routed prefill route: the grouped tensor-core GEMM over expert segments
(tcgen05, segment offsets read on the device), the row gather and SwiGLU kernels around it, and
the whole routed layer through the method class against the per-expert loop chain of the oracle.
The floating-point reference of the GEMM alone is a plain fp32 matmul in torch."""
import numpy as np
import pytest
import torch

from oracle import cb_oracle as O
from oracle import oracle_kwargs
from tests.helpers import f32_of

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


def _segments(counts, dev):
    off = np.zeros(len(counts) + 1, dtype=np.int32)
    off[1:] = np.cumsum(counts)
    return torch.from_numpy(off).to(dev)


@pytest.mark.parametrize("counts,N,K,extra", [
    ([5, 0, 130, 128, 1, 0, 257, 0], 256, 512, 0),       # empty experts, tile edges, ragged tails
    ([300, 17], 136, 256, 9),                             # N not a tile multiple; rows past the last segment
    ([0, 0, 0, 40], 512, 1024, 0),                        # leading empty experts
    ([64] * 40, 384, 2048, 3),                            # more experts than one scan pass
])
def test_grouped_gemm_bf16_matches_fp32_matmul(dev, counts, N, K, extra):
    from gridbook_b200 import _native, kernels
    E, routed = len(counts), int(sum(counts))
    P = routed + extra
    g = torch.Generator(device=dev).manual_seed(P + N)
    a = torch.randn(P, K, generator=g, device=dev).to(torch.bfloat16)
    b = torch.randn(E * N, K, generator=g, device=dev).to(torch.bfloat16)
    off = _segments(counts, dev)
    sentinel = 77.0
    out = torch.full((P, N), sentinel, dtype=torch.bfloat16, device=dev)
    kernels.gemm_tn_grouped(a, b, off, N, global_scale=0.25, out=out)
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    ref = torch.full((P, N), sentinel, dtype=torch.float32, device=dev)
    r0 = 0
    for e, c in enumerate(counts):
        ref[r0:r0 + c] = (a[r0:r0 + c].float() @ b[e * N:(e + 1) * N].float().t()) * 0.25
        r0 += c
    err = (out.float() - ref).abs()
    assert bool((err <= ref.abs() * 2.0 ** -7 + 1e-2).all()), float(err.max())
    assert bool((out[routed:].float() == sentinel).all())           # rows past the segments untouched

    # the same through a row map: the result lands at row_map[j]
    perm = torch.randperm(P, generator=torch.Generator().manual_seed(1)).to(torch.int32).to(dev)
    out2 = torch.full((P, N), sentinel, dtype=torch.bfloat16, device=dev)
    kernels.gemm_tn_grouped(a, b, off, N, row_map=perm, global_scale=0.25, out=out2)
    assert torch.equal(out2[perm[:routed].long()], out[:routed])


def test_grouped_gemm_e4m3_with_scales(dev):
    from gridbook_b200 import kernels
    counts, N, K = [150, 0, 70, 129], 264, 512
    E, P = len(counts), int(sum(counts))
    g = torch.Generator(device=dev).manual_seed(3)
    a = (torch.randn(P, K, generator=g, device=dev) * 4).to(torch.float8_e4m3fn)
    b = (torch.randn(E * N, K, generator=g, device=dev) * 4).to(torch.float8_e4m3fn)
    sa = torch.rand(P, generator=g, device=dev) + 0.5
    sb = (torch.rand(E * N, generator=g, device=dev) + 0.5) * 0.02
    out = kernels.gemm_tn_grouped(a, b, _segments(counts, dev), N, a_scale=sa, b_scale=sb)
    r0 = 0
    for e, c in enumerate(counts):
        ref = (a[r0:r0 + c].float() @ b[e * N:(e + 1) * N].float().t()) * sa[r0:r0 + c, None] * sb[None, e * N:(e + 1) * N]
        got = out[r0:r0 + c].float()
        assert float((got - ref).norm() / ref.norm().clamp_min(1e-9)) <= 3e-3, e
        r0 += c


def test_gather_and_swiglu_rows(dev):
    from gridbook_b200 import kernels, synth
    T, topk, E, K, inter = 37, 3, 8, 512, 256
    ids, _ = synth.make_routing(T, E, topk, seed=4)
    ids[5, 1] = -1
    idd = torch.from_numpy(ids).to(dev)
    _, offsets, order = kernels.moe_route(idd, E)
    routed = int(offsets[-1])
    assert routed == T * topk - 1
    x = synth.bf16_tensor(synth.make_activations(T, K, seed=1), dev)
    x_row = (torch.arange(T * topk, device=dev, dtype=torch.int32) // topk).contiguous()
    got = kernels.moe_gather_rows(x, order, offsets, x_row=x_row)
    assert torch.equal(got[:routed], x[(order[:routed] // topk).long()])

    h = synth.make_activations(T * topk, 2 * inter, seed=2) * 3.0
    a = kernels.moe_swiglu_rows(synth.bf16_tensor(h, dev), offsets)
    ref = O.silu_mul(O.bf16_round(h))
    got = f32_of(a[:routed])
    # the device exponential differs from libm's in the last place: a bf16 step at most, rarely
    assert np.abs(got - ref[:routed]).max() <= np.abs(ref).max() * 2.0 ** -7
    assert np.mean(got != ref[:routed]) < 0.02
    # with the fused bucket: the same bits as the bucket kernel on the plain result
    fused = kernels.moe_swiglu_rows(synth.bf16_tensor(h, dev), offsets, act="fp4")
    assert torch.equal(fused[:routed], kernels.fp4_act_qdq(a)[:routed])


@pytest.mark.parametrize("f13,f2,T", [("lit", "lit", 300), ("k16v2", "k16v2", 150), ("f8k32", "f8k32", 130),
                                      ("f8lit", "lit", 90)])
def test_moe_method_prefill_route_matches_loop_chain(dev, monkeypatch, f13, f2, T):
    """The routed layer on the grouped-GEMM route (forced on for this small shape) against the
    per-expert loop chain, with a padded (-1) slot and an expert nobody routes to."""
    from gridbook_b200 import synth
    from gridbook_b200.moe import CBMoE
    from tests.test_gpu_plugin import _formats, _tables
    fmt13, fmt2 = _formats()[f13], _formats()[f2]
    E, hidden, inter, topk = 8, 512, 256, 2
    w13d, w2d = synth.make_moe(fmt13, fmt2, E, hidden, inter, seed=T)
    ids, tw = synth.make_routing(T, E - 1, topk, seed=T)          # expert E-1 stays empty
    x = synth.make_activations(T, hidden, seed=T + 1)
    ids[2, 1] = -1
    ids_ref = np.where(ids < 0, 0, ids)
    tw_ref = np.where(ids < 0, 0.0, tw).astype(np.float32)
    ref = O.moe_loop_chain(x, ids_ref, tw_ref, w13d, w2d, E=E, hidden=hidden, inter=inter,
                           fmt13=oracle_kwargs(fmt13), fmt2=oracle_kwargs(fmt2), scale_rule="recip")
    moe = CBMoE(fmt13, fmt2, E, hidden, inter, _tables(fmt13, w13d["cb"]), _tables(fmt2, w2d["cb"]))
    moe.load(torch.from_numpy(w13d["qw"]), torch.from_numpy(w2d["qw"]),
             None if w13d["scale"] is None else torch.from_numpy(w13d["scale"]),
             None if w2d["scale"] is None else torch.from_numpy(w2d["scale"]), dev)
    moe.method.prefill_min_pairs_per_expert = 1            # the route's threshold is an attribute of the method
    got = f32_of(moe(synth.bf16_tensor(x, dev), torch.from_numpy(tw).to(dev), torch.from_numpy(ids).to(dev)))
    assert "grouped prefill" in moe._cb_route
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-2, rel                                         # acceptance bar of the path
    assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("f13,f2,T", [("lit", "lit", 40), ("lit", "lit", 150), ("lit", "lit", 700),
                                      ("k16v2", "k16v2", 150), ("f8k32", "f8k32", 150), ("f8lit", "lit", 150),
                                      ("f8lit", "lit", 3), ("lit", "f8k32", 300)])
def test_moe_method_sorted_rows_route_matches_loop_chain(dev, monkeypatch, f13, f2, T):
    """The routed layer on the sorted-rows route (decode into tensor memory + tcgen05 per expert
    tile), forced on for this small shape: experts with no rows, with a few, and with more than one
    64-row pass; a padded (-1) slot; every format the kernel decodes, also two grids in one layer
    (each projection's rows through its own grid's bucket) and two-tier stacks, which the method
    keeps in 80-byte superblock slots."""
    from gridbook_b200 import _native, synth
    from gridbook_b200.moe import CBMoE
    from tests.test_gpu_plugin import _formats, _tables
    fmt, fmt_2 = _formats()[f13], _formats()[f2]
    E, hidden, inter, topk = 8, 1024, 512, 2
    w13d, w2d = synth.make_moe(fmt, fmt_2, E, hidden, inter, seed=T)
    ids, tw = synth.make_routing(T, E - 1, topk, seed=T)          # expert E-1 stays empty
    x = synth.make_activations(T, hidden, seed=T + 1)
    ids[2, 1] = -1
    ids_ref = np.where(ids < 0, 0, ids)
    tw_ref = np.where(ids < 0, 0.0, tw).astype(np.float32)
    ref = O.moe_loop_chain(x, ids_ref, tw_ref, w13d, w2d, E=E, hidden=hidden, inter=inter,
                           fmt13=oracle_kwargs(fmt), fmt2=oracle_kwargs(fmt_2), scale_rule="recip")
    moe = CBMoE(fmt, fmt_2, E, hidden, inter, _tables(fmt, w13d["cb"]), _tables(fmt_2, w2d["cb"]))
    moe.load(torch.from_numpy(w13d["qw"]), torch.from_numpy(w2d["qw"]),
             None if w13d["scale"] is None else torch.from_numpy(w13d["scale"]),
             None if w2d["scale"] is None else torch.from_numpy(w2d["scale"]), dev)
    moe.method.sorted_min_pairs_per_expert = 0              # the routes' thresholds are attributes of the method
    moe.method.sorted_min_pairs_other = 0
    moe.method.prefill_min_pairs_per_expert = 1000000
    got = f32_of(moe(synth.bf16_tensor(x, dev), torch.from_numpy(tw).to(dev), torch.from_numpy(ids).to(dev)))
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    assert "sorted rows" in moe._cb_route
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-2, rel                                         # acceptance bar of the path
    assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())
