"""GPU parity through the plugin surface: the linear / MoE methods driven as an engine
drives them, and the reference-signature ``prismaquant::*`` ops."""
import numpy as np
import pytest
import torch

from oracle import cb_oracle as O
from oracle import oracle_kwargs
from tests.helpers import assert_close_bf16, bits_of, f32_of, oracle_linear, oracle_weight

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


def _tables(fmt, flat):
    out, pos = [], 0
    for r, d in fmt.table_shapes():
        out.append(torch.from_numpy(flat[pos:pos + r * d].reshape(r, d).copy()))
        pos += r * d
    return out


def _formats():
    from gridbook_b200 import formats as F
    return {"lit": F.NVFP4_LITERAL, "k16v2": F.NVFP4_CB_K16, "f8k32": F.FP8_CB_K32, "f8lit": F.FP8_LITERAL}


@pytest.mark.parametrize("name", ["lit", "k16v2", "f8k32", "f8lit"])
def test_linear_method_decode_and_prefill(dev, name):
    """create_weights -> load -> process_weights_after_loading -> apply, for decode batches and
    for a prefill batch (M > 16), with two fused roles that carry their own codebooks."""
    from gridbook_b200 import synth
    from gridbook_b200.linear import CBLinear
    fmt = _formats()[name]
    N, K = 192, 1024
    gs = 1.0 / 448.0 if name == "lit" else 1.0
    d = synth.make_linear(fmt, N, K, seed=17, n_books=2, global_scale=gs)
    n = fmt.codebook_elems()
    lin = CBLinear(fmt, K, [96, 96], [_tables(fmt, d["cb"][:n]), _tables(fmt, d["cb"][n:])], global_scale=gs)
    ws = None if fmt.is_fp4 else torch.from_numpy(d["weight_scale"])
    lin.load(torch.from_numpy(d["qw"]), ws, dev)
    lin.method.prefill_route = "bf16"        # the route that keeps the decode contract (the block-scaled one: test_gpu_gemm_fp4)
    for M in (1, 7, 16, 40, 300):
        x = synth.make_activations(M, K, seed=M)
        y = lin(synth.bf16_tensor(x, dev).reshape(1, M, K))
        assert y.shape == (1, M, N)
        ref = oracle_linear(x, d, bucket=True, scale_rule="recip")
        if M > 16 and not fmt.is_fp4:
            # fp8 prefill multiplies both scales into the accumulator (the reference's fp8
            # prefill epilogue) instead of rounding bf16(value*scale) per weight: acceptance bar
            got = f32_of(y).reshape(M, N)
            assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-2
            assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()
        else:
            assert_close_bf16(f32_of(y).reshape(M, N), ref, f"{name} M={M}")


def test_reference_signature_ops(dev):
    """The dense and expander ops with the reference's argument lists (gridbook/ops.py:52-134),
    on its padded row layout (gridbook/codec.py:200-229)."""
    from gridbook_b200 import codec, synth
    from gridbook_b200.formats import FP8_CB_K32, NVFP4_CB_K16
    import gridbook_b200.ops  # noqa: F401  (registers the ops)
    P = torch.ops.prismaquant
    N, K = 72, 768
    # fp8
    d = synth.make_linear(FP8_CB_K32, N, K, seed=3)
    qwp = codec.with_tail_slack(codec.pad_qweight(torch.from_numpy(d["qw"]).to(dev)))
    cb8 = torch.from_numpy(synth.f32_to_e4m3_bytes(d["cb"])).to(dev)
    off = torch.zeros(N, dtype=torch.int32, device=dev)
    sc = torch.from_numpy(d["weight_scale"]).to(dev)
    x = synth.make_activations(4, K, seed=8)
    y = P.cb_gemv_fp8(synth.bf16_tensor(x, dev), qwp, cb8, off, sc, N, K, 32, 4, 128)
    assert_close_bf16(f32_of(y), oracle_linear(x, d, bucket=True), "cb_gemv_fp8")
    t = P.cb_expand_fp8(qwp, cb8, off, N, K, 32, 4, 128)
    vals = O.decode_values(d["qw"], d["cb"], np.zeros(N, np.int32), N=N, K=K, k_bits=32, n_sub=4, type_size=128)
    assert t.dtype is torch.float8_e4m3fn and np.array_equal(t.view(torch.uint8).cpu().numpy(), O.f32_to_e4m3(vals))
    assert torch.equal(P.fp8_act_qdq(synth.bf16_tensor(x, dev)).cpu(),
                       torch.from_numpy(O.fp8_dynamic_act_qdq(x, "recip")).to(torch.bfloat16))
    # fp4 two-tier
    d = synth.make_linear(NVFP4_CB_K16, N, K, seed=4)
    qwp = codec.with_tail_slack(codec.pad_qweight(torch.from_numpy(d["qw"]).to(dev)))
    cb = torch.from_numpy(d["cb"]).to(torch.bfloat16).to(dev)
    comp = torch.from_numpy(d["compose"]).to(dev)
    xq = P.fp4_act_qdq(synth.bf16_tensor(x, dev))
    assert np.array_equal(bits_of(xq), O.f32_to_bf16_bits(O.fp4_group16_act_qdq(x, "recip")))
    y = P.cb_gemv_fp4_v2(xq, qwp, cb, off, comp, N, K, 16, 2, 73)
    assert_close_bf16(f32_of(y), oracle_linear(x, d, bucket=True), "cb_gemv_fp4_v2")
    t = P.cb_expand_fp4_v2(qwp, cb, comp, 8, 40, K, 16, 73)
    assert np.array_equal(bits_of(t), O.f32_to_bf16_bits(oracle_weight(d)[8:48]))


def test_reference_signature_moe_ops(dev):
    """cb_moe_gemv_* take pairs in ANY order (gridbook/ops.py:494-604): token-major,
    expert-ascending as the reference builds them (gridbook/moe.py:2400-2411)."""
    from gridbook_b200 import synth
    from gridbook_b200.formats import NVFP4_CB_K16
    import gridbook_b200.ops  # noqa: F401
    P = torch.ops.prismaquant
    fmt = NVFP4_CB_K16
    E, hidden, rows, T, topk = 8, 512, 64, 5, 3
    w13d, _ = synth.make_moe(fmt, fmt, E, hidden, rows // 2, seed=2)
    ids, tw = synth.make_routing(T, E, topk, seed=2)
    ids_sorted = np.sort(ids, axis=1)
    x = synth.make_activations(T, hidden, seed=5)
    xq = O.fp4_group16_act_qdq(x, "recip")
    w = synth.to_device_weight(w13d, dev)
    pair_expert = torch.from_numpy(ids_sorted.reshape(-1).astype(np.int32)).to(dev)
    pair_xrow = torch.arange(T, dtype=torch.int32, device=dev).repeat_interleave(topk)
    y = P.cb_moe_gemv_fp4_v2(synth.bf16_tensor(xq, dev), w.qw, w.codebook, w.compose, pair_expert, pair_xrow,
                             16, 2, 73)
    y2 = P.cb_moe_gemv_v2(synth.bf16_tensor(xq, dev), w.qw, w.codebook, w.compose, pair_expert, pair_xrow,
                          16, 73, 0, 0)
    assert torch.equal(y, y2) and y.shape == (T * topk, rows)
    for p in range(T * topk):
        e, t = int(ids_sorted.reshape(-1)[p]), p // topk
        ref = O.cb_linear(xq[t:t + 1], w13d["qw"][e], w13d["cb"], np.zeros(rows, np.int32), N=rows, K=hidden,
                          compose=w13d["compose"], **oracle_kwargs(fmt))
        assert_close_bf16(f32_of(y[p:p + 1]), ref, f"pair {p}")
    pw = torch.from_numpy(tw.reshape(-1)).to(dev)
    out = P.cb_moe_combine(y, pw, torch.arange(T + 1, dtype=torch.int32, device=dev) * topk, T)
    ref = (f32_of(y).reshape(T, topk, rows) * tw[:, :, None]).sum(1)
    assert_close_bf16(f32_of(out), O.bf16_round(ref.astype(np.float32)), "combine")


@pytest.mark.parametrize("f13,f2,T", [("k16v2", "k16v2", 1), ("k16v2", "k16v2", 16), ("k16v2", "k16v2", 70),
                                      ("lit", "lit", 9), ("f8k32", "f8k32", 12), ("f8lit", "lit", 33)])
def test_moe_method_matches_loop_chain(dev, f13, f2, T):
    """The whole routed operator through PrismaQuantCBMoEMethod.apply against the per-expert
    loop chain, for decode batches and past sixteen tokens, same and mixed formats, with a
    padded (-1) route."""
    from gridbook_b200 import synth
    from gridbook_b200.moe import CBMoE
    fmt13, fmt2 = _formats()[f13], _formats()[f2]
    E, hidden, inter, topk = 16, 512, 256, 4
    w13d, w2d = synth.make_moe(fmt13, fmt2, E, hidden, inter, seed=T)
    ids, tw = synth.make_routing(T, E, topk, seed=T)
    x = synth.make_activations(T, hidden, seed=T + 1)
    if T > 4:
        ids[2, 1] = -1                     # vLLM's padding sentinel: that slot contributes nothing
    ids_ref = np.where(ids < 0, 0, ids)
    tw_ref = np.where(ids < 0, 0.0, tw).astype(np.float32)
    ref = O.moe_loop_chain(x, ids_ref, tw_ref, w13d, w2d, E=E, hidden=hidden, inter=inter,
                           fmt13=oracle_kwargs(fmt13), fmt2=oracle_kwargs(fmt2), scale_rule="recip")
    moe = CBMoE(fmt13, fmt2, E, hidden, inter, _tables(fmt13, w13d["cb"]), _tables(fmt2, w2d["cb"]))
    moe.load(torch.from_numpy(w13d["qw"]), torch.from_numpy(w2d["qw"]),
             None if w13d["scale"] is None else torch.from_numpy(w13d["scale"]),
             None if w2d["scale"] is None else torch.from_numpy(w2d["scale"]), dev)
    got = f32_of(moe(synth.bf16_tensor(x, dev), torch.from_numpy(tw).to(dev), torch.from_numpy(ids).to(dev)))
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-2, rel                                         # acceptance bar of the path
    assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())


def test_linear_under_cuda_graph(dev):
    """Capture and replay of the dispatch op returns the eager result (the reference's
    capture gate, tests/test_cb_gemv_v2_cuda.py:145-187)."""
    from gridbook_b200 import synth
    from gridbook_b200.formats import NVFP4_CB_K16
    from gridbook_b200.linear import CBLinear
    fmt = NVFP4_CB_K16
    d = synth.make_linear(fmt, 128, 512, seed=1)
    lin = CBLinear(fmt, 512, [128], [_tables(fmt, d["cb"])]).load(torch.from_numpy(d["qw"]), None, dev)
    x = synth.bf16_tensor(synth.make_activations(2, 512, seed=3), dev)
    eager = lin(x).clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = lin(x)
    x.copy_(synth.bf16_tensor(synth.make_activations(2, 512, seed=4), dev))
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, lin(x)) and not torch.equal(out, eager)
