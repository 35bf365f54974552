"""GPU parity at the shapes of the benchmark configurations that the other files do not reach:

  * configuration 1: the q and o projections at one activation row;
  * configuration 2: the linear method at M = 2048 on gate_up and down, both grids, against the
    oracle on a sample of weight rows (the oracle's cost is linear in the rows);
  * configuration 3 at full size with 64 and 256 tokens through the layer method;
  * configuration 4, one rank's share: 32 of 256 experts, hidden 7168, intermediate 2048,
    FP8-grid gate_up (4-element vectors) + NVFP4-grid down, the routed pairs of 512 tokens that
    fall on this rank's experts, against the per-expert loop chain with each stage's own bucket.

The oracle side is the C restatement (OpenMP), seconds per case."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import oracle_kwargs
from oracle import cb_oracle as O
from tests.helpers import assert_close_bf16, f32_of, nvfp4_dequant, nvfp4_quantize_rows_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


def _fmt(name):
    from gridbook_b200 import formats as F
    return {"lit": F.NVFP4_LITERAL, "f8lit": F.FP8_LITERAL, "k16v2": F.NVFP4_CB_K16, "f8k32": F.FP8_CB_K32}[name]


def _c_linear(xq, d, rows=None, expert=None):
    """The oracle's linear on bucketed activations; `rows` picks a sample of weight rows, `expert`
    one matrix of a stack."""
    fmt = d["fmt"]
    qw = d["qw"] if expert is None else d["qw"][expert]
    ws = d.get("weight_scale", d.get("scale"))
    if ws is not None and expert is not None:
        ws = ws[expert]
    if rows is not None:
        qw = np.ascontiguousarray(qw[rows])
        ws = None if ws is None else np.ascontiguousarray(ws[rows])
    return C.linear(xq, qw, d["cb"], None, N=qw.shape[0], K=d["K"], compose=d.get("compose"), weight_scale=ws,
                    global_scale=d.get("global_scale"), **oracle_kwargs(fmt))


def c_loop_chain(x, ids, tw, w13, w2, experts, hidden, inter, scale_rule="recip"):
    """The per-expert loop chain of tests/test_cuda_gemv.py:329-348 (bucket, gate/up, SiLU * up,
    bucket, down, bf16 router weight, bf16 index_add) over the C oracle, each stage with its own
    format and its own activation bucket.  `ids` are local expert ids; anything outside
    [0, experts) is a pair this rank does not serve."""
    T = x.shape[0]
    out = np.zeros((T, hidden), dtype=np.float32)
    f13, f2 = w13["fmt"], w2["fmt"]
    for e in range(experts):
        tok, slot = np.nonzero(ids == e)
        if tok.size == 0:
            continue
        gu = _c_linear(C.act_qdq(x[tok], f13.grid, scale_rule), w13, expert=e)
        a = O.silu_mul(O.bf16_round(gu))
        oe = O.bf16_round(_c_linear(C.act_qdq(a, f2.grid, scale_rule), w2, expert=e))
        oe = O.bf16_round(oe * O.bf16_round(tw[tok, slot])[:, None])
        for i, t in enumerate(tok):
            out[t] = O.bf16_round(out[t] + oe[i])
    return out


def _assert_moe_close(got, ref, tag):
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-2, (tag, rel)
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max(), tag


@pytest.mark.parametrize("N,K", [(6144, 5120), (5120, 6144)])           # q, o
def test_config1_q_and_o_one_row(dev, N, K):
    from gridbook_b200 import _native, kernels, synth
    fmt = _fmt("lit")
    d = synth.make_linear(fmt, N, K, seed=N, global_scale=1.0 / 448.0)
    x = synth.make_activations(1, K, seed=N)
    ref = _c_linear(C.act_qdq(x, "fp4", "recip"), d)
    w = synth.to_device_weight(d, dev)
    y = kernels.gemv(synth.bf16_tensor(x, dev), w, act="fp4")
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    assert_close_bf16(f32_of(y), ref, f"{N}x{K}")


@pytest.mark.parametrize("name", ["lit", "f8lit"])
@pytest.mark.parametrize("N,K", [(34816, 5120), (5120, 17408)])        # gate_up, down
def test_config2_prefill_m2048_row_sample(dev, name, N, K):
    """The linear method's prefill route at M = 2048; 64 sampled weight rows against the oracle."""
    from gridbook_b200 import _native, synth
    from gridbook_b200.linear import CBLinear
    fmt = _fmt(name)
    M = 2048
    gs = 1.0 / 448.0 if name == "lit" else 1.0
    d = synth.make_linear(fmt, N, K, seed=K + len(name), global_scale=gs)
    lin = CBLinear(fmt, K, [N], [_tables(fmt, d["cb"])], global_scale=gs)
    ws = None if fmt.is_fp4 else torch.from_numpy(d["weight_scale"])
    lin.load(torch.from_numpy(d["qw"]), ws, dev)
    x = synth.make_activations(M, K, seed=3)
    y = lin(synth.bf16_tensor(x, dev))
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0 and y.shape == (M, N)
    rows = np.sort(np.random.default_rng(5).choice(N, 64, replace=False))
    got = f32_of(y)[:, rows]
    if fmt.is_fp4:
        # block-scaled route: native NVFP4 activations x the exact weights; the oracle runs on the
        # dequantised activation bytes, and only the summation order differs
        assert "mxf4nvf4" in lin._cb_route["prefill"]
        xa = nvfp4_dequant(*nvfp4_quantize_rows_ref(x))
        assert_close_bf16(got, O.bf16_round(_c_linear(xa, d, rows=rows)), f"{name} {N}x{K} M={M}")
        # and the route that keeps the decode contract (bucketed bf16 rows, bf16 tensor cores)
        lin.method.prefill_route = "bf16"
        y2 = lin(synth.bf16_tensor(x, dev))
        assert_close_bf16(f32_of(y2)[:, rows], _c_linear(C.act_qdq(x, "fp4", "recip"), d, rows=rows),
                          f"{name} {N}x{K} M={M} bf16 route")
    else:                     # E4M3 activations with both scales in the epilogue: the acceptance bar
        ref = _c_linear(C.act_qdq(x, fmt.grid, "recip"), d, rows=rows)
        _assert_moe_close(got, ref, f"{name} {N}x{K} M={M}")


@pytest.mark.parametrize("T", [64, 256])
def test_config3_full_size_through_the_layer_method(dev, T):
    from gridbook_b200 import _native, synth
    from gridbook_b200.moe import CBMoE
    fmt = _fmt("lit")
    E, topk, hidden, inter = 128, 8, 2048, 768
    w13d, w2d = synth.make_moe(fmt, fmt, E, hidden, inter, seed=3)
    ids, tw = synth.make_routing(T, E, topk, seed=T)
    x = synth.make_activations(T, hidden, seed=T)
    ref = c_loop_chain(x, ids, tw, w13d, w2d, E, hidden, inter)
    moe = CBMoE(fmt, fmt, E, hidden, inter, _tables(fmt, w13d["cb"]), _tables(fmt, w2d["cb"]))
    moe.load(torch.from_numpy(w13d["qw"]), torch.from_numpy(w2d["qw"]), None, None, dev)
    out = moe(synth.bf16_tensor(x, dev), torch.from_numpy(tw).to(dev), torch.from_numpy(ids).to(dev))
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    _assert_moe_close(f32_of(out), ref, f"config 3 T={T} ({getattr(moe, '_cb_route', '?')})")


def _tables(fmt, flat):
    out, pos = [], 0
    for r, c in fmt.table_shapes():
        out.append(torch.from_numpy(flat[pos:pos + r * c].reshape(r, c).copy()))
        pos += r * c
    return out


def test_config4_one_ranks_experts(dev):
    """256 experts top-8 over 512 tokens; this rank holds experts 64..95.  Global ids go in, ids
    of other ranks' experts are dropped by the routing launch (as padding is), and the result is
    this rank's partial sum of the routed output."""
    from gridbook_b200 import _native, synth
    from gridbook_b200.moe import CBMoE
    f13, f2 = _fmt("f8lit"), _fmt("lit")
    E_all, E, base, topk, hidden, inter, T = 256, 32, 64, 8, 7168, 2048, 512
    w13d, w2d = synth.make_moe(f13, f2, E, hidden, inter, seed=4)
    ids_all, tw = synth.make_routing(T, E_all, topk, seed=4)
    ids = ids_all - base                                  # local ids; outside [0, 32): another rank's
    x = synth.make_activations(T, hidden, seed=4)
    ref = c_loop_chain(x, ids, tw, w13d, w2d, E, hidden, inter)
    moe = CBMoE(f13, f2, E, hidden, inter, _tables(f13, w13d["cb"]), _tables(f2, w2d["cb"]))
    moe.load(torch.from_numpy(w13d["qw"]), torch.from_numpy(w2d["qw"]), torch.from_numpy(w13d["scale"]), None, dev)
    local = np.where((ids >= 0) & (ids < E), ids, -1).astype(np.int32)
    out = moe(synth.bf16_tensor(x, dev), torch.from_numpy(tw).to(dev), torch.from_numpy(local).to(dev))
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    assert int((local >= 0).sum()) > 400                  # about 512 routed pairs land on this rank
    _assert_moe_close(f32_of(out), ref, f"config 4 rank share ({getattr(moe, '_cb_route', '?')})")


@pytest.mark.parametrize("name,T", [("lit", 3), ("lit", 40), ("lit", 450), ("f8k32", 5), ("f8k32", 450)])
def test_per_role_routed_codebooks(dev, name, T):
    """gate, up and down with a codebook each (configuration 3's wording; docs/SPEC.md:480-527):
    the gate and up rows of w13 select their book by row in the decode kernel and in the decoded
    prefill tile."""
    from gridbook_b200 import _native, synth
    from gridbook_b200.moe import CBMoE
    fmt = _fmt(name)
    E, topk, hidden, inter = 16, 4, 512, 256
    w13d, w2d = synth.make_moe(fmt, fmt, E, hidden, inter, seed=8)
    up_book = synth.make_codebook(fmt, np.random.default_rng(99))
    gate_book = w13d["cb"]
    w13d["cb"] = np.concatenate([gate_book, up_book])
    w13d["cb_row_offset"] = np.concatenate([np.zeros(inter, np.int32),
                                            np.full(inter, fmt.codebook_elems(), np.int32)])
    ids, tw = synth.make_routing(T, E, topk, seed=T)
    x = synth.make_activations(T, hidden, seed=T)
    ref = O.moe_loop_chain(x, ids, tw, w13d, w2d, E=E, hidden=hidden, inter=inter, fmt13=oracle_kwargs(fmt),
                           fmt2=oracle_kwargs(fmt), scale_rule="recip")
    moe = CBMoE(fmt, fmt, E, hidden, inter, [_tables(fmt, gate_book), _tables(fmt, up_book)], _tables(fmt, w2d["cb"]))
    s13 = None if fmt.is_fp4 else torch.from_numpy(w13d["scale"])
    s2 = None if fmt.is_fp4 else torch.from_numpy(w2d["scale"])
    moe.load(torch.from_numpy(w13d["qw"]), torch.from_numpy(w2d["qw"]), s13, s2, dev)
    assert moe._cb_w13.cb_row_offset is not None
    out = moe(synth.bf16_tensor(x, dev), torch.from_numpy(tw).to(dev), torch.from_numpy(ids).to(dev))
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    _assert_moe_close(f32_of(out), ref, f"per-role books {name} T={T} ({getattr(moe, '_cb_route', '?')})")
