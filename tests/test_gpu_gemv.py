"""GPU parity, part 2: the decode-batch linear and the routed MoE path against the
oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import cb_oracle as O
from oracle import oracle_kwargs
from tests.helpers import assert_close_bf16, assert_linear_close, f32_of, oracle_linear

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


def _fmt(name):
    from gridbook_b200.formats import CBFormat
    return {
        "lit": CBFormat("fp4", 8, mode="full", scale_coding="v1"),
        "k16v2": CBFormat("fp4", 16, n_sub=2, scale_coding="v2"),
        "k13v2": CBFormat("fp4", 13, n_sub=2, scale_coding="v2"),
        "k20v1": CBFormat("fp4", 20, n_sub=2, scale_coding="v1"),
        "s13": CBFormat("fp4", 13, mode="signed", scale_coding="v2"),
        "f8k32": CBFormat("fp8", 32, n_sub=4),
        "f8k30": CBFormat("fp8", 30, n_sub=4),
        "f8k44": CBFormat("fp8", 44, n_sub=4),
        "f8lit": CBFormat("fp8", 16, n_sub=2),
    }[name]


@pytest.mark.parametrize("name", ["lit", "k16v2", "k13v2", "k20v1", "s13", "f8k32", "f8k30", "f8k44", "f8lit"])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("route", ["default", "no tensor-core decode"])
def test_gemv_matches_oracle(dev, request, name, M, route):
    """Every format at decode batch sizes, on the default routes and with the tensor-core decode kernel
    switched off (the generic decode kernel and the per-row table route of the literal format)."""
    from gridbook_b200 import _native, kernels, synth
    if route != "default":
        _native.set_row_routes(umma_min=129)
        request.addfinalizer(lambda: _native.set_row_routes())
    fmt = _fmt(name)
    N, K = 203, 1024                     # ragged last tile
    d = synth.make_linear(fmt, N, K, seed=5, global_scale=(1.0 / 448.0 if name == "lit" else None))
    w = synth.to_device_weight(d, dev)
    x = synth.make_activations(M, K, seed=M)
    xq = O.act_bucket(x, fmt.grid, "recip")
    y = kernels.gemv(synth.bf16_tensor(xq, dev), w)
    assert_linear_close(f32_of(y), oracle_linear(xq, d, bucket=False), fmt, f"{name} M={M}")
    # fused activation bucket
    y2 = kernels.gemv(synth.bf16_tensor(x, dev), w, act=fmt.grid)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("name", ["lit", "k16v2", "f8k32"])
def test_gemv_padded_rows_and_role_codebooks(dev, name):
    """Row stride wider than the packed row (the reference pads 16 bytes,
    gridbook/codec.py:200-229) and per-row codebook offsets whose boundary cuts a tile."""
    from gridbook_b200 import kernels, synth
    fmt = _fmt(name)
    N, K = 100, 512
    d = synth.make_linear(fmt, N, K, seed=9, n_books=3)       # boundaries at rows 34 and 68
    w = synth.to_device_weight(d, dev, pad_rows=True)
    assert w.row_stride == fmt.row_bytes(K) + 16
    x = synth.make_activations(3, K, seed=2)
    xq = O.act_bucket(x, fmt.grid, "recip")
    y = kernels.gemv(synth.bf16_tensor(xq, dev), w)
    assert_linear_close(f32_of(y), oracle_linear(xq, d, bucket=False), fmt, name)


@pytest.mark.parametrize("name,M,K", [("lit", 16, 8192), ("k16v2", 16, 6144), ("f8k32", 9, 7168)])
def test_gemv_k_sliced(dev, name, M, K):
    """Activation rows too large for one shared-memory slice: K-sliced launch with fp32
    partial sums in the workspace."""
    from gridbook_b200 import kernels, synth
    fmt = _fmt(name)
    N = 264
    d = synth.make_linear(fmt, N, K, seed=11)
    w = synth.to_device_weight(d, dev)
    x = synth.make_activations(M, K, seed=4)
    xq = O.act_bucket(x, fmt.grid, "recip")
    y = kernels.gemv(synth.bf16_tensor(xq, dev), w)
    assert_linear_close(f32_of(y), oracle_linear(xq, d, bucket=False), fmt, f"{name} sliced")


def test_gemv_reference_fixture_k16(dev, golden):
    """y of the reference's own cb_linear_reference on its fixture bytes."""
    from gridbook_b200 import kernels
    from gridbook_b200.formats import CBFormat
    p = "fp4v2_k16_"
    qw = torch.zeros(6 * golden[p + "qw"].shape[1] + 16, dtype=torch.uint8, device=dev)
    qw[:-16] = torch.from_numpy(golden[p + "qw"]).reshape(-1).to(dev)
    w = kernels.make_weight(qw[:-16].view(6, -1),
                            torch.from_numpy(golden[p + "cb"].view(np.int16)).view(torch.bfloat16).to(dev),
                            CBFormat("fp4", 16, n_sub=2, scale_coding="v2"), 512,
                            cb_row_offset=torch.from_numpy(golden[p + "off"]).to(dev),
                            compose=torch.from_numpy(golden["compose"]).to(dev))
    xq = torch.from_numpy(golden[p + "xq"].view(np.int16)).view(torch.bfloat16).to(dev)
    y = kernels.gemv(xq, w)
    assert_close_bf16(f32_of(y), O.bf16_bits_to_f32(golden[p + "y"]), "reference fixture")


def test_gemv_shape_errors(dev):
    from gridbook_b200 import kernels, synth
    d = synth.make_linear(_fmt("lit"), 16, 256, seed=1)
    w = synth.to_device_weight(d, dev)
    # a small layer has no 17..128-row kernel; no layer has one past 128 rows
    with pytest.raises(RuntimeError, match="more than 16 rows"):
        kernels.gemv(torch.zeros(17, 256, dtype=torch.bfloat16, device=dev), w)
    with pytest.raises(RuntimeError, match="1..128 rows"):
        kernels.gemv(torch.zeros(129, 256, dtype=torch.bfloat16, device=dev), w)


# ---- routed MoE -----------------------------------------------------------------
def test_route_matches_oracle(dev):
    from gridbook_b200 import kernels, synth
    # the last three take the tiled ordering (4096 pairs and more, up to 256 experts)
    for T, E, topk in ((1, 128, 8), (16, 128, 8), (256, 128, 8), (37, 9, 3), (512, 128, 8), (4099, 7, 1),
                       (3001, 256, 6)):
        ids, _ = synth.make_routing(T, E, topk, seed=T)
        if T in (37, 4099, 3001):
            ids[0, 0] = -1                                    # padding sentinel is dropped
            ids[T // 2, topk - 1] = -1
        counts, offsets, order = kernels.moe_route(torch.from_numpy(ids).to(dev), E)
        keep = ids.reshape(-1) >= 0
        rc, ro, rorder = O.route_by_expert(np.where(keep, ids.reshape(-1), E).reshape(ids.shape), E + 1)
        assert np.array_equal(counts.cpu().numpy(), rc[:E])
        assert np.array_equal(offsets.cpu().numpy(), ro[:E + 1])
        n = int(ro[E])
        assert np.array_equal(order.cpu().numpy()[:n], rorder[:n])
        if T * topk >= 4096:
            # the wrapper took the three-launch route; the entry point without a workspace orders
            # the same batch inside one CTA
            import ctypes
            from gridbook_b200 import _native as nat
            lib = nat.load("MoE routing")
            idd = torch.from_numpy(ids).to(dev).to(torch.int32).contiguous()
            c2, o2, ord2 = torch.empty_like(counts), torch.empty_like(offsets), torch.empty(T * topk, dtype=torch.int32, device=dev)
            vp = lambda t: ctypes.c_void_p(t.data_ptr())
            nat.check(lib.gb_moe_route(vp(idd), T, topk, E, 0, vp(c2), vp(o2), vp(ord2), None, None,
                                       nat.stream_ptr(dev)), lib)
            assert torch.equal(c2, counts) and torch.equal(o2, offsets) and torch.equal(ord2[:n], order[:n])


def test_route_weights_and_combine_skip_dropped_pairs(dev):
    """The routing launch also writes the combine weights (bf16-rounded, zero for a dropped
    pair), and a combine that is told the ids never reads a dropped pair's row."""
    from gridbook_b200 import kernels, synth
    T, E, topk, H = 9, 12, 4, 64
    ids, tw = synth.make_routing(T, E, topk, seed=3)
    ids[1, 2] = -1
    ids[8, 0] = -1
    idd = torch.from_numpy(ids).to(dev)
    twd = torch.from_numpy(tw).to(dev)
    c0, o0, r0 = kernels.moe_route(idd, E)
    c1, o1, r1, pw = kernels.moe_route(idd, E, twd)
    assert torch.equal(c0, c1) and torch.equal(o0, o1)
    n = int(o0[-1])
    assert torch.equal(r0[:n], r1[:n])
    want = twd.to(torch.bfloat16).float().reshape(-1).masked_fill(idd.reshape(-1) < 0, 0.0)
    assert torch.equal(pw, want)
    rng = np.random.default_rng(0)
    y = torch.from_numpy(rng.standard_normal((T * topk, H)).astype(np.float32)).to(dev).to(torch.bfloat16)
    base = kernels.moe_combine(y.masked_fill((idd.reshape(-1) < 0)[:, None], 0.0), pw, T, topk)
    poisoned = y.clone()
    poisoned[idd.reshape(-1) < 0] = float("nan")          # what an uncleared buffer may hold
    got = kernels.moe_combine(poisoned, pw, T, topk, topk_ids=idd, E=E)
    assert torch.equal(got, base)


def _moe_case(dev, fmt13, fmt2, E, hidden, inter, T, topk, seed):
    from gridbook_b200 import kernels, synth
    w13d, w2d = synth.make_moe(fmt13, fmt2, E, hidden, inter, seed=seed)
    ids, tw = synth.make_routing(T, E, topk, seed=seed)
    x = synth.make_activations(T, hidden, seed=seed)
    f13 = oracle_kwargs(fmt13)
    f2 = oracle_kwargs(fmt2)
    ref = O.moe_loop_chain(x, ids, tw, w13d, w2d, E=E, hidden=hidden, inter=inter, fmt13=f13, fmt2=f2,
                           scale_rule="recip")
    w13 = synth.to_device_weight(w13d, dev)
    w2 = synth.to_device_weight(w2d, dev)
    xd = synth.bf16_tensor(x, dev)
    idd = torch.from_numpy(ids).to(dev)
    _, offsets, order = kernels.moe_route(idd, E)
    xq = (kernels.fp4_act_qdq if fmt13.is_fp4 else kernels.fp8_act_qdq)(xd)
    x_row = (torch.arange(T * topk, device=dev, dtype=torch.int32) // topk).contiguous()
    a = kernels.moe_gemv(xq, w13, offsets, order, x_row=x_row, swiglu=True)
    aq = (kernels.fp4_act_qdq if fmt2.is_fp4 else kernels.fp8_act_qdq)(a)
    yd = kernels.moe_gemv(aq, w2, offsets, order)
    pw = torch.from_numpy(tw).to(dev).to(torch.bfloat16).float().reshape(-1)
    out = kernels.moe_combine(yd, pw, T, topk)
    return f32_of(out), ref


@pytest.mark.parametrize("name", ["k16v2", "lit"])
def test_moe_fused_bucket_equals_separate_bucket(dev, name):
    """The fp4 bucket applied while the grouped kernel stages its rows gives the bits of the
    separate bucket launch, for the gate/up (gathered rows) and the down projection."""
    from gridbook_b200 import kernels, synth
    fmt = _fmt(name)
    E, hidden, inter, T, topk = 8, 512, 256, 7, 3
    w13d, w2d = synth.make_moe(fmt, fmt, E, hidden, inter, seed=9)
    ids, _ = synth.make_routing(T, E, topk, seed=9)
    w13, w2 = synth.to_device_weight(w13d, dev), synth.to_device_weight(w2d, dev)
    xd = synth.bf16_tensor(synth.make_activations(T, hidden, seed=9), dev)
    _, offsets, order = kernels.moe_route(torch.from_numpy(ids).to(dev), E)
    x_row = (torch.arange(T * topk, device=dev, dtype=torch.int32) // topk).contiguous()
    a_sep = kernels.moe_gemv(kernels.fp4_act_qdq(xd), w13, offsets, order, x_row=x_row, swiglu=True)
    a_fused = kernels.moe_gemv(xd, w13, offsets, order, x_row=x_row, swiglu=True, act="fp4")
    assert torch.equal(a_sep, a_fused)
    y_sep = kernels.moe_gemv(kernels.fp4_act_qdq(a_sep), w2, offsets, order)
    y_fused = kernels.moe_gemv(a_sep, w2, offsets, order, act="fp4")
    assert torch.equal(y_sep, y_fused)


@pytest.mark.parametrize("T,inter", [(1, 768), (7, 768), (40, 768), (5, 1280)])
def test_moe_per_pair_table_kernel_matches_grouped_kernel(dev, T, inter):
    """Literal format: every routed pair as its own table GEMV (gate/up K = 2048: two K slices and
    SwiGLU in the summing kernel; down K = 768: one ragged slice, stored straight from the kernel)
    against the grouped MMA kernel on the same bits and against the loop-chain oracle, with a
    padded route."""
    from gridbook_b200 import kernels, synth
    fmt = _fmt("lit")
    E, hidden, topk = 8, 2048, 3            # inter = 1280: the down projection has two K slices too
    w13d, w2d = synth.make_moe(fmt, fmt, E, hidden, inter, seed=T)
    ids, tw = synth.make_routing(T, E, topk, seed=T)
    if T > 1:
        ids[1, 0] = -1
    x = synth.make_activations(T, hidden, seed=T)
    w13, w2 = synth.to_device_weight(w13d, dev), synth.to_device_weight(w2d, dev)
    xd = synth.bf16_tensor(x, dev)
    idd = torch.from_numpy(ids).to(dev)
    x_row = (torch.arange(T * topk, device=dev, dtype=torch.int32) // topk).contiguous()
    _, offsets, order = kernels.moe_route(idd, E)
    a_ref = kernels.moe_gemv(kernels.fp4_act_qdq(xd), w13, offsets, order, x_row=x_row, swiglu=True)
    a = kernels.moe_gemv_pairs(xd, w13, idd, x_row=x_row, swiglu=True, act="fp4")
    assert a is not None
    live = (idd.reshape(-1) >= 0)
    # SwiGLU rounds gate and up to bf16 first: a last-bit difference of the two summation orders in
    # either one moves the product by a few steps, hence the wider elementwise gate here
    assert_close_bf16(f32_of(a[live]), f32_of(a_ref[live]), "per-pair gate/up vs grouped", ulps=8.0)
    y_ref = kernels.moe_gemv(kernels.fp4_act_qdq(a), w2, offsets, order)
    y = kernels.moe_gemv_pairs(a, w2, idd, act="fp4")
    assert_close_bf16(f32_of(y[live]), f32_of(y_ref[live]), "per-pair down vs grouped")
    # both projections chained (the down projection sums the gate/up slices itself): same bits
    y_chain = kernels.moe_mlp_pairs(xd, w13, w2, idd, x_row=x_row)
    assert torch.equal(y_chain[live], y[live])
    out = kernels.moe_combine(y, torch.from_numpy(tw).to(dev), T, topk, topk_ids=idd, E=E, round_weights=True)
    keep = ids >= 0
    ref = O.moe_loop_chain(x, np.where(keep, ids, 0), np.where(keep, tw, 0.0).astype(np.float32), w13d, w2d, E=E,
                           hidden=hidden, inter=inter, fmt13=oracle_kwargs(fmt), fmt2=oracle_kwargs(fmt),
                           scale_rule="recip")
    got = f32_of(out)
    rel = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-9)
    assert rel <= 1e-2, rel
    # a format without the kernel is refused, not served some other way
    k16 = _fmt("k16v2")
    o13, _ = synth.make_moe(k16, k16, 4, 512, 256, seed=1)
    assert kernels.moe_gemv_pairs(synth.bf16_tensor(synth.make_activations(2, 512, seed=1), dev),
                                  synth.to_device_weight(o13, dev),
                                  torch.zeros(2, dtype=torch.int32, device=dev), swiglu=True) is None


@pytest.mark.parametrize("T", [1, 5, 16, 40])
def test_moe_fp4_k16_matches_loop_chain(dev, T):
    fmt = _fmt("k16v2")
    got, ref = _moe_case(dev, fmt, fmt, E=16, hidden=512, inter=256, T=T, topk=4, seed=T)
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-2 and np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max()), rel


def test_moe_literal_and_fp8_and_mixed(dev):
    for f13, f2 in (("lit", "lit"), ("f8k32", "f8k32"), ("f8lit", "lit")):
        got, ref = _moe_case(dev, _fmt(f13), _fmt(f2), E=8, hidden=512, inter=256, T=6, topk=2, seed=3)
        rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert rel <= 1e-2, (f13, f2, rel)


@pytest.mark.parametrize("N,K", [(512, 1024), (1000, 2304), (640, 1536), (768, 2816), (2048, 5120), (5120, 4352)])
def test_literal_single_row_table_kernel(dev, N, K):
    """M = 1 on the literal format with enough rows takes the inner-product-table kernel: ragged
    row count, a last K slice of one, two or three superblocks, padded row stride, bucket fused
    or applied beforehand, including zero, subnormal and negative scale bytes."""
    from gridbook_b200 import kernels, synth
    fmt = _fmt("lit")
    d = synth.make_linear(fmt, N, K, seed=N + K, global_scale=1.0 / 448.0)
    qw = d["qw"].reshape(N, K // 256, 48)
    qw[::7, 0, 32:40] = np.arange(8, dtype=np.uint8)          # E4M3 zero and subnormal scales
    qw[::5, -1, 40:44] = np.array([0x88, 0xB8, 0xFE, 0x81], dtype=np.uint8)   # negative scales, -448 included
    d["qw"] = qw.reshape(N, -1)
    x = synth.make_activations(1, K, seed=3)
    ref = oracle_linear(x, d, bucket=True, scale_rule="recip")
    for pad in (False, True):
        w = synth.to_device_weight(d, dev, pad_rows=pad)
        y = kernels.gemv(synth.bf16_tensor(x, dev), w, act="fp4")
        assert_close_bf16(f32_of(y), ref, f"fused bucket pad={pad}")
        xq = O.act_bucket(x, "fp4", "recip")
        y2 = kernels.gemv(synth.bf16_tensor(xq, dev), w)
        assert torch.equal(y, y2)


@pytest.mark.parametrize("N,K,M", [(256, 1024, 2), (384, 2048, 16), (1000, 2304, 5), (640, 1536, 100),
                                   (2048, 5120, 9), (5120, 4352, 128), (300, 1280, 33),
                                   # shards of the benchmark's projections over eight and four ranks: few
                                   # row tiles, up to seventeen K slices
                                   (768, 5120, 16), (256, 5120, 16), (640, 6144, 16), (4352, 5120, 16),
                                   (640, 17408, 16), (1280, 17408, 5)])
def test_literal_row_batch_tensor_core_decode_kernel(dev, request, N, K, M):
    """2..128 rows of the literal format take the kernel that decodes into shared memory and runs
    tcgen05 MMAs with the weights on the M side: ragged row counts on both sides, a last raw stage
    of one to three superblocks, one or several K slices, padded row stride, bucket applied by the
    call or beforehand, zero / subnormal / negative scale bytes."""
    from gridbook_b200 import _native, kernels, synth
    _native.set_row_routes(umma_min=2)                        # by default it serves 5 rows and more
    request.addfinalizer(lambda: _native.set_row_routes())
    fmt = _fmt("lit")
    d = synth.make_linear(fmt, N, K, seed=N + K + M, global_scale=1.0 / 448.0)
    qw = d["qw"].reshape(N, K // 256, 48)
    qw[::7, 0, 32:40] = np.arange(8, dtype=np.uint8)
    qw[::5, -1, 40:44] = np.array([0x88, 0xB8, 0xFE, 0x81], dtype=np.uint8)
    d["qw"] = qw.reshape(N, -1)
    x = synth.make_activations(M, K, seed=M)
    ref = oracle_linear(x, d, bucket=True, scale_rule="recip")
    for pad in (False, True):
        w = synth.to_device_weight(d, dev, pad_rows=pad)
        y = kernels.gemv(synth.bf16_tensor(x, dev), w, act="fp4")
        torch.cuda.synchronize()
        assert _native.device_status(0) == 0
        assert_close_bf16(f32_of(y), ref, f"M={M} pad={pad}")
        y2 = kernels.gemv(synth.bf16_tensor(O.act_bucket(x, "fp4", "recip"), dev), w)
        assert torch.equal(y, y2)


@pytest.mark.parametrize("name,N,K,M", [("k16v2", 256, 1024, 1), ("k16v2", 1000, 2304, 5), ("k16v2", 384, 2048, 16),
                                        ("k16v2", 640, 1536, 64), ("k16v2", 2048, 5120, 96),
                                        ("f8k32", 256, 1024, 1), ("f8k32", 1000, 2304, 7), ("f8k32", 384, 2048, 16),
                                        ("f8k32", 640, 1536, 48), ("f8k32", 2048, 5120, 80),
                                        ("f8lit", 256, 1024, 1), ("f8lit", 1000, 2304, 7), ("f8lit", 640, 1536, 64),
                                        ("f8lit", 2048, 5120, 96)])
def test_product_formats_on_the_tensor_core_decode_kernel(dev, name, N, K, M):
    """The two-tier fp4 k = 16 format (its 73-byte superblocks kept in 80-byte slots) and the fp8
    product formats k = 32 and k = 16 run on the kernel that decodes into tensor memory from ONE row on: ragged row
    counts on both sides, a last raw stage of one superblock, one or several K slices, legal and
    extreme super-block exponents, against the oracle on the unpadded bytes."""
    from gridbook_b200 import _native, codec, kernels, synth
    fmt = _fmt(name)
    d = synth.make_linear(fmt, N, K, seed=N + K + M, super_span=None if name == "k16v2" else 4)
    x = synth.make_activations(M, K, seed=M)
    ref = oracle_linear(x, d, bucket=True, scale_rule="recip")
    if name == "k16v2":
        dp = dict(d, fmt=fmt.padded(80), qw=codec.pad_superblocks(torch.from_numpy(d["qw"]), 73, 80).numpy())
    else:
        dp = d
    w = synth.to_device_weight(dp, dev)
    assert kernels.row_batch_max_rows(w) >= M
    y = kernels.gemv(synth.bf16_tensor(x, dev), w, act=fmt.grid)
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    # several accumulators added at the end and sums of thousands of large terms that cancel (the
    # whole range of super-block exponents): an absolute allowance next to the two ULPs
    assert_close_bf16(f32_of(y), ref, f"{name} M={M}", atol_rel=2e-4)
    # the padded layout decodes to the same weights through the generic kernels too
    wt = kernels.expand_fp4_bf16(w) if fmt.is_fp4 else kernels.expand_fp8_bf16(w)
    wu = synth.to_device_weight(d, dev)
    wt_u = kernels.expand_fp4_bf16(wu) if fmt.is_fp4 else kernels.expand_fp8_bf16(wu)
    assert torch.equal(wt, wt_u)


def test_two_tier_scale_table_that_is_not_exact_in_bf16_takes_the_fp32_path(dev):
    """A custom sub-table with more than eight significant bits: the kernel notices while it converts
    the table and multiplies in fp32, so the served weight is still bf16(value * scale)."""
    from gridbook_b200 import codec, kernels, synth
    fmt = _fmt("k16v2")
    N, K, M = 256, 1024, 4
    d = synth.make_linear(fmt, N, K, seed=5)
    table = np.array([1.0 + i * (1.0 / 16) + 2.0 ** -12 for i in range(16)], dtype=np.float64)
    d["compose"] = synth.compose_table(tuple(table))
    x = synth.make_activations(M, K, seed=2)
    ref = oracle_linear(x, d, bucket=True, scale_rule="recip")
    dp = dict(d, fmt=fmt.padded(80), qw=codec.pad_superblocks(torch.from_numpy(d["qw"]), 73, 80).numpy())
    y = kernels.gemv(synth.bf16_tensor(x, dev), synth.to_device_weight(dp, dev), act="fp4")
    assert_close_bf16(f32_of(y), ref, "inexact table")
