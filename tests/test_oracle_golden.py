"""The numpy oracle against fixtures produced by the reference's own torch
decoder and codec (tests/golden/make_golden.py), plus hand-packed known-answer
rows in the style of the reference's tests/test_cb_torch_reference.py:20-101 and
the worked example of docs/SPEC.md:224-240."""
import numpy as np
import pytest

from oracle import cb_oracle as O


def f32(bits):
    return O.bf16_bits_to_f32(bits)


def pack_row(codes, k_bits, tail=b""):
    stream = 0
    for v, c in enumerate(codes):
        stream |= int(c) << (v * k_bits)
    return np.frombuffer(stream.to_bytes(4 * k_bits, "little") + tail, dtype=np.uint8)


@pytest.mark.parametrize("k", [12, 13, 16, 20])
def test_fp4_v2_product_matches_reference(golden, k):
    p = f"fp4v2_k{k}_"
    N, K, ts = 6, 512, 4 * k + 9
    qw, cb, off = golden[p + "qw"], f32(golden[p + "cb"]), golden[p + "off"]
    codes = O.extract_codewords(qw, N=N, K=K, k_bits=k, type_size=ts)
    assert np.array_equal(codes, golden[p + "codes"])
    vals = O.decode_values(qw, cb, off, N=N, K=K, k_bits=k, n_sub=2, type_size=ts)
    assert np.array_equal(O.f32_to_bf16_bits(vals), golden[p + "vals"])
    w = O.reconstruct_weight(qw, cb, off, N=N, K=K, k_bits=k, n_sub=2, type_size=ts,
                             grid="fp4", scale_coding="v2")
    assert np.array_equal(O.f32_to_bf16_bits(w), golden[p + "w"])
    xq = O.fp4_group16_act_qdq(f32(golden[p + "x"]), "div")
    assert np.array_equal(O.f32_to_bf16_bits(xq), golden[p + "xq"])
    y = O.cb_linear(xq, qw, cb, off, N=N, K=K, k_bits=k, n_sub=2, type_size=ts,
                    grid="fp4", scale_coding="v2")
    ref = f32(golden[p + "y"])
    assert np.all(np.abs(y - ref) <= np.maximum(np.abs(y), np.abs(ref)) * 2.0 ** -7 + 1e-5)


def test_compose_and_legality(golden):
    assert np.array_equal(O.compose_table().view(np.uint32), golden["compose"].view(np.uint32))
    assert np.array_equal(O.compose_legal_supers(), golden["legal_supers"])
    legal = O.compose_legal_supers()
    comp = O.compose_table().reshape(256, 16)[legal]
    assert np.array_equal(O.f32_to_e4m3(comp), golden["compose_u8"].reshape(256, 16)[legal])


def test_fp4_v1_scale_bytes(golden):
    k, N, K = 14, 4, 256
    qw, cb = golden["fp4v1_k14_qw"], f32(golden["fp4v1_k14_cb"])
    plane = O.fp4_scale_plane(qw, N=N, K=K, k_bits=k, type_size=4 * k + 16, scale_coding="v1")
    assert np.array_equal(plane, golden["fp4v1_k14_plane"])
    w = O.reconstruct_weight(qw, cb, np.zeros(N, np.int32), N=N, K=K, k_bits=k, n_sub=2,
                             type_size=4 * k + 16, grid="fp4", scale_coding="v1")
    assert np.array_equal(O.f32_to_bf16_bits(w), golden["fp4v1_k14_w"])


def test_fp4_signed(golden):
    k, N, K = 13, 3, 256
    w = O.reconstruct_weight(golden["fp4s_k13_qw"], f32(golden["fp4s_k13_cb"]),
                             np.zeros(N, np.int32), N=N, K=K, k_bits=k, n_sub=1,
                             type_size=4 * k + 9, grid="fp4", scale_coding="v2")
    assert np.array_equal(O.f32_to_bf16_bits(w), golden["fp4s_k13_w"])


@pytest.mark.parametrize("k,n_sub", [(28, 4), (30, 4), (32, 4), (37, 4), (16, 2)])
def test_fp8_product_matches_reference(golden, k, n_sub):
    p = f"fp8_k{k}_n{n_sub}_"
    N, K, ts = 5, 512, 4 * k
    qw, cb, ws = golden[p + "qw"], f32(golden[p + "cb"]), golden[p + "ws"]
    off = np.zeros(N, np.int32)
    assert np.array_equal(O.f32_to_e4m3(cb), golden[p + "cb8"])
    vals = O.decode_values(qw, cb, off, N=N, K=K, k_bits=k, n_sub=n_sub, type_size=ts)
    assert np.array_equal(O.f32_to_e4m3(vals), golden[p + "vals8"])
    w = O.reconstruct_weight(qw, cb, off, N=N, K=K, k_bits=k, n_sub=n_sub, type_size=ts,
                             grid="fp8", weight_scale=ws)
    assert np.array_equal(O.f32_to_bf16_bits(w), golden[p + "w"])
    xq = O.fp8_dynamic_act_qdq(f32(golden[p + "x"]), "div")
    assert np.array_equal(O.f32_to_bf16_bits(xq), golden[p + "xq"])
    y = O.cb_linear(xq, qw, cb, off, N=N, K=K, k_bits=k, n_sub=n_sub, type_size=ts,
                    grid="fp8", weight_scale=ws)
    ref = f32(golden[p + "y"])
    assert np.all(np.abs(y - ref) <= np.maximum(np.abs(y), np.abs(ref)) * 2.0 ** -7 + 1e-5)


def test_activation_buckets_bit_exact(golden):
    x = f32(golden["act_x"])
    assert np.array_equal(O.f32_to_bf16_bits(O.fp4_group16_act_qdq(x, "div")), golden["act_fp4"])
    assert np.array_equal(O.f32_to_bf16_bits(O.fp8_dynamic_act_qdq(x, "div")), golden["act_fp8"])
    packed, sf, recip = O.nvfp4_act_quant(x, 0.37)
    assert np.array_equal(packed, golden["act_nvfp4_packed"])
    assert np.array_equal(sf, golden["act_nvfp4_sf"])
    assert np.float32(recip) == golden["act_nvfp4_recip"][0]


def test_midpoint_trap_separates_the_two_scale_rules():
    """x = -amax/8 sits exactly on the 0.5|1.0 midpoint; the reciprocal-multiply
    scale is one ulp high and lands it on 0.5 (gridbook/csrc/cb_gemv.cu:485-511)."""
    amax = np.float32(1.7265625)
    x = np.zeros((1, 16), np.float32)
    x[0, 0], x[0, 1] = amax, -amax / 8
    lo = O.fp4_group16_act_qdq(x, "recip")[0, 1]
    hi = O.fp4_group16_act_qdq(x, "div")[0, 1]
    assert {abs(float(lo)) / abs(float(hi)), abs(float(hi)) / abs(float(lo))} == {0.5, 2.0}


def test_activation_edge_cases_match_the_reference_codec():
    """Rows the reference's kernel test pins (tests/test_fp4_act_qdq.py:107-149), with the outputs its
    codec gave them (tests/golden/act_edge_cases.json, made by make_act_edge_cases.py): a NaN or an
    infinity inside a group, signed zeros, the smallest bf16 subnormals, the rule-separating midpoint.
    Value classes and every finite output agree for the numpy and the C restatement; NaN payloads are
    not part of the contract."""
    import json
    import os
    from oracle import c_oracle as C
    with open(os.path.join(os.path.dirname(__file__), "golden", "act_edge_cases.json")) as fh:
        cases = json.load(fh)
    assert set(cases) == {"nonfinite", "signed_zero_subnormal", "midpoint"}
    with np.errstate(all="ignore"):
        for name, case in cases.items():
            x = f32(np.array(case["x"], np.uint16)).reshape(case["shape"])
            for grid in ("fp4", "fp8"):
                want = f32(np.array(case[grid], np.uint16)).reshape(case["shape"])
                fin = np.isfinite(want)
                for impl, got in (("numpy", O.bf16_round(O.act_bucket(x, grid, "div"))),
                                  ("c", O.bf16_round(C.act_qdq(x, grid, "div")))):
                    assert np.array_equal(np.isnan(got), np.isnan(want)), (name, grid, impl)
                    assert np.array_equal(np.isposinf(got), np.isposinf(want)), (name, grid, impl)
                    assert np.array_equal(np.isneginf(got), np.isneginf(want)), (name, grid, impl)
                    assert np.array_equal(O.f32_to_bf16_bits(got[fin]), O.f32_to_bf16_bits(want[fin])), (name, grid, impl)


def _e2m1_codes(packed, k):
    return np.stack((packed & 0xF, packed >> 4), axis=-1).reshape(-1, k)


def test_nvfp4_activation_quantiser_rounds_e2m1_midpoints_to_even():
    """Known answer of the reference (tests/test_nvfp4_act_quant_ref.py:17-27,68-77): with a unit
    scale factor every midpoint between two E2M1 rungs goes to the rung with the even code."""
    mids = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    row = np.array([mids + [-v for v in mids] + [6.0, 0.0]], np.float32)
    packed, sf, recip = O.nvfp4_act_quant(row, 1.0)
    even = [0, 2, 2, 4, 4, 6, 6]
    assert _e2m1_codes(packed, 16)[0].tolist() == even + [c | 8 for c in even] + [7, 0]
    assert sf.tolist() == [[0x38]] and float(recip) == 1.0        # E4M3 byte of 1.0


def test_nvfp4_activation_quantiser_scale_factor_underflow_boundary():
    """Known answer of the reference (tests/test_nvfp4_act_quant_ref.py:29-50,80-91): the smallest E4M3
    subnormal is 2^-9, so a group whose maximum is at or under 6 * 2^-10 rounds its scale factor to
    zero (ties to even) and must come out as an all-zero payload, sign bits kept; just above the
    boundary the scale factor is the code 1."""
    edge = 6.0 * 2.0 ** -10
    values = [0.0, 2.0 ** -20, 0.001, 0.003, 0.005, 0.0058, edge, 0.006, 0.008,
              -(2.0 ** -20), -0.001, -0.003, -0.005, -0.0058, -edge, -0.006]
    x = O.bf16_round(np.repeat(np.array(values, np.float32), 16).reshape(1, -1))
    packed, sf, _ = O.nvfp4_act_quant(x, 1.0)
    codes = _e2m1_codes(packed, x.shape[1])[0].reshape(-1, 16)
    under = list(range(7)) + list(range(9, 15))
    assert sf[0, under].tolist() == [0] * len(under)
    assert sf[0, [7, 8, 15]].tolist() == [1, 1, 1]
    assert not codes[:7].any()
    assert np.unique(codes[9:15]).tolist() == [8]                 # a signed numerical zero


def test_sf_swizzle(golden):
    assert np.array_equal(O.swizzle_sf_plane(golden["sf_plain"]), golden["sf_swizzled"])


def test_moe_loop_chain(golden):
    E, hidden, inter, k = 4, 256, 256, 16
    fmt = dict(grid="fp4", k_bits=k, n_sub=2, type_size=4 * k + 9, scale_coding="v2")
    cb = f32(golden["moe_cb"])
    out = O.moe_loop_chain(
        f32(golden["moe_x"]), golden["moe_ids"], golden["moe_tw"],
        dict(qw=golden["moe_w13"], cb=cb), dict(qw=golden["moe_w2"], cb=cb),
        E=E, hidden=hidden, inter=inter, fmt13=fmt, fmt2=fmt)
    ref = f32(golden["moe_out"])
    d = np.abs(out - ref)
    assert np.linalg.norm(d) / np.linalg.norm(ref) < 4e-3


# ---- hand-packed known answers ------------------------------------------------
def test_spec_worked_example_k12():
    """docs/SPEC.md:224-240: K12 product, vector 0 picks (5, 3) -> codeword 197."""
    codes = [5 | (3 << 6)] + [0] * 31
    row = pack_row(codes, 12, bytes([0x38] * 16)).reshape(1, -1)      # E4M3 0x38 = 1.0
    assert row.shape == (1, 64) and row[0, 0] == 197 and row[0, 1] == 0
    t0 = np.arange(64 * 4, dtype=np.float32)
    t1 = -np.arange(64 * 4, dtype=np.float32)
    vals = O.decode_values(row, np.concatenate((t0, t1)), np.zeros(1, np.int32), N=1, K=256,
                           k_bits=12, n_sub=2, type_size=64)
    assert list(vals[0, :8]) == [20, 21, 22, 23, -12, -13, -14, -15]


def test_uneven_split_and_row_offsets():
    k = 13
    codes = [((v * 3) & 0x7F) | (((31 - v) & 0x3F) << 7) for v in range(32)]
    row = pack_row(codes, k)
    qw = np.stack((row, row))
    a = np.concatenate((np.arange(512, dtype=np.float32), -np.arange(256, dtype=np.float32)))
    cb = np.concatenate((a, O.bf16_round(a * 0.25)))
    off = np.array([0, a.size], np.int32)
    got = O.extract_codewords(qw, N=2, K=256, k_bits=k, type_size=4 * k)
    assert list(got[0, 0]) == codes
    vals = O.decode_values(qw, cb, off, N=2, K=256, k_bits=k, n_sub=2, type_size=4 * k)
    for r, blk in enumerate((cb[:a.size], cb[a.size:])):
        exp = []
        for c in codes:
            i0, i1 = c & 0x7F, (c >> 7) & 0x3F
            exp += list(blk[i0 * 4:i0 * 4 + 4]) + list(blk[512 + i1 * 4:512 + i1 * 4 + 4])
        assert list(vals[r]) == exp


def test_signed_sign_bits_and_full_mode():
    k = 13
    codes = [((v % 32) << 8) | ((v * 17) & 0xFF) for v in range(32)]
    qw = pack_row(codes, k).reshape(1, -1)
    cb = np.arange(32 * 8, dtype=np.float32)
    vals = O.decode_values(qw, cb, np.zeros(1, np.int32), N=1, K=256, k_bits=k, n_sub=1,
                           type_size=4 * k)
    for v, c in enumerate(codes):
        for j in range(8):
            e = cb[(c >> 8) * 8 + j]
            assert vals[0, v * 8 + j] == (-e if c & (1 << j) else e)
    # full mode (docs/SPEC.md:97-101): the codeword is the row of a 2^k x 8 table
    codes8 = [(v * 37 + 5) & 0xFF for v in range(32)]
    qw8 = pack_row(codes8, 8).reshape(1, -1)
    cb8 = np.arange(256 * 8, dtype=np.float32)
    vals = O.decode_values(qw8, cb8, np.zeros(1, np.int32), N=1, K=256, k_bits=8, n_sub=1,
                           type_size=32, mode=O.MODE_FULL)
    assert np.array_equal(vals[0].reshape(32, 8), cb8.reshape(256, 8)[codes8])


def test_two_tier_unit_scale_and_fp8_rounding():
    k = 13
    codes = [((v * 5) & 0x7F) | (((v + 7) & 0x3F) << 7) for v in range(32)]
    body = pack_row(codes, k)
    cb = O.bf16_round(np.linspace(-2, 2, 128 * 4 + 64 * 4).astype(np.float32))
    off = np.zeros(1, np.int32)
    vals = O.decode_values(body.reshape(1, -1), cb, off, N=1, K=256, k_bits=k, n_sub=2,
                           type_size=4 * k)
    w8 = O.reconstruct_weight(body.reshape(1, -1), cb, off, N=1, K=256, k_bits=k, n_sub=2,
                              type_size=4 * k, grid="fp8", weight_scale=np.array([0.75], np.float32))
    assert np.array_equal(w8, O.bf16_round(vals * np.float32(0.75)))
    v2 = np.concatenate((body, np.array([127] + [0] * 8, np.uint8))).reshape(1, -1)
    w4 = O.reconstruct_weight(v2, cb, off, N=1, K=256, k_bits=k, n_sub=2, type_size=4 * k + 9,
                              grid="fp4", scale_coding="v2")
    assert np.array_equal(w4, O.bf16_round(vals))


def test_e4m3_round_trip_and_ties():
    allb = np.arange(256, dtype=np.uint8)
    ok = ~np.isnan(O.E4M3_TO_F32)
    assert np.array_equal(O.f32_to_e4m3(O.E4M3_TO_F32[ok]), allb[ok])
    # 0.7265625 is the value the reference notes double-rounds through fp16
    # (gridbook/csrc/cb_gemv.cu:103-129): single rounding gives 0.75 (0x34 -> 0x34)
    assert O.f32_to_e4m3(np.array([0.7265625], np.float32))[0] == O.f32_to_e4m3(
        np.array([0.75], np.float32))[0]
    assert O.f32_to_e4m3(np.array([464.0], np.float32))[0] == 0x7E     # ties-to-even -> 448


def test_route_by_expert():
    ids = np.array([[3, 1], [1, 0], [3, 3]])
    counts, offs, order = O.route_by_expert(ids, 4)
    assert list(counts) == [1, 2, 0, 3] and list(offs) == [0, 1, 3, 3, 6]
    assert list(order) == [3, 1, 2, 0, 4, 5]
