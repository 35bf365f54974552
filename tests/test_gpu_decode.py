"""GPU parity, part 1: activation buckets and decoded tiles, bit-exact against the
oracle and against the reference-generated fixtures.  All calls go through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import cb_oracle as O
from oracle import oracle_kwargs
from tests.helpers import bits_of, oracle_weight

pytestmark = pytest.mark.gpu

FORMATS = None


def _formats():
    from gridbook_b200.formats import CBFormat
    return [
        CBFormat("fp4", 8, mode="full", scale_coding="v1"),
        CBFormat("fp4", 8, mode="full", scale_coding="v2"),
        CBFormat("fp4", 12, n_sub=2, scale_coding="v2"),
        CBFormat("fp4", 13, n_sub=2, scale_coding="v2"),
        CBFormat("fp4", 16, n_sub=2, scale_coding="v2"),
        CBFormat("fp4", 16, n_sub=2, scale_coding="v1"),
        CBFormat("fp4", 21, n_sub=2, scale_coding="v2"),
        CBFormat("fp4", 24, n_sub=2, scale_coding="v2"),
        CBFormat("fp4", 13, mode="signed", scale_coding="v2"),
        CBFormat("fp4", 16, mode="signed", scale_coding="v1"),
        CBFormat("fp8", 16, n_sub=2),
        CBFormat("fp8", 28, n_sub=4),
        CBFormat("fp8", 30, n_sub=4),
        CBFormat("fp8", 32, n_sub=4),
        CBFormat("fp8", 37, n_sub=4),
        CBFormat("fp8", 48, n_sub=4),
    ]


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


@pytest.mark.parametrize("idx", range(16))
def test_expand_bit_exact(dev, idx):
    from gridbook_b200 import kernels, synth
    fmt = _formats()[idx]
    N, K = 37, 768                      # odd row count, three superblocks
    d = synth.make_linear(fmt, N, K, seed=10 + idx, n_books=2, super_span=None)
    w = synth.to_device_weight(d, dev)
    ref = oracle_weight(d)
    if fmt.is_fp4:
        got = kernels.expand_fp4_bf16(w)
        assert np.array_equal(bits_of(got), O.f32_to_bf16_bits(ref))
        # a row window that starts and ends mid-matrix
        part = kernels.expand_fp4_bf16(w, 5, 11)
        assert np.array_equal(bits_of(part), O.f32_to_bf16_bits(ref[5:16]))
        packed, sf = kernels.expand_fp4_nvfp4(w)
        rp, rs = O.decode_nvfp4_tile(d["qw"], d["cb"], d["cb_row_offset"], N=N, K=K, compose=d["compose"],
                                     **{k: v for k, v in oracle_kwargs(fmt).items() if k != "grid"})
        assert np.array_equal(packed.cpu().numpy(), rp)
        assert np.array_equal(sf.cpu().numpy(), rs)
        _, sfs = kernels.expand_fp4_nvfp4(w, swizzled=True)
        assert np.array_equal(sfs.cpu().numpy(), O.swizzle_sf_plane(rs))
    else:
        got = kernels.expand_fp8(w)
        vals = O.decode_values(d["qw"], d["cb"], d["cb_row_offset"], N=N, K=K, k_bits=fmt.k, n_sub=fmt.n_sub,
                               type_size=fmt.type_size)
        assert np.array_equal(got.view(torch.uint8).cpu().numpy(), O.f32_to_e4m3(vals))
        # the served weight bf16(value * row scale), whole and over a row window
        assert np.array_equal(bits_of(kernels.expand_fp8_bf16(w)), O.f32_to_bf16_bits(ref))
        assert np.array_equal(bits_of(kernels.expand_fp8_bf16(w, 5, 11)), O.f32_to_bf16_bits(ref[5:16]))


def test_expand_matches_reference_fixtures(dev, golden):
    """Decoded tiles of the reference's own fixtures (its decoder's outputs are stored)."""
    from gridbook_b200 import kernels
    from gridbook_b200.formats import CBFormat
    comp = torch.from_numpy(golden["compose"]).to(dev)
    for k in (12, 13, 16, 20):
        p = f"fp4v2_k{k}_"
        qw = torch.zeros(6 * golden[p + "qw"].shape[1] + 16, dtype=torch.uint8, device=dev)
        qw[:-16] = torch.from_numpy(golden[p + "qw"]).reshape(-1).to(dev)
        w = kernels.make_weight(qw[:-16].view(6, -1),
                                torch.from_numpy(golden[p + "cb"].view(np.int16)).view(torch.bfloat16).to(dev),
                                CBFormat("fp4", k, n_sub=2, scale_coding="v2"), 512,
                                cb_row_offset=torch.from_numpy(golden[p + "off"]).to(dev), compose=comp)
        assert np.array_equal(bits_of(kernels.expand_fp4_bf16(w)), golden[p + "w"])
    for k, n_sub in ((28, 4), (30, 4), (32, 4), (37, 4), (16, 2)):
        p = f"fp8_k{k}_n{n_sub}_"
        qw = torch.zeros(5 * golden[p + "qw"].shape[1] + 16, dtype=torch.uint8, device=dev)
        qw[:-16] = torch.from_numpy(golden[p + "qw"]).reshape(-1).to(dev)
        w = kernels.make_weight(qw[:-16].view(5, -1), torch.from_numpy(golden[p + "cb8"]).to(dev),
                                CBFormat("fp8", k, n_sub=n_sub), 512,
                                weight_scale=torch.from_numpy(golden[p + "ws"]).to(dev))
        got = kernels.expand_fp8(w)
        assert np.array_equal(got.view(torch.uint8).cpu().numpy(), golden[p + "vals8"])


def test_activation_buckets_bit_exact(dev, golden):
    from gridbook_b200 import kernels
    x = torch.from_numpy(golden["act_x"].view(np.int16)).view(torch.bfloat16).to(dev)
    # division rule == the fixtures the reference's codec produced on the CPU
    assert np.array_equal(bits_of(kernels.fp4_act_qdq(x, "div")), golden["act_fp4"])
    assert np.array_equal(bits_of(kernels.fp8_act_qdq(x, "div")), golden["act_fp8"])
    # reciprocal rule == the oracle's restatement of the reference's CUDA kernels
    xf = O.bf16_bits_to_f32(golden["act_x"])
    assert np.array_equal(bits_of(kernels.fp4_act_qdq(x, "recip")),
                          O.f32_to_bf16_bits(O.fp4_group16_act_qdq(xf, "recip")))
    assert np.array_equal(bits_of(kernels.fp8_act_qdq(x, "recip")),
                          O.f32_to_bf16_bits(O.fp8_dynamic_act_qdq(xf, "recip")))


@pytest.mark.parametrize("seed", [0, 1])
def test_activation_buckets_random_and_ties(dev, seed):
    """Tie hunting (tests/test_fp4_act_qdq.py in the reference): values placed on exact
    grid midpoints of their group scale, both scale rules, large random rows."""
    from gridbook_b200 import kernels
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((16, 4096)).astype(np.float32) * rng.choice([1e-3, 1.0, 50.0], (16, 1))
    amax = np.abs(x.reshape(16, -1, 16)).max(axis=-1, keepdims=True)
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32) / 6.0
    xt = x.reshape(16, -1, 16).copy()
    xt[:, ::3, 1] = (amax[:, ::3, 0] * mids[seed % 7])
    xt[:, 1::3, 2] = -(amax[:, 1::3, 0] * mids[(seed + 3) % 7])
    xf = O.bf16_round(xt.reshape(16, 4096))
    xd = torch.from_numpy(xf).to(torch.bfloat16).to(dev)
    for rule in ("recip", "div"):
        assert np.array_equal(bits_of(kernels.fp4_act_qdq(xd, rule)),
                              O.f32_to_bf16_bits(O.fp4_group16_act_qdq(xf, rule))), rule
        assert np.array_equal(bits_of(kernels.fp8_act_qdq(xd, rule)),
                              O.f32_to_bf16_bits(O.fp8_dynamic_act_qdq(xf, rule))), rule


def test_recip_rule_is_what_torch_cuda_computes(dev):
    """The reciprocal rule exists because torch on CUDA evaluates `amax / 6.0` that way
    (gridbook/csrc/cb_gemv.cu:485-511); check the claim on this device."""
    a = torch.tensor([1.7265625, 7.0, 0.3, 123.456], dtype=torch.float32, device=dev)
    assert torch.equal(a / 6.0, a * torch.tensor(1.0 / 6.0, dtype=torch.float32, device=dev))


def test_argument_errors(dev):
    from gridbook_b200 import kernels, synth
    from gridbook_b200.formats import CBFormat
    with pytest.raises(RuntimeError, match="multiple of the fp4 group"):
        kernels.fp4_act_qdq(torch.zeros(2, 24, dtype=torch.bfloat16, device=dev))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernels.fp4_act_qdq(torch.zeros(2, 32, dtype=torch.bfloat16))
    d = synth.make_linear(CBFormat("fp8", 32, n_sub=4), 8, 256, seed=3)
    w = synth.to_device_weight(d, dev)
    with pytest.raises(RuntimeError, match="outside"):
        kernels.expand_fp8(w, 4, 8)
    with pytest.raises(RuntimeError, match="fp4-grid"):
        kernels.expand_fp4_bf16(w)


def test_activation_buckets_nonfinite_groups_signed_zero_and_subnormals(dev):
    """The classes the reference pins for the group-16 bucket in tests/test_fp4_act_qdq.py:118-149: a NaN
    or an infinity in a group decides the whole group the way torch.amax does (CUDA's fmaxf alone
    would ignore a lone NaN); signed zeros and bf16 subnormals keep the codec's bits.  Value classes
    and every finite output must match the oracle (which matches the reference's codec on these
    rows); NaN payloads are not part of the contract.  The per-token fp8 bucket is not part of this
    contract: the reference's own kernel (gridbook/csrc/cb_gemv.cu:135-172) takes the row maximum
    with fmaxf, so a lone NaN there clamps to -448 instead of spreading, and this library does the
    same; only finite rows are pinned for it."""
    from gridbook_b200 import kernels
    rows = torch.tensor([[float("nan"), 1.0] + [0.0] * 14 + [1.0, -2.0] + [0.5] * 14,
                         [float("inf"), -1.0] + [0.0] * 14 + [3.0, 0.25] + [0.0] * 14,
                         [float("-inf"), 1.0] + [0.0] * 14 + [float("nan")] + [1.0] * 15], dtype=torch.bfloat16)
    with np.errstate(all="ignore"):
        for rule in ("recip", "div"):
            got = kernels.fp4_act_qdq(rows.to(dev), rule).float().cpu().numpy()
            ref = O.bf16_round(O.fp4_group16_act_qdq(rows.float().numpy(), rule))
            assert np.array_equal(np.isnan(got), np.isnan(ref)), (rule, got, ref)
            assert np.array_equal(np.isposinf(got), np.isposinf(ref)), rule
            assert np.array_equal(np.isneginf(got), np.isneginf(ref)), rule
            fin = np.isfinite(ref)
            assert np.array_equal(got[fin], ref[fin]), rule
    raw = torch.tensor([0, -32768, 1, -32767] * 8, dtype=torch.int16)
    x = raw.view(torch.bfloat16).reshape(1, 32)
    for rule in ("recip", "div"):
        got = bits_of(kernels.fp4_act_qdq(x.to(dev), rule))
        assert np.array_equal(got, O.f32_to_bf16_bits(O.fp4_group16_act_qdq(x.float().numpy(), rule))), rule
