"""The restatement against the reference's own torch decoder and codec, run live on fresh seeded
inputs (beyond the committed fixtures), wherever oracle/_ref is present.  oracle/make_ref.py makes
that folder from a reference checkout; a machine without one skips this file."""
import numpy as np
import pytest
import torch

from gridbook_b200 import formats, synth
from oracle import c_oracle as C
from oracle import cb_oracle as O
from oracle import make_ref, oracle_kwargs

pytestmark = pytest.mark.skipif(not make_ref.available(), reason="oracle/_ref is not present on this machine")


@pytest.fixture(scope="module")
def ref():
    return make_ref.load()


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def _ref_args(d, fmt):
    N = d["N"]
    off = d["cb_row_offset"] if d["cb_row_offset"] is not None else np.zeros(N, np.int32)
    qwp = torch.nn.functional.pad(torch.from_numpy(d["qw"]), (0, 16))
    scale = torch.from_numpy(d["weight_scale"]) if d["weight_scale"] is not None else torch.zeros(1)
    compose = torch.from_numpy(d["compose"]) if d["compose"] is not None else torch.zeros(1)
    args = (qwp, torch.from_numpy(d["cb"]).to(torch.bfloat16), torch.from_numpy(off), scale, compose)
    kw = dict(N=N, K=d["K"], k_bits=fmt.k, n_sub=fmt.n_sub, type_size=fmt.type_size, is_fp4=fmt.is_fp4,
              is_v2=fmt.scale_coding == "v2")
    return args, kw, off


@pytest.mark.parametrize("name,n_books", [("NVFP4_CB_K16", 1), ("NVFP4_CB_K16", 3), ("FP8_CB_K32", 1),
                                          ("FP8_LITERAL", 2)])
@pytest.mark.parametrize("seed", [11, 12])
def test_weight_and_linear_match_the_reference_code(ref, name, n_books, seed):
    cbref, codec = ref
    fmt = getattr(formats, name)
    N, K, M = 24, 768, 3
    d = synth.make_linear(fmt, N, K, seed=seed, n_books=n_books)
    args, kw, off = _ref_args(d, fmt)
    w_ref = cbref.reconstruct_cb_weight(*args, **kw)
    okw = oracle_kwargs(fmt)
    w = O.reconstruct_weight(d["qw"], d["cb"], off, N=N, K=K, compose=d["compose"],
                             weight_scale=d["weight_scale"], **okw)
    assert np.array_equal(O.f32_to_bf16_bits(w), _bits(w_ref))
    w_c = C.reconstruct(d["qw"], d["cb"], off, N=N, K=K, compose=d["compose"],
                        weight_scale=d["weight_scale"], **okw)
    assert np.array_equal(O.f32_to_bf16_bits(w_c), _bits(w_ref))

    x = torch.from_numpy(synth.make_activations(M, K, seed=seed)).to(torch.bfloat16)
    xq_ref = codec.fp4_group16_act_qdq(x) if fmt.is_fp4 else codec.fp8_dynamic_act_qdq(x)
    xq = O.act_bucket(x.float().numpy(), fmt.grid, "div")
    assert np.array_equal(O.f32_to_bf16_bits(xq), _bits(xq_ref))
    y_ref = cbref.cb_linear_reference(xq_ref, *args, **kw).float().numpy()
    y = O.cb_linear(xq, d["qw"], d["cb"], off, N=N, K=K, compose=d["compose"],
                    weight_scale=d["weight_scale"], **okw)
    tol = np.maximum(np.abs(y), np.abs(y_ref)) * 2.0 ** -7 + 1e-5     # one bf16 step: only the sum's order differs
    assert np.all(np.abs(y - y_ref) <= tol)


@pytest.mark.parametrize("seed", [21, 22])
def test_nvfp4_activation_quantiser_matches_the_reference_code(ref, seed):
    _, codec = ref
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((5, 256)) * rng.choice([1e-3, 1.0, 50.0], size=(5, 1))).astype(np.float32)
    x[3, 16:32] = 0.0
    xb = torch.from_numpy(x).to(torch.bfloat16)
    gs = torch.tensor(448.0 * 6.0 / float(xb.float().abs().max()))
    packed_ref, sf_ref, _ = codec.nvfp4_act_quant_ref(xb.float(), gs)
    out = O.nvfp4_act_quant(xb.float().numpy(), float(gs))
    packed, sf = out[0], out[1]
    assert np.array_equal(packed, packed_ref.view(torch.uint8).numpy())
    assert np.array_equal(sf, sf_ref.view(torch.uint8).numpy().reshape(sf.shape))


def test_activation_buckets_on_nonfinite_groups_signed_zero_and_subnormals_match_the_reference_code(ref):
    """Rows the reference's kernel test pins against its codec (tests/test_fp4_act_qdq.py:118-149): a NaN
    or an infinity decides its whole group (torch.amax spreads a NaN), signed zeros and bf16
    subnormals come back as the codec writes them.  Value classes and every finite output agree;
    NaN payloads are not compared."""
    _, codec = ref
    rows = torch.tensor([[float("nan"), 1.0] + [0.0] * 14 + [1.0, -2.0] + [0.5] * 14,
                         [float("inf"), -1.0] + [0.0] * 14 + [3.0, 0.25] + [0.0] * 14,
                         [float("-inf"), 1.0] + [0.0] * 14 + [float("nan")] + [1.0] * 15], dtype=torch.bfloat16)
    raw = torch.tensor([0, -32768, 1, -32767] * 8, dtype=torch.int16).view(torch.bfloat16).reshape(1, 32)
    with np.errstate(all="ignore"):
        for fn_ref, fn in ((codec.fp4_group16_act_qdq, O.fp4_group16_act_qdq),
                           (codec.fp8_dynamic_act_qdq, O.fp8_dynamic_act_qdq)):
            want = fn_ref(rows).to(torch.bfloat16).float().numpy()
            got = O.bf16_round(fn(rows.float().numpy(), "div"))
            assert np.array_equal(np.isnan(got), np.isnan(want))
            assert np.array_equal(np.isposinf(got), np.isposinf(want))
            assert np.array_equal(np.isneginf(got), np.isneginf(want))
            fin = np.isfinite(want)
            assert np.array_equal(got[fin], want[fin])
            assert np.array_equal(O.f32_to_bf16_bits(fn(raw.float().numpy(), "div")), _bits(fn_ref(raw)))
