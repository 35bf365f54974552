"""The block-scaled FP4 prefill through the C ABI: the NVFP4 row quantiser bit for bit against
the oracle, the tcgen05 kind::mxf4nvf4 GEMM against an fp64 product of the dequantised operands
(ragged M, several tiles per CTA, negative group scales folded into the values), and the linear
method's prefill route against the oracle run on the dequantised NVFP4 activation bytes - the
reference's own check of this lane (tests/test_fused_fp4_prefill.py:118-140,254)."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import cb_oracle as O
from tests.helpers import assert_close_bf16, f32_of, nvfp4_dequant, nvfp4_quantize_rows_ref, oracle_weight

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


def _unswizzle(plane: np.ndarray, rows: int, groups: int) -> np.ndarray:
    return plane[O.sf_swizzle_offsets(rows, groups).reshape(-1)].reshape(rows, groups)


def test_row_quantiser_is_bit_exact(dev):
    from gridbook_b200 import kernels, synth
    M, K = 37, 1024
    x = synth.make_activations(M, K, seed=9)
    x[3] = 0.0                                              # an all-zero row
    x[4, :16] = 0.0                                         # a zero group inside a live row
    x[5] *= 2.0 ** -60                                      # tiny
    x[6] *= 2.0 ** 40                                       # huge
    x[7, 16:32] = np.float32(-0.0)
    # exact midpoints between E2M1 rungs once divided by a power-of-two scale factor
    x[8, :16] = np.array([6, 5, 3.5, 2.5, 1.75, 1.25, 0.75, 0.25, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5, -6],
                         np.float32)
    x = synth.bf16_round(x)
    packed, sf, a_scale = kernels.nvfp4_quantize_rows(synth.bf16_tensor(x, dev))
    rp, rs, ra = nvfp4_quantize_rows_ref(x)
    assert np.array_equal(a_scale.cpu().numpy(), ra)
    assert np.array_equal(_unswizzle(sf.cpu().numpy(), M, K // 16), rs)
    assert np.array_equal(packed.cpu().numpy(), rp)
    # the padding rows of the last 128-row tile carry zero scale factors
    plane = sf.cpu().numpy()
    full = plane[O.sf_swizzle_offsets(128, K // 16).reshape(-1)].reshape(128, K // 16)
    assert not full[M:].any()


@pytest.mark.parametrize("M,N,K", [(128, 256, 256), (300, 512, 1024), (77, 384, 768), (1024, 2048, 2048)])
def test_gemm_fp4_against_dequantised_product(dev, M, N, K):
    from gridbook_b200 import _native, kernels, synth
    from gridbook_b200.formats import NVFP4_LITERAL
    d = synth.make_linear(NVFP4_LITERAL, N, K, seed=M + N, global_scale=1.0 / 448.0)
    qw = d["qw"].reshape(N, K // 256, 48)
    qw[::3, :, 32 + 5] |= 0x80                              # some negative group scales
    d["qw"] = qw.reshape(N, -1)
    w = synth.to_device_weight(d, dev)
    x = synth.make_activations(M, K, seed=M)
    a, sfa, a_scale = kernels.nvfp4_quantize_rows(synth.bf16_tensor(x, dev))
    b, sfb = kernels.expand_fp4_nvfp4(w, operand=True)
    y = kernels.gemm_fp4(a, sfa, b, sfb, a_scale=a_scale, global_scale=w.global_scale)
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    xa = nvfp4_dequant(*nvfp4_quantize_rows_ref(x))
    wt = oracle_weight(d)                                   # value * scale, sign included
    ref = (xa.astype(np.float64) @ wt.astype(np.float64).T * (1.0 / 448.0)).astype(np.float32)
    assert_close_bf16(f32_of(y), O.bf16_round(ref), f"gemm_fp4 {M}x{N}x{K}")


@pytest.mark.parametrize("name", ["lit", "k16v2"])
def test_linear_method_prefill_takes_the_block_scaled_route(dev, name):
    from gridbook_b200 import formats as F
    from gridbook_b200 import synth
    from gridbook_b200.linear import CBLinear
    fmt = {"lit": F.NVFP4_LITERAL, "k16v2": F.NVFP4_CB_K16}[name]
    N, K, M = 768, 2048, 640
    gs = 1.0 / 448.0 if name == "lit" else 1.0
    d = synth.make_linear(fmt, N, K, seed=5, global_scale=gs)
    tabs, pos = [], 0
    for r, c in fmt.table_shapes():
        tabs.append(torch.from_numpy(d["cb"][pos:pos + r * c].reshape(r, c).copy()))
        pos += r * c
    lin = CBLinear(fmt, K, [N], [tabs], global_scale=gs).load(torch.from_numpy(d["qw"]), None, dev)
    x = synth.make_activations(M, K, seed=6)
    y = lin(synth.bf16_tensor(x, dev))
    assert "mxf4nvf4" in lin._cb_route["prefill"]
    xa = nvfp4_dequant(*nvfp4_quantize_rows_ref(x))
    # fp64 product of the dequantised activations and the exact weights: two-tier scales span twelve
    # binades, and an fp32 reference sum loses more to cancellation than the tensor cores do
    wt = oracle_weight(d).astype(np.float64)
    ref = O.bf16_round((xa.astype(np.float64) @ wt.T * (d.get("global_scale") or 1.0)).astype(np.float32))
    got = f32_of(y)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-2
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()
    assert_close_bf16(got, ref, f"{name} block-scaled prefill", atol_rel=2e-4)
    # the exact-contract route stays selectable: bucketed bf16 rows x bf16 weights
    lin.method.prefill_route = "bf16"
    y2 = lin(synth.bf16_tensor(x, dev))
    xq = C.act_qdq(x, "fp4", "recip").astype(np.float64)
    ref2 = O.bf16_round((xq @ wt.T * (d.get("global_scale") or 1.0)).astype(np.float32))
    assert_close_bf16(f32_of(y2), ref2, f"{name} bf16 prefill", atol_rel=2e-4)
