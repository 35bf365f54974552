"""GPU parity of the prefill tensor-core GEMM (tcgen05, accumulator in tensor memory) and of
the prefill routes built on it, through the C ABI.  The floating-point reference is a plain
fp32 matmul of the same operands in torch."""
import numpy as np
import pytest
import torch

from oracle import cb_oracle as O
from tests.helpers import f32_of, oracle_linear

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gridbook_b200 import _native
    _native.prepare(0)
    return torch.device("cuda:0")


def _rel(got, ref):
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-9))


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (256, 384, 512), (200, 136, 1024), (17, 72, 256), (640, 1024, 5120)])
def test_gemm_bf16_matches_fp32_matmul(dev, M, N, K):
    from gridbook_b200 import _native, kernels
    g = torch.Generator(device=dev).manual_seed(M + N)
    a = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, generator=g, device=dev).to(torch.bfloat16)
    d = kernels.gemm_tn(a, b, global_scale=0.5)
    ref = (a.float() @ b.float().t()) * 0.5
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    # one bf16 rounding of an fp32-accumulated sum: tolerance 2^-8 relative per element
    err = (d.float() - ref).abs()
    assert bool((err <= ref.abs() * 2.0 ** -7 + 1e-2).all()), float(err.max())
    assert _rel(f32_of(d), f32_of(ref)) <= 3e-3


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (300, 264, 1024)])
def test_gemm_e4m3_with_scales(dev, M, N, K):
    from gridbook_b200 import kernels
    g = torch.Generator(device=dev).manual_seed(7)
    a = (torch.randn(M, K, generator=g, device=dev) * 4).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, generator=g, device=dev) * 4).to(torch.float8_e4m3fn)
    sa = torch.rand(M, generator=g, device=dev) + 0.5
    sb = (torch.rand(N, generator=g, device=dev) + 0.5) * 0.02
    d = kernels.gemm_tn(a, b, a_scale=sa, b_scale=sb)
    ref = (a.float() @ b.float().t()) * sa[:, None] * sb[None, :]
    assert _rel(f32_of(d), f32_of(ref)) <= 3e-3


def test_fp8_row_quantiser_matches_bucket(dev):
    """q * scale reproduces the per-token activation bucket bit for bit."""
    from gridbook_b200 import kernels, synth
    x = synth.make_activations(9, 768, seed=2)
    q, s = kernels.fp8_quantize_rows(synth.bf16_tensor(x, dev))
    deq = O.bf16_round((O.e4m3_to_f32(q.view(torch.uint8).cpu().numpy()) * s.cpu().numpy()[:, None]).astype(np.float32))
    assert np.array_equal(deq, O.fp8_dynamic_act_qdq(x, "recip"))
