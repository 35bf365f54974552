"""Shared helpers of the GPU parity tests (oracle side and comparison rules)."""
import numpy as np
import torch

from oracle import cb_oracle as O
from oracle import oracle_kwargs


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def f32_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def oracle_weight(d):
    fmt = d["fmt"]
    off = d.get("cb_row_offset")
    if off is None:
        off = np.zeros(d["N"], np.int32)
    return O.reconstruct_weight(d["qw"], d["cb"], off, N=d["N"], K=d["K"], compose=d.get("compose"),
                                weight_scale=d.get("weight_scale"), **oracle_kwargs(fmt))


def oracle_linear(x, d, bucket=True, scale_rule="recip"):
    fmt = d["fmt"]
    off = d.get("cb_row_offset")
    if off is None:
        off = np.zeros(d["N"], np.int32)
    xq = O.act_bucket(x, fmt.grid, scale_rule) if bucket else x
    return O.cb_linear(xq, d["qw"], d["cb"], off, N=d["N"], K=d["K"], compose=d.get("compose"),
                       weight_scale=d.get("weight_scale"), global_scale=d.get("global_scale"),
                       **oracle_kwargs(fmt))


def assert_close_bf16(got: np.ndarray, ref: np.ndarray, tag: str, ulps: float = 2.0, rel_l2: float = 1e-3,
                      atol_rel: float = 0.0):
    """The reference's GEMV gate (tests/test_cuda_gemv.py:50-65), which allows one bf16
    output ULP (2^-7 relative + 1e-5) per element plus a relative-L2 backstop of 1e-3.  The
    weights and activations are bit-identical on both sides, only the fp32 summation order
    differs (MMA tiles, K slices added atomically), so a sum that lands next to a rounding
    boundary may move by one more step: two ULPs per element here, the same 1e-3 backstop.
    Both are far inside the acceptance bar of rel-L2 <= 1e-2.  ``atol_rel`` adds an absolute
    allowance of that fraction of the largest reference magnitude, for sums of thousands of
    terms on the tensor cores whose result is small next to its terms (cancellation): the
    fp32 accumulator's error scales with the terms, not with the result."""
    d = np.abs(got - ref)
    tol = np.maximum(np.abs(got), np.abs(ref)) * (2.0 ** -7) * ulps + 1e-5 + atol_rel * float(np.abs(ref).max())
    bad = int((d > tol).sum())
    assert bad == 0, f"{tag}: {bad}/{d.size} elements beyond {ulps} bf16 ULP (max diff {d.max():.3e})"
    rel = np.linalg.norm(d) / max(np.linalg.norm(ref), 1e-6)
    assert rel <= rel_l2, f"{tag}: rel-L2 {rel:.3e} > {rel_l2}"



def assert_linear_close(got, ref, fmt, tag):
    assert_close_bf16(got, ref, tag)


# ---- native NVFP4 activations (the block-scaled prefill's bucket) -------------------------
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def nvfp4_quantize_rows_ref(x: np.ndarray, range_multiplier: float = 448.0):
    """The oracle's NVFP4 activation quantiser (gridbook/codec.py:377-425) with one global scale
    per row, gs = (range * 6) / rowmax in fp32, as the reference's row quantiser picks it
    (gridbook/csrc/cb_fused_fp4_gemm.cu:345-355): -> (packed [M, K/2], sf bytes [M, K/16],
    a_scale [M])."""
    x = np.asarray(x, dtype=np.float32)
    M, K = x.shape
    packed = np.zeros((M, K // 2), np.uint8)
    sf = np.zeros((M, K // 16), np.uint8)
    a_scale = np.zeros(M, np.float32)
    for m in range(M):
        amax = np.abs(x[m]).max()
        live = amax > 0 and np.isfinite(amax)
        gs = (np.float32(range_multiplier) * np.float32(6.0)) / np.float32(amax) if live else np.float32(1.0)
        p, s, _ = O.nvfp4_act_quant(x[m:m + 1], gs)
        packed[m], sf[m] = p[0], s[0]
        a_scale[m] = np.float32(1.0) / np.float32(gs) if live else 0.0
    return packed, sf, a_scale


def nvfp4_dequant(packed: np.ndarray, sf: np.ndarray, a_scale: np.ndarray | None = None) -> np.ndarray:
    """(code * SF) [* a_scale] as fp32 [M, K]."""
    lo, hi = packed & 0xF, packed >> 4
    codes = np.stack([lo, hi], axis=-1).reshape(packed.shape[0], -1)
    vals = E2M1_VALUES[codes & 7] * np.where(codes & 8, -1.0, 1.0).astype(np.float32)
    out = vals * np.repeat(O.e4m3_to_f32(sf), 16, axis=1)
    return out if a_scale is None else out * a_scale[:, None]
