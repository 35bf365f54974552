"""Shared helpers of the GPU parity tests (oracle side and comparison rules)."""
import numpy as np
import torch

from oracle import cb_oracle as O


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
                                weight_scale=d.get("weight_scale"), **fmt.oracle_kwargs())


def oracle_linear(x, d, bucket=True, scale_rule="recip"):
    fmt = d["fmt"]
    off = d.get("cb_row_offset")
    if off is None:
        off = np.zeros(d["N"], np.int32)
    xq = O.act_bucket(x, fmt.grid, scale_rule) if bucket else x
    return O.cb_linear(xq, d["qw"], d["cb"], off, N=d["N"], K=d["K"], compose=d.get("compose"),
                       weight_scale=d.get("weight_scale"), global_scale=d.get("global_scale"),
                       **fmt.oracle_kwargs())


def assert_close_bf16(got: np.ndarray, ref: np.ndarray, tag: str, ulps: float = 2.0, rel_l2: float = 1e-3):
    """The reference's GEMV gate (tests/test_cuda_gemv.py:50-65), which allows one bf16
    output ULP (2^-7 relative + 1e-5) per element plus a relative-L2 backstop of 1e-3.  The
    weights and activations are bit-identical on both sides, only the fp32 summation order
    differs (MMA tiles, K slices added atomically), so a sum that lands next to a rounding
    boundary may move by one more step: two ULPs per element here, the same 1e-3 backstop.
    Both are far inside the acceptance bar of rel-L2 <= 1e-2."""
    d = np.abs(got - ref)
    tol = np.maximum(np.abs(got), np.abs(ref)) * (2.0 ** -7) * ulps + 1e-5
    bad = int((d > tol).sum())
    assert bad == 0, f"{tag}: {bad}/{d.size} elements beyond {ulps} bf16 ULP (max diff {d.max():.3e})"
    rel = np.linalg.norm(d) / max(np.linalg.norm(ref), 1e-6)
    assert rel <= rel_l2, f"{tag}: rel-L2 {rel:.3e} > {rel_l2}"



def assert_linear_close(got, ref, fmt, tag):
    assert_close_bf16(got, ref, tag)
