"""Every servable format of the reference's runtime contract (fixture tests/golden/format_rungs.json,
made from gridbook/runtime_contract.json by tests/golden/make_format_rungs.py) is expressible here:
the scheme parses, the superblock size is the reference's, the C ABI's host-side validation accepts
the descriptor (no GPU needed: gb_gemv_row_batch_max only validates and plans), and a wrong
superblock size is refused."""
import ctypes
import json
import os

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
RUNGS = json.load(open(os.path.join(HERE, "golden", "format_rungs.json")))["formats"]


def _scheme(r):
    s = {"grid": r["grid"], "mode": r["mode"], "k": r["k"], "n_sub": r["n_sub"], "type_size": r["type_size"]}
    if r["grid"] == "fp4" and r["layout_version"] == 2:
        s["scale_coding"] = {"kind": "two_tier"}
    return s


def _native_weight(nat, fmt, rows=256, K=1024):
    return nat.GbWeight(qw=16, row_stride=fmt.row_bytes(K), codebook=16, cb_row_offset=None,
                        compose=16 if fmt.scale_coding == "v2" else None,
                        weight_scale=None if fmt.is_fp4 else 16, global_scale=1.0, rows=rows, K=K,
                        fmt=fmt.to_native())


@pytest.mark.parametrize("r", RUNGS, ids=[f"{r['name']}-v{r['layout_version']}" for r in RUNGS])
def test_reference_format_rung_is_expressible_and_validates(r):
    from gridbook_b200 import _native as nat
    from gridbook_b200.formats import CBFormat
    fmt = CBFormat.from_scheme(_scheme(r))
    assert fmt.type_size == r["type_size"] == fmt.packed_type_size
    assert fmt.mode == r["mode"] and fmt.n_sub == r["n_sub"] and fmt.k == r["k"]
    lib = nat.load()
    w = _native_weight(nat, fmt)
    if r["mode"] == "signed" and r["k"] >= 23:
        # the two widest signed rungs (magnitude tables of 512 KiB and 1 MiB) are not served: refused
        # at the boundary with a reason, never decoded wrongly
        assert lib.gb_gemv_row_batch_max(ctypes.byref(w)) == 0 and b"signed mode" in lib.gb_last_error()
        return
    assert lib.gb_gemv_row_batch_max(ctypes.byref(w)) >= 16, lib.gb_last_error()
    bad = _native_weight(nat, fmt)
    bad.fmt.type_size = r["type_size"] - 1
    assert lib.gb_gemv_row_batch_max(ctypes.byref(bad)) == 0


def test_row_batch_limits_of_the_formats_the_tensor_core_decode_kernel_serves():
    """Host-side planning: how many rows each served format gets (what its rings and tables leave of
    the shared memory for four activation stages), 16 for everything else."""
    from gridbook_b200 import _native as nat
    from gridbook_b200 import formats as F
    lib = nat.load()
    want = [(F.NVFP4_LITERAL, 128), (F.NVFP4_CB_K16.padded(80), 96), (F.NVFP4_CB_K16, 16), (F.FP8_CB_K32, 80),
            (F.FP8_LITERAL, 96), (F.CBFormat("fp8", 30, n_sub=4), 16), (F.CBFormat("fp4", 13, mode="signed", scale_coding="v2"), 16)]
    for fmt, rows in want:
        w = _native_weight(nat, fmt)
        assert lib.gb_gemv_row_batch_max(ctypes.byref(w)) == rows, (fmt, rows)
    small = _native_weight(nat, F.NVFP4_LITERAL, rows=64)           # fewer than 128 weight rows: not served
    assert lib.gb_gemv_row_batch_max(ctypes.byref(small)) == 16
