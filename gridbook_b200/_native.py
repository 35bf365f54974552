"""ctypes loader for libgridbook_b200.so — the only route to the kernels.

Replaces the reference's JIT loader (gridbook/cuda_ext.py:344-431,446-522): one
prebuilt library, a strict required-symbol list, and the same fail-closed rule.
A missing library or symbol raises :class:`NativeKernelUnavailableError`
(gridbook/cuda_ext.py:107-113); there is no CPU or eager fallback anywhere.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

GB_ABI_VERSION = 3
GEMM_BF16, GEMM_E4M3 = 0, 1

REQUIRED_SYMBOLS = (
    "gb_abi_version", "gb_last_error", "gb_prepare", "gb_device_status", "gb_gemv_row_batch_max",
    "gb_fp8_act_qdq", "gb_fp4_act_qdq",
    "gb_expand_fp8", "gb_expand_fp4_bf16", "gb_expand_fp4_nvfp4",
    "gb_gemv_workspace_bytes", "gb_gemv", "gb_gemv_static",
    "gb_gemv_tab_slots_bytes", "gb_gemv_tab_arm", "gb_gemv_tab", "gb_device_status_reset", "gb_set_wait_limit_ms",
    "gb_set_row_routes", "gb_nvfp4_sf_bytes", "gb_nvfp4_quantize_rows", "gb_gemm_fp4",
    "gb_moe_route", "gb_moe_route_ws", "gb_moe_route_workspace_bytes", "gb_moe_gemv_workspace_bytes", "gb_moe_gemv", "gb_moe_combine",
    "gb_moe_gemv_pairs_workspace_bytes", "gb_moe_gemv_pairs",
    "gb_moe_mlp_pairs_workspace_bytes", "gb_moe_mlp_pairs",
    "gb_expand_fp8_bf16", "gb_fp8_quantize_rows", "gb_gemm_tn", "gb_gemm_tn_grouped", "gb_moe_gather_rows", "gb_moe_swiglu_rows", "gb_moe_gemv_sorted",
    "gb_peer_alloc", "gb_peer_free", "gb_peer_export", "gb_peer_open", "gb_peer_close",
    "gb_peer_allgather", "gb_peer_allgather_ll", "gb_peer_barrier", "gb_launch_count", "gb_gemv_allgather", "gb_moe_combine_peer",
)
PEER_MAX, PEER_HANDLE_BYTES, PEER_FLAG_BYTES = 8, 64, 128

OK, EINVAL, ECUDA, EUNSUPPORTED, EWORKSPACE = 0, 1, 2, 3, 4       # status codes of the C ABI
GRID_FP4, GRID_FP8 = 0, 1
MODE_PRODUCT, MODE_SIGNED, MODE_FULL = 0, 1, 2
SCALE_NONE, SCALE_V1, SCALE_V2 = 0, 1, 2
SCALE_RULE_RECIP, SCALE_RULE_DIV = 0, 1
ACT_NONE, ACT_FP4_GROUP16, ACT_FP8_TOKEN = 0, 1, 2


class NativeKernelUnavailableError(RuntimeError):
    """The compiled sm_100a library (or one of its entry points) is missing."""


class StaleExtensionError(NativeKernelUnavailableError):
    """The library on disk does not match this package's ABI version."""


class GbFormat(ctypes.Structure):
    _fields_ = [("grid", ctypes.c_int32), ("mode", ctypes.c_int32),
                ("k_bits", ctypes.c_int32), ("n_sub", ctypes.c_int32),
                ("type_size", ctypes.c_int32), ("scale_coding", ctypes.c_int32)]


class GbWeight(ctypes.Structure):
    _fields_ = [("qw", ctypes.c_void_p), ("row_stride", ctypes.c_int64),
                ("codebook", ctypes.c_void_p), ("cb_row_offset", ctypes.c_void_p),
                ("compose", ctypes.c_void_p), ("weight_scale", ctypes.c_void_p),
                ("global_scale", ctypes.c_float), ("rows", ctypes.c_int64),
                ("K", ctypes.c_int64), ("fmt", GbFormat)]


class GbPeerGroup(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("flags", ctypes.c_void_p * 8)]


class GbPeerPiece(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst", ctypes.c_void_p * 8), ("rows", ctypes.c_int64),
                ("row_bytes", ctypes.c_int64), ("src_pitch", ctypes.c_int64), ("dst_pitch", ctypes.c_int64)]


class GbPeerLLPiece(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst_local", ctypes.c_void_p * 8), ("rows", ctypes.c_int64),
                ("row_bytes", ctypes.c_int64), ("src_pitch", ctypes.c_int64), ("dst_pitch", ctypes.c_int64)]


class GbGatherLayout(ctypes.Structure):
    _fields_ = [("n_roles", ctypes.c_int32), ("lcol", ctypes.c_int64 * 4), ("gcol0", ctypes.c_int64 * 4),
                ("width", ctypes.c_int64 * 4)]


class GbPeerRows(ctypes.Structure):
    _fields_ = [("base", ctypes.c_void_p * 8), ("rows_per_rank", ctypes.c_int64)]


_LOCK = threading.Lock()
_LIB = None
_PREPARED: set[int] = set()


def library_path() -> str:
    override = os.environ.get("GRIDBOOK_B200_LIB")
    if override:
        return override
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "libgridbook_b200.so")


def _declare(lib) -> None:
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    wp = ctypes.POINTER(GbWeight)
    lib.gb_abi_version.restype = i32
    lib.gb_last_error.restype = ctypes.c_char_p
    lib.gb_prepare.argtypes = [i32]
    lib.gb_gemv_row_batch_max.argtypes = [ctypes.POINTER(GbWeight)]
    lib.gb_gemv_row_batch_max.restype = i32
    lib.gb_device_status.argtypes = [i32, ctypes.POINTER(ctypes.c_int)]
    lib.gb_fp8_act_qdq.argtypes = [vp, vp, i64, i64, i32, vp]
    lib.gb_fp4_act_qdq.argtypes = [vp, vp, i64, i64, i32, vp]
    lib.gb_expand_fp8.argtypes = [wp, i64, i64, vp, vp]
    lib.gb_expand_fp4_bf16.argtypes = [wp, i64, i64, vp, vp]
    lib.gb_expand_fp8_bf16.argtypes = [wp, i64, i64, vp, vp]
    lib.gb_expand_fp4_nvfp4.argtypes = [wp, i64, i64, vp, vp, i32, vp]
    lib.gb_gemv_workspace_bytes.argtypes = [i64, i64, i64]
    lib.gb_gemv_workspace_bytes.restype = i64
    lib.gb_gemv.argtypes = [vp, i64, wp, i32, i32, vp, vp, i64, vp]
    lib.gb_gemv_static.argtypes = [vp, i64, wp, i32, i32, vp, vp]
    wpp = ctypes.POINTER(wp)
    lib.gb_gemv_tab_slots_bytes.argtypes = [wpp, i32]
    lib.gb_gemv_tab_slots_bytes.restype = i64
    lib.gb_gemv_tab_arm.argtypes = [vp, i64, vp]
    lib.gb_gemv_tab.argtypes = [vp, wpp, ctypes.POINTER(vp), i32, i32, i32, vp, i64, vp]
    lib.gb_nvfp4_sf_bytes.argtypes = [i64, i64]
    lib.gb_nvfp4_sf_bytes.restype = i64
    lib.gb_nvfp4_quantize_rows.argtypes = [vp, i64, i64, ctypes.c_float, vp, vp, vp, vp]
    lib.gb_gemm_fp4.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, vp, ctypes.c_float, vp]
    lib.gb_set_row_routes.argtypes = [i32, i32]
    lib.gb_device_status_reset.argtypes = [i32]
    lib.gb_set_wait_limit_ms.argtypes = [i32]
    lib.gb_moe_route.argtypes = [vp, i64, i64, i64, i64, vp, vp, vp, vp, vp, vp]
    lib.gb_moe_route_ws.argtypes = [vp, i64, i64, i64, i64, vp, vp, vp, vp, vp, vp, i64, vp]
    lib.gb_moe_route_workspace_bytes.argtypes = [i64, i64, i64]
    lib.gb_moe_route_workspace_bytes.restype = i64
    lib.gb_moe_gemv_workspace_bytes.argtypes = [i64, i64]
    lib.gb_moe_gemv_workspace_bytes.restype = i64
    lib.gb_moe_gemv.argtypes = [vp, vp, wp, i64, i64, vp, vp, i64, i32, i32, i32, vp, vp, vp, i64, vp]
    lib.gb_moe_combine.argtypes = [vp, vp, vp, i64, i64, i64, i64, i32, vp, vp]
    lib.gb_moe_gemv_pairs_workspace_bytes.argtypes = [i64, i64, i64]
    lib.gb_moe_gemv_pairs_workspace_bytes.restype = i64
    lib.gb_moe_mlp_pairs_workspace_bytes.argtypes = [i64, i64, i64]
    lib.gb_moe_mlp_pairs_workspace_bytes.restype = i64
    lib.gb_moe_mlp_pairs.argtypes = [vp, vp, wp, i64, wp, i64, i64, i64, vp, i64, i64, i32, i32, vp, vp, vp, i64, vp]
    lib.gb_moe_gemv_pairs.argtypes = [vp, vp, wp, i64, i64, i64, vp, i64, i64, i32, i32, i32, vp, vp, vp, i64, vp]
    lib.gb_fp8_quantize_rows.argtypes = [vp, vp, vp, i64, i64, i32, vp]
    lib.gb_gemm_tn.argtypes = [vp, vp, vp, i64, i64, i64, i32, vp, vp, ctypes.c_float, vp]
    lib.gb_gemm_tn_grouped.argtypes = [vp, vp, vp, i64, i64, i64, i32, i64, vp, vp, vp, vp, ctypes.c_float, vp]
    lib.gb_moe_gather_rows.argtypes = [vp, vp, vp, vp, i64, i64, i64, vp, vp]
    lib.gb_moe_gemv_sorted.argtypes = [vp, wp, i64, i64, vp, vp, i64, vp, vp, vp]
    lib.gb_moe_swiglu_rows.argtypes = [vp, vp, i64, i64, i64, i32, i32, vp, vp]
    lib.gb_launch_count.restype = i64
    lib.gb_peer_alloc.argtypes = [i64, ctypes.POINTER(vp)]
    lib.gb_peer_free.argtypes = [vp]
    lib.gb_peer_export.argtypes = [vp, vp]
    lib.gb_peer_open.argtypes = [vp, ctypes.POINTER(vp)]
    lib.gb_peer_close.argtypes = [vp]
    lib.gb_peer_allgather.argtypes = [ctypes.POINTER(GbPeerGroup), ctypes.POINTER(GbPeerPiece), i32, vp]
    lib.gb_peer_barrier.argtypes = [ctypes.POINTER(GbPeerGroup), vp]
    lib.gb_moe_combine_peer.argtypes = [vp, vp, vp, i64, i64, i64, i64, i32, vp, ctypes.POINTER(GbPeerGroup), vp]
    lib.gb_gemv_allgather.argtypes = [vp, wp, i32, i32, ctypes.POINTER(GbPeerGroup), ctypes.POINTER(vp), i64,
                                      ctypes.POINTER(GbGatherLayout), vp, vp, i64, vp]
    lib.gb_peer_allgather_ll.argtypes = [ctypes.POINTER(GbPeerGroup), ctypes.POINTER(vp), i64,
                                         ctypes.POINTER(GbPeerLLPiece), i32, vp]
    for name in REQUIRED_SYMBOLS:
        fn = getattr(lib, name)
        if fn.restype is ctypes.c_int:
            fn.restype = i32


def load(what: str = "gridbook_b200 kernels"):
    """Return the loaded library or raise NativeKernelUnavailableError."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not os.path.exists(path):
            raise NativeKernelUnavailableError(
                f"[prismaquant-cb] {what}: {path} is missing. Build it with "
                "`python -m gridbook_b200.build`; there is no fallback path.")
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise NativeKernelUnavailableError(
                f"[prismaquant-cb] {what}: cannot load {path}: {exc}") from exc
        missing = [s for s in REQUIRED_SYMBOLS if not hasattr(lib, s)]
        if missing:
            raise StaleExtensionError(
                f"[prismaquant-cb] {what}: {path} lacks required symbols {missing}; rebuild it")
        _declare(lib)
        got = lib.gb_abi_version()
        if got != GB_ABI_VERSION:
            raise StaleExtensionError(
                f"[prismaquant-cb] {what}: {path} has ABI version {got}, this package "
                f"wants {GB_ABI_VERSION}; rebuild it")
        _LIB = lib
        return lib


def check(rc: int, lib=None) -> None:
    if rc != 0:
        lib = lib or load()
        raise RuntimeError(f"gridbook_b200: {lib.gb_last_error().decode()} (status {rc})")


def prepare(device: int | torch.device | None = None) -> None:
    """One-time per-device set-up; call at model load, never inside a capture."""
    lib = load()
    if device is None:
        device = torch.cuda.current_device()
    if isinstance(device, torch.device):
        device = device.index if device.index is not None else torch.cuda.current_device()
    if device in _PREPARED:
        return
    with _LOCK:
        if device in _PREPARED:
            return
        check(lib.gb_prepare(int(device)), lib)
        _PREPARED.add(device)


def launch_count() -> int:
    """Kernel launches the library has issued so far in this process."""
    return int(load("launch counter").gb_launch_count())


def device_status(device: int = 0) -> int:
    lib = load()
    out = ctypes.c_int(0)
    check(lib.gb_device_status(int(device), ctypes.byref(out)), lib)
    return out.value


def device_status_reset(device: int = 0) -> None:
    lib = load()
    check(lib.gb_device_status_reset(int(device)), lib)


def set_wait_limit_ms(ms: int) -> None:
    """Test hook: how long the exchange kernels and the one-launch table GEMV spin before a wait
    gives up (0 restores the default of two seconds)."""
    lib = load()
    check(lib.gb_set_wait_limit_ms(int(ms)), lib)


def set_row_routes(dot_rows: int = 0, umma_min: int = 0) -> None:
    """Row counts at which the dense decode entry changes kernel for the literal format (0 = default)."""
    lib = load()
    check(lib.gb_set_row_routes(int(dot_rows), int(umma_min)), lib)


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream
