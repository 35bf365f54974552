"""Tensor-level wrappers over the C ABI: build a ``gb_weight`` from torch tensors,
pass raw pointers and the current stream, turn a non-zero status into
RuntimeError.  Every function here launches CUDA work or raises; none computes
on the host."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _native as nat
from .formats import CBFormat

_ZERO = ctypes.c_void_p(0)


def _ptr(t: torch.Tensor | None):
    return _ZERO if t is None else ctypes.c_void_p(t.data_ptr())


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("gridbook_b200 kernels take CUDA tensors only (no CPU path exists)")


@dataclass
class PackedWeight:
    """One packed matrix (or one expert's matrix of a stack) as the kernels see it."""
    qw: torch.Tensor                      # uint8 [rows, >= row_bytes] (or [E, rows, bytes])
    codebook: torch.Tensor                # bf16 flat (fp4) / uint8 E4M3 flat (fp8)
    fmt: CBFormat
    K: int
    rows: int
    row_stride: int
    cb_row_offset: torch.Tensor | None = None   # int32 [rows]
    compose: torch.Tensor | None = None         # fp32 [4096], v2 only
    weight_scale: torch.Tensor | None = None    # fp32 [rows] (or [E, rows]), fp8 only
    global_scale: float = 1.0
    expert_stride: int = 0
    experts: int = 1

    def native(self) -> nat.GbWeight:
        return nat.GbWeight(
            qw=self.qw.data_ptr(), row_stride=self.row_stride,
            codebook=self.codebook.data_ptr(),
            cb_row_offset=None if self.cb_row_offset is None else self.cb_row_offset.data_ptr(),
            compose=None if self.compose is None else self.compose.data_ptr(),
            weight_scale=None if self.weight_scale is None else self.weight_scale.data_ptr(),
            global_scale=float(self.global_scale), rows=self.rows, K=self.K,
            fmt=self.fmt.to_native())

    @property
    def packed_bytes(self) -> int:
        """Algorithmic weight-stream bytes of one pass over this matrix (all experts)."""
        return self.experts * self.rows * self.fmt.packed_row_bytes(self.K)


def make_weight(qw, codebook, fmt: CBFormat, K: int, *, cb_row_offset=None, compose=None,
                weight_scale=None, global_scale: float = 1.0) -> PackedWeight:
    _need_cuda(qw, codebook, cb_row_offset, compose, weight_scale)
    if qw.dtype is not torch.uint8 or qw.stride(-1) != 1:
        raise RuntimeError("packed weights must be uint8 with a unit inner stride")
    if fmt.is_fp4:
        if codebook.dtype is not torch.bfloat16:
            raise RuntimeError("fp4-grid codebooks are bf16 flat tables")
        if fmt.scale_coding == "v2" and compose is None:
            raise RuntimeError("two-tier scale coding needs the compose table")
    else:
        if codebook.dtype is not torch.uint8:
            raise RuntimeError("fp8-grid codebooks are E4M3 bytes")
        if weight_scale is None:
            raise RuntimeError("fp8-grid weights need weight_scale")
    if qw.dim() == 3:
        experts, rows = qw.shape[0], qw.shape[1]
        return PackedWeight(qw, codebook, fmt, K, rows, qw.stride(1), cb_row_offset, compose,
                            weight_scale, global_scale, qw.stride(0), experts)
    return PackedWeight(qw, codebook, fmt, K, qw.shape[0], qw.stride(0), cb_row_offset, compose,
                        weight_scale, global_scale)


def _rule(scale_rule: str) -> int:
    return nat.SCALE_RULE_DIV if scale_rule == "div" else nat.SCALE_RULE_RECIP


def fp4_act_qdq(x: torch.Tensor, scale_rule: str = "recip") -> torch.Tensor:
    _need_cuda(x)
    lib = nat.load("FP4 activation QDQ")
    if x.dtype is not torch.bfloat16:
        raise TypeError("native FP4 activation QDQ requires CUDA BF16")
    if x.shape[-1] % 16:
        raise RuntimeError("fp4_act_qdq needs a last dim that is a multiple of the fp4 group (16)")
    x = x.contiguous()
    out = torch.empty_like(x)
    K = x.shape[-1]
    nat.check(lib.gb_fp4_act_qdq(_ptr(x), _ptr(out), x.numel() // K, K, _rule(scale_rule),
                                 nat.stream_ptr(x.device)), lib)
    return out


def fp8_act_qdq(x: torch.Tensor, scale_rule: str = "recip") -> torch.Tensor:
    _need_cuda(x)
    lib = nat.load("FP8 activation QDQ")
    if x.dtype is not torch.bfloat16:
        raise TypeError("native FP8 activation QDQ requires CUDA BF16")
    x = x.contiguous()
    out = torch.empty_like(x)
    K = x.shape[-1]
    nat.check(lib.gb_fp8_act_qdq(_ptr(x), _ptr(out), x.numel() // K, K, _rule(scale_rule),
                                 nat.stream_ptr(x.device)), lib)
    return out


def expand_fp8(w: PackedWeight, row0: int = 0, nrows: int | None = None) -> torch.Tensor:
    lib = nat.load("FP8-CB transient expansion")
    nrows = w.rows - row0 if nrows is None else nrows
    out = torch.empty((nrows, w.K), dtype=torch.float8_e4m3fn, device=w.qw.device)
    nw = w.native()
    nat.check(lib.gb_expand_fp8(ctypes.byref(nw), row0, nrows, _ptr(out),
                                nat.stream_ptr(w.qw.device)), lib)
    return out


def expand_fp8_bf16(w: PackedWeight, row0: int = 0, nrows: int | None = None) -> torch.Tensor:
    """The served fp8-grid weight bf16(value * row scale) as a [nrows, K] bf16 tile."""
    lib = nat.load("FP8-CB transient expansion to bf16")
    nrows = w.rows - row0 if nrows is None else nrows
    out = torch.empty((nrows, w.K), dtype=torch.bfloat16, device=w.qw.device)
    nw = w.native()
    nat.check(lib.gb_expand_fp8_bf16(ctypes.byref(nw), row0, nrows, _ptr(out),
                                     nat.stream_ptr(w.qw.device)), lib)
    return out


def expand_fp4_bf16(w: PackedWeight, row0: int = 0, nrows: int | None = None) -> torch.Tensor:
    lib = nat.load("FP4-CB transient expansion")
    nrows = w.rows - row0 if nrows is None else nrows
    out = torch.empty((nrows, w.K), dtype=torch.bfloat16, device=w.qw.device)
    nw = w.native()
    nat.check(lib.gb_expand_fp4_bf16(ctypes.byref(nw), row0, nrows, _ptr(out),
                                     nat.stream_ptr(w.qw.device)), lib)
    return out


def expand_fp4_nvfp4(w: PackedWeight, row0: int = 0, nrows: int | None = None,
                     swizzled: bool = False, operand: bool = False):
    """-> (packed E2M1 [nrows, K/2] uint8, E4M3 group scales: [nrows, K/16] or the flat
    128x4-atom plane).  ``operand``: the atom plane in the form the block-scaled MMA takes (a
    negative group scale hands its sign to the group's values)."""
    lib = nat.load("NVFP4 tile expansion")
    nrows = w.rows - row0 if nrows is None else nrows
    dev = w.qw.device
    packed = torch.empty((nrows, w.K // 2), dtype=torch.uint8, device=dev)
    groups = w.K // 16
    swizzled = swizzled or operand
    if swizzled:
        sf = torch.zeros(((nrows + 127) // 128 * 128) * ((groups + 3) // 4 * 4),
                         dtype=torch.uint8, device=dev)
    else:
        sf = torch.empty((nrows, groups), dtype=torch.uint8, device=dev)
    nw = w.native()
    nat.check(lib.gb_expand_fp4_nvfp4(ctypes.byref(nw), row0, nrows, _ptr(packed), _ptr(sf),
                                      2 if operand else (1 if swizzled else 0), nat.stream_ptr(dev)), lib)
    return packed, sf


_ACT = {None: nat.ACT_NONE, "none": nat.ACT_NONE, "fp4": nat.ACT_FP4_GROUP16,
        "fp8": nat.ACT_FP8_TOKEN}


ROW_BATCH_MAX_M = 128      # rows the tensor-core decode kernel of the literal format takes


def row_batch_max_rows(w: PackedWeight) -> int:
    """Most activation rows :func:`gemv` takes for this weight: 16, or up to 128 where the kernel that
    decodes into tensor memory and multiplies on the tensor cores serves the format and layout (the
    library decides)."""
    if w.experts != 1:
        return 16
    cached = w.__dict__.get("_row_batch_max")
    if cached is None:
        nw = w.native()
        cached = int(nat.load("codebook decode GEMV").gb_gemv_row_batch_max(ctypes.byref(nw)))
        w.__dict__["_row_batch_max"] = cached
    return cached


def row_batch_kernel_applies(w: PackedWeight) -> bool:
    """Whether more than 16 activation rows of this weight are served without a decoded transient."""
    return row_batch_max_rows(w) > 16


def gemv(x: torch.Tensor, w: PackedWeight, *, act: str | None = None, scale_rule: str = "recip",
         out: torch.Tensor | None = None, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """y[..., N] = bucket(x)[..., K] . W^T for up to 16 activation rows (up to 128 where
    :func:`row_batch_kernel_applies`)."""
    _need_cuda(x)
    lib = nat.load("codebook decode GEMV")
    if x.dtype is not torch.bfloat16:
        raise TypeError("the decode GEMV takes bf16 activations")
    x2 = x.reshape(-1, w.K).contiguous()
    M = x2.shape[0]
    if out is None:
        out = torch.empty((M, w.rows), dtype=torch.bfloat16, device=x.device)
    need = lib.gb_gemv_workspace_bytes(M, w.rows, w.K)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    nw = w.native()
    nat.check(lib.gb_gemv(_ptr(x2), M, ctypes.byref(nw), _ACT[act], _rule(scale_rule), _ptr(out),
                          _ptr(workspace), workspace.numel(), nat.stream_ptr(x.device)), lib)
    return out.reshape(*x.shape[:-1], w.rows)


def table_kernel_applies(w: PackedWeight) -> bool:
    """Whether ONE activation row of this weight is served by the one-launch table kernel
    (:func:`gemv_tab`): the conditions the library checks."""
    f = w.fmt
    return (f.is_fp4 and f.mode == "full" and f.k == 8 and f.scale_coding == "v1" and w.experts == 1
            and w.cb_row_offset is None and w.rows >= 64 and w.row_stride % 16 == 0
            and w.qw.data_ptr() % 16 == 0 and w.K // 1024 + (1 if w.K % 1024 else 0) <= 148)


def _weight_array(ws):
    natives = [w.native() for w in ws]
    arr = (ctypes.POINTER(nat.GbWeight) * len(ws))(*[ctypes.pointer(n) for n in natives])
    return natives, arr


def new_tab_slots(ws, device=None) -> torch.Tensor:
    """An armed slot buffer (every byte 0xFF) large enough for :func:`gemv_tab` over the weights
    ``ws`` together.  Allocate once per module, or once per stream for modules that run one after
    the other: every call leaves the buffer armed again."""
    lib = nat.load("one-launch table GEMV")
    ws = list(ws)
    _natives, arr = _weight_array(ws)
    need = lib.gb_gemv_tab_slots_bytes(arr, len(ws))
    if need <= 0:
        raise RuntimeError("gemv_tab takes one to four weight matrices")
    return torch.full((need,), 0xFF, dtype=torch.uint8, device=device or ws[0].qw.device)


def gemv_tab(x: torch.Tensor, ws, slots: torch.Tensor, *, act: str | None = "fp4", scale_rule: str = "recip",
             outs=None):
    """One activation row against up to four weights that read it, in ONE launch (literal format):
    -> list of [1, N_i] bf16 outputs, or None when a weight has no such kernel (use :func:`gemv`).
    ``slots`` is an armed buffer from :func:`new_tab_slots`."""
    _need_cuda(x, slots)
    lib = nat.load("one-launch table GEMV")
    if x.dtype is not torch.bfloat16:
        raise TypeError("the table GEMV takes bf16 activations")
    ws = list(ws)
    x2 = x.reshape(-1, ws[0].K).contiguous()
    if x2.shape[0] != 1:
        raise RuntimeError(f"gemv_tab takes exactly one activation row, got {x2.shape[0]}")
    if outs is None:
        outs = [torch.empty((1, w.rows), dtype=torch.bfloat16, device=x.device) for w in ws]
    natives, arr = _weight_array(ws)
    yarr = (ctypes.c_void_p * len(ws))(*[o.data_ptr() for o in outs])
    rc = lib.gb_gemv_tab(_ptr(x2), arr, yarr, len(ws), nat.ACT_FP4_GROUP16 if act == "fp4" else nat.ACT_NONE,
                         _rule(scale_rule), _ptr(slots), slots.numel(), nat.stream_ptr(x.device))
    del natives
    if rc == nat.EUNSUPPORTED:
        return None
    nat.check(rc, lib)
    return outs


def moe_route(topk_ids: torch.Tensor, E: int, topk_weights: torch.Tensor | None = None, *,
              expert_base: int = 0):
    """-> (counts [E], offsets [E+1], order [P]) int32, all on device, no host read.  With
    ``topk_weights`` a fourth result: pair_w [P] fp32, the bf16-rounded router weight of every
    pair and zero for a dropped one, written by the same launch.  ``expert_base``: the E experts
    held here are the global ids [expert_base, expert_base + E); other ids are dropped."""
    _need_cuda(topk_ids, topk_weights)
    lib = nat.load("MoE routing")
    ids = topk_ids.to(torch.int32).contiguous()
    T, topk = ids.shape
    dev = ids.device
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    order = torch.empty(max(T * topk, 1), dtype=torch.int32, device=dev)
    tw = pw = None
    if topk_weights is not None:
        tw = topk_weights.reshape(-1).to(torch.float32).contiguous()
        pw = torch.empty(max(T * topk, 1), dtype=torch.float32, device=dev)
    need = lib.gb_moe_route_workspace_bytes(T, topk, E)       # large batches: tiles over the whole GPU
    ws = torch.empty(need, dtype=torch.uint8, device=dev) if need else None
    nat.check(lib.gb_moe_route_ws(_ptr(ids), T, topk, E, expert_base, _ptr(counts), _ptr(offsets), _ptr(order),
                                  _ptr(tw), _ptr(pw), _ptr(ws), need, nat.stream_ptr(dev)), lib)
    if topk_weights is None:
        return counts, offsets, order[:T * topk]
    return counts, offsets, order[:T * topk], pw[:T * topk]


def moe_gemv(x: torch.Tensor, w: PackedWeight, offsets: torch.Tensor, order: torch.Tensor, *,
             x_row: torch.Tensor | None = None, swiglu: bool = False,
             out: torch.Tensor | None = None, clear: bool = True, peer_rows=None,
             act: str | None = None, scale_rule: str = "recip") -> torch.Tensor | None:
    """Grouped GEMV over the routed pairs; y[p] for pair p (rows/2 wide with swiglu).  Rows of
    pairs that routing dropped are not written: they read zero, or are left unset when
    ``clear`` is False (a caller that hands the dropped ids to :func:`moe_combine`).
    ``peer_rows`` (a ``GbPeerRows``): rows go to their home rank's buffer instead of ``out``.
    ``act="fp4"`` applies the fp4 group-16 bucket to ``x`` inside the kernel."""
    _need_cuda(x, offsets, order, x_row)
    lib = nat.load("grouped codebook decode GEMV")
    if x.dtype is not torch.bfloat16:
        raise TypeError("the grouped decode GEMV takes bf16 activations")
    x = x.contiguous()
    P = order.numel()
    width = w.rows // 2 if swiglu else w.rows
    if out is None and peer_rows is None:
        alloc = torch.zeros if clear else torch.empty
        out = alloc((P, width), dtype=torch.bfloat16, device=x.device)
    nw = w.native()
    nat.check(lib.gb_moe_gemv(_ptr(x), _ptr(x_row), ctypes.byref(nw), w.expert_stride, w.experts,
                              _ptr(offsets), _ptr(order), P, 1 if swiglu else 0,
                              nat.ACT_FP4_GROUP16 if act == "fp4" else nat.ACT_NONE, _rule(scale_rule), _ptr(out),
                              ctypes.byref(peer_rows) if peer_rows is not None else None,
                              _ZERO, 0, nat.stream_ptr(x.device)), lib)
    return out


def moe_gemv_pairs(x: torch.Tensor, w: PackedWeight, pair_expert: torch.Tensor, *,
                   x_row: torch.Tensor | None = None, swiglu: bool = False, act: str | None = None,
                   scale_rule: str = "recip", expert_base: int = 0, pairs_expected: int = 0,
                   peer_rows=None) -> torch.Tensor | None | bool:
    """The routed projection with every pair as its own M = 1 linear through the
    inner-product-table kernel (literal format, small batches).  ``pair_expert`` [P] int32 holds
    each pair's global expert id; ids outside this stack's range are skipped and their output
    rows left unset.  Returns the [P, width] output (True with ``peer_rows``), or None when the
    format has no such kernel and the caller should use :func:`moe_gemv`."""
    _need_cuda(x, pair_expert, x_row)
    lib = nat.load("per-pair table GEMV")
    if x.dtype is not torch.bfloat16:
        raise TypeError("the per-pair GEMV takes bf16 activations")
    x = x.contiguous()
    ids = pair_expert.reshape(-1).to(torch.int32).contiguous()
    P = ids.numel()
    width = w.rows // 2 if swiglu else w.rows
    out = None if peer_rows is not None else torch.empty((P, width), dtype=torch.bfloat16, device=x.device)
    need = lib.gb_moe_gemv_pairs_workspace_bytes(P, w.rows, w.K)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    nw = w.native()
    rc = lib.gb_moe_gemv_pairs(_ptr(x), _ptr(x_row), ctypes.byref(nw), w.expert_stride, w.experts, expert_base,
                               _ptr(ids), P, pairs_expected, 1 if swiglu else 0,
                               nat.ACT_FP4_GROUP16 if act == "fp4" else nat.ACT_NONE, _rule(scale_rule), _ptr(out),
                               ctypes.byref(peer_rows) if peer_rows is not None else None,
                               _ptr(ws), ws.numel(), nat.stream_ptr(x.device))
    if rc == nat.EUNSUPPORTED:
        return None
    nat.check(rc, lib)
    return True if peer_rows is not None else out


def pair_kernel_applies(w: PackedWeight) -> bool:
    """Whether the stack is of the literal fp4 format, the one the per-pair table kernel serves."""
    f = w.fmt
    return f.is_fp4 and f.mode == "full" and f.k == 8 and f.scale_coding == "v1" and f.type_size == 48


def moe_mlp_pairs(x: torch.Tensor, w13: PackedWeight, w2: PackedWeight, pair_expert: torch.Tensor, *,
                  x_row: torch.Tensor | None = None, act: str | None = "fp4", scale_rule: str = "recip",
                  expert_base: int = 0, pairs_expected: int = 0, peer_rows=None):
    """Both projections of the routed MLP for small batches of the literal format, two launches
    (see :func:`moe_gemv_pairs`): y[p] = W2[e_p] . bucket(silu(gate) * up) with gate/up =
    W13[e_p] . bucket(x[x_row[p]]).  Returns [P, hidden] (True with ``peer_rows``), or None when
    the formats have no such kernel."""
    _need_cuda(x, pair_expert, x_row)
    lib = nat.load("per-pair table MLP")
    if x.dtype is not torch.bfloat16:
        raise TypeError("the per-pair MLP takes bf16 activations")
    x = x.contiguous()
    ids = pair_expert.reshape(-1).to(torch.int32).contiguous()
    P = ids.numel()
    out = None if peer_rows is not None else torch.empty((P, w2.rows), dtype=torch.bfloat16, device=x.device)
    need = lib.gb_moe_mlp_pairs_workspace_bytes(P, w13.K, w2.K)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    n13, n2 = w13.native(), w2.native()
    rc = lib.gb_moe_mlp_pairs(_ptr(x), _ptr(x_row), ctypes.byref(n13), w13.expert_stride, ctypes.byref(n2),
                              w2.expert_stride, w13.experts, expert_base, _ptr(ids), P, pairs_expected,
                              nat.ACT_FP4_GROUP16 if act == "fp4" else nat.ACT_NONE, _rule(scale_rule), _ptr(out),
                              ctypes.byref(peer_rows) if peer_rows is not None else None,
                              _ptr(ws), ws.numel(), nat.stream_ptr(x.device))
    if rc == nat.EUNSUPPORTED:
        return None
    nat.check(rc, lib)
    return True if peer_rows is not None else out


def moe_combine(y: torch.Tensor, pair_w: torch.Tensor, T: int, topk: int, *,
                topk_ids: torch.Tensor | None = None, E: int = 0, round_weights: bool = False,
                peer_group=None) -> torch.Tensor:
    """out[t] = sum_slot pair_w * y, fp32 accumulate, one bf16 rounding.  ``topk_ids`` (int32,
    with ``E``) names the pairs routing dropped, whose rows of ``y`` are then never read.
    ``round_weights``: ``pair_w`` are raw router weights, rounded to bf16 inside the kernel.
    ``peer_group`` (a ``GbPeerGroup``): the launch first exchanges "stores visible" flags with the
    other ranks, whose down projections wrote the rows of ``y``."""
    _need_cuda(y, pair_w, topk_ids)
    lib = nat.load("grouped CB router combine")
    y = y.contiguous()
    H = y.shape[-1]
    out = torch.empty((T, H), dtype=torch.bfloat16, device=y.device)
    pw = pair_w.reshape(-1).to(torch.float32).contiguous()
    ids = None
    if topk_ids is not None:
        ids = topk_ids.to(torch.int32).contiguous()
    if peer_group is not None:
        nat.check(lib.gb_moe_combine_peer(_ptr(y), _ptr(pw), _ptr(ids), E, T, topk, H, 1 if round_weights else 0,
                                          _ptr(out), ctypes.byref(peer_group), nat.stream_ptr(y.device)), lib)
        return out
    nat.check(lib.gb_moe_combine(_ptr(y), _ptr(pw), _ptr(ids), E, T, topk, H, 1 if round_weights else 0,
                                 _ptr(out), nat.stream_ptr(y.device)), lib)
    return out


def fp8_quantize_rows(x: torch.Tensor, scale_rule: str = "recip"):
    """Per-token E4M3 quantisation: (q [M, K] float8_e4m3fn, scale [M] fp32), x ~ q * scale."""
    _need_cuda(x)
    lib = nat.load("FP8 activation quantisation")
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    M, K = x2.shape
    q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    nat.check(lib.gb_fp8_quantize_rows(_ptr(x2), _ptr(q), _ptr(scale), M, K, _rule(scale_rule),
                                       nat.stream_ptr(x.device)), lib)
    return q.view(torch.float8_e4m3fn), scale


NVFP4_ACT_RANGE = 448.0      # a row's largest group scale factor: the top of the UE4M3 range


def nvfp4_quantize_rows(x: torch.Tensor, range_multiplier: float = NVFP4_ACT_RANGE):
    """Native NVFP4 quantisation of bf16 rows: (packed [M, K/2] uint8, scale-factor plane in the
    128x4 atom layout uint8, a_scale [M] fp32), x ~ a_scale * SF * E2M1."""
    _need_cuda(x)
    lib = nat.load("NVFP4 activation quantisation")
    if x.dtype is not torch.bfloat16:
        raise TypeError("the NVFP4 quantiser takes bf16 rows")
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    M, K = x2.shape
    packed = torch.empty((M, K // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty(lib.gb_nvfp4_sf_bytes(M, K), dtype=torch.uint8, device=x.device)
    a_scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    nat.check(lib.gb_nvfp4_quantize_rows(_ptr(x2), M, K, float(range_multiplier), _ptr(packed), _ptr(sf),
                                         _ptr(a_scale), nat.stream_ptr(x.device)), lib)
    return packed, sf, a_scale


def gemm_fp4(a_packed: torch.Tensor, sfa: torch.Tensor, b_packed: torch.Tensor, sfb: torch.Tensor, *,
             a_scale: torch.Tensor | None = None, global_scale: float = 1.0) -> torch.Tensor:
    """bf16 D[M, N] = global_scale * a_scale[m] * (A SFA)(B SFB)^T on the block-scaled FP4 tensor
    cores (tcgen05 kind::mxf4nvf4); operands packed E2M1 [rows, K/2], scale planes in the atom layout."""
    _need_cuda(a_packed, sfa, b_packed, sfb, a_scale)
    lib = nat.load("block-scaled FP4 GEMM")
    a_packed, b_packed = a_packed.contiguous(), b_packed.contiguous()
    M, kb = a_packed.shape
    N = b_packed.shape[0]
    if b_packed.shape[1] != kb:
        raise RuntimeError(f"gemm_fp4: K mismatch {2 * kb} vs {2 * b_packed.shape[1]}")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=a_packed.device)
    nat.check(lib.gb_gemm_fp4(_ptr(a_packed), _ptr(sfa), _ptr(b_packed), _ptr(sfb), _ptr(out), M, N, 2 * kb,
                              _ptr(a_scale), float(global_scale), nat.stream_ptr(a_packed.device)), lib)
    return out


def gemm_tn(a: torch.Tensor, b: torch.Tensor, *, a_scale=None, b_scale=None, global_scale: float = 1.0):
    """bf16 D[M, N] = scales * A[M, K] . B[N, K]^T on the tcgen05 tensor cores; A and B both bf16
    or both float8_e4m3fn."""
    _need_cuda(a, b, a_scale, b_scale)
    lib = nat.load("prefill tensor-core GEMM")
    if a.dtype is not b.dtype or a.dtype not in (torch.bfloat16, torch.float8_e4m3fn):
        raise TypeError("gemm_tn takes two bf16 or two float8_e4m3fn operands")
    a, b = a.contiguous(), b.contiguous()
    M, K = a.shape
    N = b.shape[0]
    if b.shape[1] != K:
        raise RuntimeError(f"gemm_tn: K mismatch {K} vs {b.shape[1]}")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    kind = nat.GEMM_BF16 if a.dtype is torch.bfloat16 else nat.GEMM_E4M3
    nat.check(lib.gb_gemm_tn(_ptr(a), _ptr(b), _ptr(out), M, N, K, kind, _ptr(a_scale), _ptr(b_scale),
                             float(global_scale), nat.stream_ptr(a.device)), lib)
    return out


def gemm_tn_grouped(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, n_per_expert: int, *,
                    row_map: torch.Tensor | None = None, a_scale=None, b_scale=None,
                    global_scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped GEMM over expert segments: ``a`` [P, K] rows sorted by expert (expert e owns rows
    ``offsets[e]:offsets[e+1]``), ``b`` [E * n_per_expert, K] the decoded stack; -> [P, n_per_expert]
    bf16, row j at ``row_map[j]`` (or j).  Rows past ``offsets[E]`` are left unwritten."""
    _need_cuda(a, b, offsets, row_map, a_scale, b_scale)
    lib = nat.load("grouped prefill tensor-core GEMM")
    if a.dtype is not b.dtype or a.dtype not in (torch.bfloat16, torch.float8_e4m3fn):
        raise TypeError("gemm_tn_grouped takes two bf16 or two float8_e4m3fn operands")
    a, b = a.contiguous(), b.contiguous()
    P, K = a.shape
    E = offsets.numel() - 1
    if b.shape != (E * n_per_expert, K):
        raise RuntimeError(f"gemm_tn_grouped: decoded stack is {tuple(b.shape)}, expected {(E * n_per_expert, K)}")
    if out is None:
        out = torch.empty((P, n_per_expert), dtype=torch.bfloat16, device=a.device)
    kind = nat.GEMM_BF16 if a.dtype is torch.bfloat16 else nat.GEMM_E4M3
    nat.check(lib.gb_gemm_tn_grouped(_ptr(a), _ptr(b), _ptr(out), P, n_per_expert, K, kind, E, _ptr(offsets),
                                     _ptr(row_map), _ptr(a_scale), _ptr(b_scale), float(global_scale),
                                     nat.stream_ptr(a.device)), lib)
    return out


def moe_gather_rows(x: torch.Tensor, order: torch.Tensor, offsets: torch.Tensor, *,
                    x_row: torch.Tensor | None = None) -> torch.Tensor:
    """The routed rows of ``x`` [T, K] bf16 in expert order: out[j] = x[x_row[order[j]]] for
    j < offsets[E]; later rows are left unset."""
    _need_cuda(x, order, offsets, x_row)
    lib = nat.load("routed row gather")
    if x.dtype is not torch.bfloat16:
        raise TypeError("moe_gather_rows takes bf16 rows")
    x = x.contiguous()
    P, K = order.numel(), x.shape[-1]
    out = torch.empty((P, K), dtype=torch.bfloat16, device=x.device)
    nat.check(lib.gb_moe_gather_rows(_ptr(x), _ptr(x_row), _ptr(order), _ptr(offsets), offsets.numel() - 1, P, K,
                                     _ptr(out), nat.stream_ptr(x.device)), lib)
    return out


def moe_swiglu_rows(h: torch.Tensor, offsets: torch.Tensor, *, act: str | None = None,
                    scale_rule: str = "recip") -> torch.Tensor:
    """bf16 silu(gate) * up over the sorted rows: h [P, 2I] -> [P, I] (rows past offsets[E] unset).
    ``act="fp4"`` also applies the fp4 group-16 bucket to the result in the same launch."""
    _need_cuda(h, offsets)
    lib = nat.load("routed SwiGLU")
    if h.dtype is not torch.bfloat16:
        raise TypeError("moe_swiglu_rows takes bf16 rows")
    h = h.contiguous()
    P, two_i = h.shape
    out = torch.empty((P, two_i // 2), dtype=torch.bfloat16, device=h.device)
    nat.check(lib.gb_moe_swiglu_rows(_ptr(h), _ptr(offsets), offsets.numel() - 1, P, two_i // 2,
                                     nat.ACT_FP4_GROUP16 if act == "fp4" else nat.ACT_NONE, _rule(scale_rule),
                                     _ptr(out), nat.stream_ptr(h.device)), lib)
    return out


def stack_rows(w: PackedWeight) -> PackedWeight:
    """An expert stack [E, rows, bytes] seen as one matrix of E * rows rows (the experts are
    contiguous), for the expanders.  Per-row codebook offsets (gate and up with their own books)
    repeat for every expert."""
    if w.experts == 1:
        return w
    if w.expert_stride != w.rows * w.row_stride:
        raise RuntimeError("the expert stack is not one contiguous matrix")
    ws = None if w.weight_scale is None else w.weight_scale.reshape(-1)
    off = None
    if w.cb_row_offset is not None:
        off = getattr(w, "_stack_offsets", None)
        if off is None:
            off = w.cb_row_offset.repeat(w.experts).contiguous()
            w._stack_offsets = off
    return PackedWeight(w.qw, w.codebook, w.fmt, w.K, w.experts * w.rows, w.row_stride, off,
                        w.compose, ws, w.global_scale)


def moe_gemv_sorted_applies(w: PackedWeight) -> bool:
    """Formats and layouts the sorted-rows expert kernel decodes (the conditions the library checks):
    the literal fp4 format, the two-tier fp4 k = 16 format in 80-byte superblock slots, the fp8
    product formats k = 32 (n_sub 4) and k = 16 (n_sub 2); one codebook, rows a multiple of 128,
    16-byte aligned rows, a contiguous stack."""
    f = w.fmt
    served = ((f.is_fp4 and f.mode == "full" and f.k == 8 and f.scale_coding == "v1" and f.type_size == 48)
              or (f.is_fp4 and f.mode == "product" and f.k == 16 and f.n_sub == 2 and f.scale_coding == "v2"
                  and f.type_size == 80)
              or (not f.is_fp4 and f.mode == "product" and ((f.k == 32 and f.n_sub == 4) or (f.k == 16 and f.n_sub == 2))))
    return (served and w.cb_row_offset is None and w.rows % 128 == 0 and w.row_stride % 16 == 0
            and w.expert_stride == w.rows * w.row_stride and w.qw.data_ptr() % 16 == 0
            and w.codebook.data_ptr() % 16 == 0)


def moe_gemv_sorted(x_sorted: torch.Tensor, w: PackedWeight, offsets: torch.Tensor, *,
                    row_map: torch.Tensor | None = None, peer_rows=None,
                    out: torch.Tensor | None = None) -> torch.Tensor | None:
    """Grouped linear over rows already in expert order, for mid-size batches: every (expert, 128-row
    tile) decodes its packed rows into tensor memory and multiplies on the tensor cores.  -> [P, rows]
    bf16 (row j at ``row_map[j]`` or j; rows past ``offsets[E]`` unset), or None when
    :func:`moe_gemv_sorted_applies` says the stack is not served.  ``peer_rows``
    (a ``GbPeerRows``): rows go to their home rank's buffer instead, nothing is returned."""
    _need_cuda(x_sorted, offsets, row_map)
    lib = nat.load("sorted-rows expert kernel")
    if not moe_gemv_sorted_applies(w):
        return None
    x_sorted = x_sorted.contiguous()
    P = x_sorted.shape[0]
    if peer_rows is not None:
        out = None
    elif out is None:
        out = torch.empty((P, w.rows), dtype=torch.bfloat16, device=x_sorted.device)
    nw = w.native()
    nat.check(lib.gb_moe_gemv_sorted(_ptr(x_sorted), ctypes.byref(nw), w.expert_stride, w.experts, _ptr(offsets),
                                     _ptr(row_map), P, _ptr(out),
                                     ctypes.byref(peer_rows) if peer_rows is not None else None,
                                     nat.stream_ptr(x_sorted.device)), lib)
    return out if peer_rows is None else True
