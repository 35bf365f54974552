"""``prismaquant::*`` custom ops — the opaque operator boundary of the plugin, with the
reference's names, argument order and shape contracts (gridbook/ops.py:52-604,731-798).
Each op allocates its output with torch, hands raw pointers and the current stream to
the C ABI, and raises when the native library is missing: there is no other path."""
from __future__ import annotations

import itertools
import weakref

import torch

from . import kernels
from .formats import CBFormat
from ._native import NativeKernelUnavailableError  # noqa: F401  (re-exported)

# How `amax / c` is evaluated inside the activation buckets.  "recip" is what the
# reference's CUDA kernels do (torch-on-CUDA semantics, gridbook/csrc/cb_gemv.cu:88-91).
ACT_SCALE_RULE = "recip"


def _fmt_fp8(k_bits: int, n_sub: int, type_size: int) -> CBFormat:
    fmt = CBFormat("fp8", int(k_bits), n_sub=int(n_sub))
    if fmt.type_size != int(type_size):
        raise RuntimeError(f"type_size {type_size} does not match fp8 k={k_bits}")
    return fmt


def _fmt_fp4(k_bits: int, n_sub: int, type_size: int) -> CBFormat:
    """The reference's fp4 ops encode signed mode as n_sub == 1 and infer the scale coding
    from type_size (4k+9 two-tier, 4k+16 E4M3-direct)."""
    coding = {4 * int(k_bits) + 9: "v2", 4 * int(k_bits) + 16: "v1"}.get(int(type_size))
    if coding is None:
        raise RuntimeError(f"type_size {type_size} matches no fp4 scale coding for k={k_bits}")
    if int(n_sub) == 1:
        return CBFormat("fp4", int(k_bits), mode="signed", scale_coding=coding)
    return CBFormat("fp4", int(k_bits), n_sub=int(n_sub), scale_coding=coding)


def _check_rows(qw: torch.Tensor, fmt: CBFormat, K: int) -> None:
    if qw.shape[-1] < fmt.row_bytes(K):
        raise RuntimeError(f"packed row has {qw.shape[-1]} bytes, needs {fmt.row_bytes(K)}")


# --------------------------------------------------------------------------- dense GEMV
@torch.library.custom_op("prismaquant::cb_gemv_fp8", mutates_args=())
def cb_gemv_fp8(x: torch.Tensor, qw_padded: torch.Tensor, cb_flat: torch.Tensor,
                cb_row_offset: torch.Tensor, scale: torch.Tensor, N: int, K: int, k_bits: int,
                n_sub: int, type_size: int) -> torch.Tensor:
    """FP8-CB decode GEMV on RAW bf16 activations: per-token E4M3 bucket fused in front
    (gridbook/ops.py:52-64).  ``cb_flat`` is the E4M3-byte flat codebook."""
    fmt = _fmt_fp8(k_bits, n_sub, type_size)
    _check_rows(qw_padded, fmt, K)
    w = kernels.make_weight(qw_padded[:N], cb_flat, fmt, K, cb_row_offset=cb_row_offset,
                            weight_scale=scale)
    return kernels.gemv(x, w, act="fp8", scale_rule=ACT_SCALE_RULE)


@cb_gemv_fp8.register_fake
def _(x, qw_padded, cb_flat, cb_row_offset, scale, N, K, k_bits, n_sub, type_size):
    return torch.empty((*x.shape[:-1], N), dtype=x.dtype, device=x.device)


@torch.library.custom_op("prismaquant::cb_gemv_fp4_v2", mutates_args=())
def cb_gemv_fp4_v2(xq: torch.Tensor, qw_padded: torch.Tensor, cb_flat: torch.Tensor,
                   cb_row_offset: torch.Tensor, compose: torch.Tensor, N: int, K: int,
                   k_bits: int, n_sub: int, type_size: int) -> torch.Tensor:
    """FP4-CB decode GEMV on ALREADY bucketed activations (gridbook/ops.py:73-87)."""
    fmt = _fmt_fp4(k_bits, n_sub, type_size)
    _check_rows(qw_padded, fmt, K)
    w = kernels.make_weight(qw_padded[:N], cb_flat, fmt, K, cb_row_offset=cb_row_offset,
                            compose=compose)
    return kernels.gemv(xq, w)


@cb_gemv_fp4_v2.register_fake
def _(xq, qw_padded, cb_flat, cb_row_offset, compose, N, K, k_bits, n_sub, type_size):
    return torch.empty((*xq.shape[:-1], N), dtype=xq.dtype, device=xq.device)


# --------------------------------------------------------------------------- expanders
@torch.library.custom_op("prismaquant::cb_expand_fp8", mutates_args=())
def cb_expand_fp8(qw_padded: torch.Tensor, cb_flat_fp8: torch.Tensor, cb_row_offset: torch.Tensor,
                  N: int, K: int, k_bits: int, n_sub: int, type_size: int) -> torch.Tensor:
    """Packed rows -> [N, K] float8_e4m3fn tile (gridbook/ops.py:96-116)."""
    fmt = _fmt_fp8(k_bits, n_sub, type_size)
    dummy = torch.ones(N, dtype=torch.float32, device=qw_padded.device)
    w = kernels.make_weight(qw_padded[:N], cb_flat_fp8, fmt, K, cb_row_offset=cb_row_offset,
                            weight_scale=dummy)
    return kernels.expand_fp8(w)


@cb_expand_fp8.register_fake
def _(qw_padded, cb_flat_fp8, cb_row_offset, N, K, k_bits, n_sub, type_size):
    return torch.empty((N, K), dtype=torch.float8_e4m3fn, device=qw_padded.device)


@torch.library.custom_op("prismaquant::cb_expand_fp4_v2", mutates_args=())
def cb_expand_fp4_v2(qw_flat: torch.Tensor, cb_flat: torch.Tensor, compose: torch.Tensor, row0: int,
                     nrows: int, K: int, k_bits: int, type_size: int) -> torch.Tensor:
    """FP4 product rows [row0, row0+nrows) -> [nrows, K] bf16 = bf16(value * scale)
    (gridbook/ops.py:119-134).  ``qw_flat`` is [rows, row_bytes] (leading dims flattened)."""
    fmt = _fmt_fp4(k_bits, 2, type_size)
    qw2 = qw_flat.reshape(-1, qw_flat.shape[-1])
    w = kernels.make_weight(qw2, cb_flat, fmt, K, compose=compose)
    return kernels.expand_fp4_bf16(w, row0, nrows)


@cb_expand_fp4_v2.register_fake
def _(qw_flat, cb_flat, compose, row0, nrows, K, k_bits, type_size):
    return torch.empty((nrows, K), dtype=torch.bfloat16, device=qw_flat.device)


# --------------------------------------------------------------------------- buckets
@torch.library.custom_op("prismaquant::fp8_act_qdq", mutates_args=())
def fp8_act_qdq(x: torch.Tensor) -> torch.Tensor:
    """Per-token dynamic E4M3 QDQ (gridbook/ops.py:441-447)."""
    return kernels.fp8_act_qdq(x, ACT_SCALE_RULE)


@fp8_act_qdq.register_fake
def _(x):
    return torch.empty_like(x)


@torch.library.custom_op("prismaquant::fp4_act_qdq", mutates_args=())
def fp4_act_qdq(x: torch.Tensor) -> torch.Tensor:
    """Group-16 E2M1 QDQ (gridbook/ops.py:454-460)."""
    return kernels.fp4_act_qdq(x, ACT_SCALE_RULE)


@fp4_act_qdq.register_fake
def _(x):
    torch._check(x.shape[-1] % 16 == 0,
                 lambda: "fp4_act_qdq needs a last dim that is a multiple of the fp4 group (16)")
    return torch.empty_like(x, memory_format=torch.contiguous_format)


def fp4_act_qdq_or_codec(x: torch.Tensor) -> torch.Tensor:
    """Native and fail-closed (gridbook/ops.py:479-491); CPU tensors are refused because
    this package ships no host arithmetic."""
    if not x.is_cuda:
        raise NativeKernelUnavailableError("FP4 activation QDQ has no CPU path in gridbook_b200")
    return fp4_act_qdq(x)


# --------------------------------------------------------------------------- grouped MoE
def _grouped(xq, w, pair_expert, pair_xrow):
    """Serve the reference's per-pair signature: group the pairs by expert on the device,
    run the grouped kernel, results land in the caller's pair order."""
    P = pair_expert.shape[0]
    _, offsets, order = kernels.moe_route(pair_expert.reshape(P, 1), w.experts)
    return kernels.moe_gemv(xq, w, offsets, order, x_row=pair_xrow.to(torch.int32).contiguous())


@torch.library.custom_op("prismaquant::cb_moe_gemv_fp4_v2", mutates_args=())
def cb_moe_gemv_fp4_v2(xq: torch.Tensor, qw: torch.Tensor, cb_flat: torch.Tensor, compose: torch.Tensor,
                       pair_expert: torch.Tensor, pair_xrow: torch.Tensor, k_bits: int, n_sub: int,
                       type_size: int) -> torch.Tensor:
    """y[p] = xq[pair_xrow[p]] . W[pair_expert[p]]^T (gridbook/ops.py:494-510)."""
    K = xq.shape[-1]
    w = kernels.make_weight(qw, cb_flat, _fmt_fp4(k_bits, n_sub, type_size), K, compose=compose)
    return _grouped(xq, w, pair_expert, pair_xrow)


@cb_moe_gemv_fp4_v2.register_fake
def _(xq, qw, cb_flat, compose, pair_expert, pair_xrow, k_bits, n_sub, type_size):
    return torch.empty((pair_expert.shape[0], qw.shape[1]), dtype=xq.dtype, device=xq.device)


@torch.library.custom_op("prismaquant::cb_moe_gemv_v2", mutates_args=())
def cb_moe_gemv_v2(xq: torch.Tensor, qw: torch.Tensor, cb_flat: torch.Tensor, compose: torch.Tensor,
                   pair_expert: torch.Tensor, pair_xrow: torch.Tensor, k_bits: int, type_size: int,
                   rpb: int, dict_mode: int) -> torch.Tensor:
    """Same job as cb_moe_gemv_fp4_v2 (gridbook/ops.py:533-551); ``rpb`` and ``dict_mode``
    tuned the reference's shared-memory dictionary and are accepted and ignored: the
    codebook is always staged in shared memory here."""
    K = xq.shape[-1]
    w = kernels.make_weight(qw, cb_flat, _fmt_fp4(k_bits, 2, type_size), K, compose=compose)
    return _grouped(xq, w, pair_expert, pair_xrow)


@cb_moe_gemv_v2.register_fake
def _(xq, qw, cb_flat, compose, pair_expert, pair_xrow, k_bits, type_size, rpb, dict_mode):
    return torch.empty((pair_expert.shape[0], qw.shape[1]), dtype=xq.dtype, device=xq.device)


@torch.library.custom_op("prismaquant::cb_moe_gemv_fp8", mutates_args=())
def cb_moe_gemv_fp8(xq: torch.Tensor, qw: torch.Tensor, cb_flat_fp8: torch.Tensor, scale: torch.Tensor,
                    pair_expert: torch.Tensor, pair_xrow: torch.Tensor, k_bits: int, n_sub: int,
                    type_size: int) -> torch.Tensor:
    """Grouped FP8-CB GEMV on bucketed activations (gridbook/ops.py:554-570)."""
    K = xq.shape[-1]
    w = kernels.make_weight(qw, cb_flat_fp8, _fmt_fp8(k_bits, n_sub, type_size), K,
                            weight_scale=scale.contiguous())
    return _grouped(xq, w, pair_expert, pair_xrow)


@cb_moe_gemv_fp8.register_fake
def _(xq, qw, cb_flat_fp8, scale, pair_expert, pair_xrow, k_bits, n_sub, type_size):
    return torch.empty((pair_expert.shape[0], qw.shape[1]), dtype=xq.dtype, device=xq.device)


@torch.library.custom_op("prismaquant::cb_moe_gemv_fp8_v2", mutates_args=())
def cb_moe_gemv_fp8_v2(xq: torch.Tensor, qw: torch.Tensor, cb_flat_fp8: torch.Tensor, scale: torch.Tensor,
                       pair_expert: torch.Tensor, pair_xrow: torch.Tensor, k_bits: int, n_sub: int,
                       type_size: int) -> torch.Tensor:
    """The reference's whole-row sibling (gridbook/ops.py:573-590): one kernel serves both."""
    K = xq.shape[-1]
    w = kernels.make_weight(qw, cb_flat_fp8, _fmt_fp8(k_bits, n_sub, type_size), K,
                            weight_scale=scale.contiguous())
    return _grouped(xq, w, pair_expert, pair_xrow)


@cb_moe_gemv_fp8_v2.register_fake
def _(xq, qw, cb_flat_fp8, scale, pair_expert, pair_xrow, k_bits, n_sub, type_size):
    return torch.empty((pair_expert.shape[0], qw.shape[1]), dtype=xq.dtype, device=xq.device)


@torch.library.custom_op("prismaquant::cb_moe_combine", mutates_args=())
def cb_moe_combine(y: torch.Tensor, pair_w: torch.Tensor, tok_start: torch.Tensor, T: int) -> torch.Tensor:
    """out[t] = sum_p w[p] * y[p] over token t's pairs (gridbook/ops.py:593-604).  Pairs are
    token-major with a fixed top-k, i.e. ``tok_start == arange(T+1) * topk`` as the
    reference builds it (gridbook/moe.py:2409-2411)."""
    P = y.shape[0]
    if T <= 0 or P % T:
        raise RuntimeError(f"cb_moe_combine: {P} pairs do not divide into {T} tokens")
    if tok_start.numel() != T + 1:
        raise RuntimeError("cb_moe_combine: tok_start must have T+1 entries")
    return kernels.moe_combine(y, pair_w, T, P // T)


@cb_moe_combine.register_fake
def _(y, pair_w, tok_start, T):
    return torch.empty((T, y.shape[1]), dtype=y.dtype, device=y.device)


# --------------------------------------------------------------------------- grouped prefill
def _segments(expert_ends: torch.Tensor, expert_start: int, n_local: int) -> torch.Tensor:
    """Cumulative row ends of the FULL expert stack -> first-row offsets [n_local + 1] of the
    local slice, on the device (no host read)."""
    ends = expert_ends.to(torch.int32).reshape(-1)
    starts = torch.cat([ends.new_zeros(1), ends])
    return starts[expert_start:expert_start + n_local + 1].contiguous()


@torch.library.custom_op("prismaquant::cb_bf16_grouped_mm_out", mutates_args=("out",))
def cb_bf16_grouped_mm_out(out: torch.Tensor, a: torch.Tensor, weights: torch.Tensor, expert_ends: torch.Tensor,
                           expert_start: int = 0) -> None:
    """Grouped bf16 GEMM over expert segments into a caller-owned [P, N] (gridbook/ops.py:163-178):
    ``a`` [P, K] rows sorted by expert, ``weights`` [E_local, N, K] the local slice of the decoded
    stack, ``expert_ends`` the cumulative row ends of the full stack.  Rows of other experts are
    left as they are."""
    e_local, n, k = weights.shape
    seg = _segments(expert_ends, int(expert_start), e_local)
    kernels.gemm_tn_grouped(a, weights.reshape(e_local * n, k), seg, n, out=out)


@cb_bf16_grouped_mm_out.register_fake
def _(out, a, weights, expert_ends, expert_start=0):
    return None


@torch.library.custom_op("prismaquant::cb_bf16_grouped_mm", mutates_args=())
def cb_bf16_grouped_mm(a: torch.Tensor, weights: torch.Tensor, expert_ends: torch.Tensor,
                       expert_start: int = 0) -> torch.Tensor:
    """The allocating form (gridbook/ops.py:137-160): rows outside the local expert slice are zero."""
    out = torch.zeros((a.shape[0], weights.shape[1]), dtype=torch.bfloat16, device=a.device)
    cb_bf16_grouped_mm_out(out, a, weights, expert_ends, expert_start)
    return out


@cb_bf16_grouped_mm.register_fake
def _(a, weights, expert_ends, expert_start=0):
    return torch.empty((a.shape[0], weights.shape[1]), dtype=torch.bfloat16, device=a.device)


def _persistent_b(out, a, w, expert_ends):
    """One projection of the routed prefill over exact segments: the sorted-rows kernel that
    decodes in shared memory where the format has it, else decode once + grouped GEMM."""
    seg = _segments(expert_ends, 0, w.experts)
    if kernels.moe_gemv_sorted_applies(w) and a.shape[0] <= 128 * w.experts:
        if kernels.moe_gemv_sorted(a, w, seg, out=out) is not None:
            return
    wm = kernels.stack_rows(w)
    tile = kernels.expand_fp4_bf16(wm) if w.fmt.is_fp4 else kernels.expand_fp8_bf16(wm)
    kernels.gemm_tn_grouped(a, tile, seg, w.rows, global_scale=w.global_scale, out=out)


@torch.library.custom_op("prismaquant::cb_moe_persistent_b_prefill", mutates_args=("out",))
def cb_moe_persistent_b_prefill(out: torch.Tensor, a: torch.Tensor, qw: torch.Tensor, lut: torch.Tensor,
                                compose: torch.Tensor, expert_ends: torch.Tensor, k_bits: int, type_size: int,
                                cfg: int) -> None:
    """Grouped decode + GEMM over the exact routed segments into a caller-owned [P, N]
    (gridbook/ops.py:309-331): ``a`` [P, K] bucketed bf16 rows sorted by expert, ``qw`` [E, N, bytes]
    packed fp4 product codewords, ``lut`` the flat bf16 codebook.  ``cfg`` selected a tile shape of
    the reference's kernel and is accepted and ignored."""
    w = kernels.make_weight(qw, lut, _fmt_fp4(k_bits, 2, type_size), a.shape[-1], compose=compose)
    _persistent_b(out, a, w, expert_ends)


@cb_moe_persistent_b_prefill.register_fake
def _(out, a, qw, lut, compose, expert_ends, k_bits, type_size, cfg):
    return None


@torch.library.custom_op("prismaquant::cb_moe_persistent_b_prefill_d2r", mutates_args=("out",))
def cb_moe_persistent_b_prefill_d2r(out: torch.Tensor, a: torch.Tensor, qw: torch.Tensor, lut: torch.Tensor,
                                    compose: torch.Tensor, expert_ends: torch.Tensor, k_bits: int, type_size: int,
                                    cfg: int) -> None:
    """Same operands and result as cb_moe_persistent_b_prefill (gridbook/ops.py:334-355; the
    reference's variant differs only in how its mainloop builds fragments)."""
    w = kernels.make_weight(qw, lut, _fmt_fp4(k_bits, 2, type_size), a.shape[-1], compose=compose)
    _persistent_b(out, a, w, expert_ends)


@cb_moe_persistent_b_prefill_d2r.register_fake
def _(out, a, qw, lut, compose, expert_ends, k_bits, type_size, cfg):
    return None


def _fp8_codebook_bytes(lut_f32: torch.Tensor) -> torch.Tensor:
    """The fp32 table the reference converts from the E4M3 codebook at load, back to its bytes
    (exact: every entry is an E4M3 value)."""
    return lut_f32.to(torch.float32).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()


@torch.library.custom_op("prismaquant::cb_moe_persistent_b_prefill_fp8", mutates_args=("out",))
def cb_moe_persistent_b_prefill_fp8(out: torch.Tensor, a: torch.Tensor, qw: torch.Tensor, lut_f32: torch.Tensor,
                                    scale: torch.Tensor, expert_ends: torch.Tensor, k_bits: int, type_size: int,
                                    cfg: int) -> None:
    """The FP8-CB form (gridbook/ops.py:380-404): n_sub = 4 product codewords, per-(expert, row)
    fp32 ``scale`` applied before the single bf16 rounding of every weight."""
    w = kernels.make_weight(qw, _fp8_codebook_bytes(lut_f32), _fmt_fp8(k_bits, 4, type_size), a.shape[-1],
                            weight_scale=scale.to(torch.float32).contiguous())
    _persistent_b(out, a, w, expert_ends)


@cb_moe_persistent_b_prefill_fp8.register_fake
def _(out, a, qw, lut_f32, scale, expert_ends, k_bits, type_size, cfg):
    return None


@torch.library.custom_op("prismaquant::cb_moe_persistent_b_decode", mutates_args=())
def cb_moe_persistent_b_decode(qw_flat: torch.Tensor, lut: torch.Tensor, compose: torch.Tensor, row0: int,
                               nrows: int, K: int, k_bits: int, type_size: int) -> torch.Tensor:
    """The decode stage alone (gridbook/ops.py:358-377): rows [row0, row0 + nrows) of the flattened
    stack -> [nrows, K] bf16 = bf16(value * group scale)."""
    qw2 = qw_flat.reshape(-1, qw_flat.shape[-1])
    w = kernels.make_weight(qw2, lut, _fmt_fp4(k_bits, 2, type_size), K, compose=compose)
    return kernels.expand_fp4_bf16(w, row0, nrows)


@cb_moe_persistent_b_decode.register_fake
def _(qw_flat, lut, compose, row0, nrows, K, k_bits, type_size):
    return qw_flat.new_empty((nrows, K), dtype=torch.bfloat16)


@torch.library.custom_op("prismaquant::cb_moe_persistent_b_decode_fp8", mutates_args=())
def cb_moe_persistent_b_decode_fp8(qw_flat: torch.Tensor, lut_f32: torch.Tensor, scale: torch.Tensor, row0: int,
                                   nrows: int, K: int, k_bits: int, type_size: int) -> torch.Tensor:
    """The FP8 decode stage alone (gridbook/ops.py:407-428): bf16(value * scale[row])."""
    qw2 = qw_flat.reshape(-1, qw_flat.shape[-1])
    w = kernels.make_weight(qw2, _fp8_codebook_bytes(lut_f32), _fmt_fp8(k_bits, 4, type_size), K,
                            weight_scale=scale.reshape(-1).to(torch.float32).contiguous())
    return kernels.expand_fp8_bf16(w, row0, nrows)


@cb_moe_persistent_b_decode_fp8.register_fake
def _(qw_flat, lut_f32, scale, row0, nrows, K, k_bits, type_size):
    return qw_flat.new_empty((nrows, K), dtype=torch.bfloat16)


# --------------------------------------------------------------------------- layer registry
# Weak, monotonic integer indirection so the two whole-dispatch ops stay opaque to Dynamo
# (gridbook/ops.py:686-728).
_LAYER_IDS = itertools.count(1)
_LAYER_REGISTRY: dict[int, tuple] = {}


_CAPTURE_NOTE_DONE: list[bool] = []


def warn_if_capture_sizes_exceed_the_decode_gates() -> None:
    """The reference warns here when the engine's cudagraph_capture_sizes reach past its decode
    gates, because its prefill arms read routing counts on the host and cannot be captured
    (gridbook/ops.py:644-683).  No arm of this package reads a device value on the host - the
    routing, the segment offsets and the route choice all stay on the device or depend on shapes
    only - so every size is capturable and there is nothing to warn about.  What is still worth
    one line, once per process: sizes past the sixteen rows the per-layer workspace is laid out
    for allocate their transient tiles inside the capture (from the graph's private pool), which
    is legal but costs memory per captured size."""
    if _CAPTURE_NOTE_DONE:
        return
    _CAPTURE_NOTE_DONE.append(True)
    try:
        from vllm.config import get_current_vllm_config
        compilation = get_current_vllm_config().compilation_config
        sizes = [int(s) for s in (getattr(compilation, "cudagraph_capture_sizes", None) or ())]
    except Exception:  # advisory only; never break a load
        return
    over = sorted(s for s in sizes if s > 16)
    if over:
        import sys
        print(f"[prismaquant-cb] note: cudagraph_capture_sizes {over} are past the decode batches; these captures "
              "hold a decoded weight tile each (prefill routes). All routes are capture-safe.", file=sys.stderr,
              flush=True)


def register_cb_layer(method, layer) -> int:
    layer_id = next(_LAYER_IDS)

    def expire(_ref, *, expected_id=layer_id):
        _LAYER_REGISTRY.pop(expected_id, None)

    _LAYER_REGISTRY[layer_id] = (weakref.ref(method, expire), weakref.ref(layer, expire))
    return layer_id


def _lookup_cb_layer(layer_id: int):
    entry = _LAYER_REGISTRY.get(layer_id)
    if entry is None:
        raise RuntimeError(f"CB dispatch layer id {layer_id} is stale or unknown; the model "
                           "may have been unloaded")
    method, layer = entry[0](), entry[1]()
    if method is None or layer is None:
        _LAYER_REGISTRY.pop(layer_id, None)
        raise RuntimeError(f"CB dispatch layer id {layer_id} expired after model unload")
    return method, layer


@torch.library.custom_op("prismaquant::cb_linear_forward", mutates_args=())
def cb_linear_forward(x: torch.Tensor, layer_id: int) -> torch.Tensor:
    method, layer = _lookup_cb_layer(layer_id)
    return method._apply_inline(layer, x)


@cb_linear_forward.register_fake
def _(x, layer_id):
    _method, layer = _lookup_cb_layer(layer_id)
    return torch.empty((*x.shape[:-1], layer._cb_N), dtype=x.dtype, device=x.device)


def _neutralize_moe_padding_sentinel(topk_weights, topk_ids):
    """vLLM marks padded routes with expert id -1; make them inert without a host read
    (gridbook/ops.py:764-784)."""
    padding = topk_ids == -1
    return topk_weights.masked_fill(padding, 0), topk_ids.masked_fill(padding, 0)


@torch.library.custom_op("prismaquant::cb_moe_forward", mutates_args=())
def cb_moe_forward(x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                   layer_id: int) -> torch.Tensor:
    # Padded routes (expert id -1) need no masking pass here: the routing launch drops them and
    # zeroes their combine weight, which gives what the reference's (expert 0, weight 0)
    # substitution gives (gridbook/ops.py:764-784) without its three elementwise launches.
    method, layer = _lookup_cb_layer(layer_id)
    return method._apply_inline(layer, x, topk_weights, topk_ids)


@cb_moe_forward.register_fake
def _(x, topk_weights, topk_ids, layer_id):
    return torch.empty_like(x)
