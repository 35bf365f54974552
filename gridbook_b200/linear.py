"""Dense codebook Linear behind the plugin surface: ``create_weights`` /
``process_weights_after_loading`` / ``apply`` (gridbook/linear.py:204-273,374-680,
1025-1264), dispatching to the sm_100a kernels through the C ABI."""
from __future__ import annotations

import torch

from . import _native, codec, kernels
from ._native import NativeKernelUnavailableError
from ._vllm_compat import (ChannelQuantScaleParameter, LinearMethodBase, ModelWeightParameter,
                           PerTensorScaleParameter, register_weight_loader_v2_supported_method)
from .formats import CBFormat

DECODE_MAX_M = 16          # the decode-batch kernels take up to sixteen rows
MIDM_MAX_M = 128           # ... and the literal format's tensor-core decode kernel up to this many


@register_weight_loader_v2_supported_method
class PrismaQuantCBLinearMethod(LinearMethodBase):
    """One CB target Linear (possibly a fused q/k/v or gate/up module whose roles carry
    their own codebooks)."""

    def __init__(self, quant_config, scheme: dict, prefix: str) -> None:
        self.quant_config = quant_config
        self.scheme = scheme
        self.prefix = prefix
        self.fmt = CBFormat.from_scheme(scheme)
        self.is_fp4 = self.fmt.is_fp4
        self.k = self.fmt.k
        self.n_sub = self.fmt.n_sub
        self.type_size = self.fmt.type_size
        self.is_v2 = self.fmt.scale_coding == "v2"
        sc = scheme.get("scale_coding")
        self._sub_table = (sc.get("table") if isinstance(sc, dict) else None) or codec.TWO_TIER_SUB_TABLE
        self.global_scale = float(scheme.get("weight_global_scale", 1.0))
        # A scheme that declares the static NVFP4 activation contract ships one calibrated
        # `input_global_scale` per logical shard (gridbook/linear.py:214-218,252-267).  The parameter
        # is created and checked here so such a checkpoint loads; the prefill route stays the
        # per-row one (the reference's "rowwise" mode), the static modes have no kernel here.
        self.has_static_fp4_activation = codec.static_activation_contract(scheme, prefix)
        # fp4 grid, past the decode batches: "nvfp4" = native NVFP4 activations x the native NVFP4
        # view of the layer on the block-scaled tensor cores; "bf16" = the decode contract kept
        # (bucketed bf16 rows x bf16(value * scale)) on the bf16 tensor cores
        self.prefill_route = "nvfp4"
        self.midm_max_rows = MIDM_MAX_M      # rows up to which the tensor-core decode kernel is preferred to expand + GEMM
        self.pad_two_tier_superblocks = True   # fp4 k = 16 two-tier: 73-byte superblocks kept in 80-byte slots (TMA-fetchable)

    # ------------------------------------------------------------------ parameters
    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size,
                       output_size, params_dtype, **extra_weight_attrs):
        del input_size, output_size, params_dtype
        weight_loader = extra_weight_attrs.get("weight_loader")
        K = input_size_per_partition
        if K % codec.SUPERBLOCK != 0:
            raise ValueError(f"{self.prefix}: in_features {K} not a multiple of {codec.SUPERBLOCK}")
        rows = sum(output_partition_sizes)
        layer.logical_widths = list(output_partition_sizes)
        layer._cb_input_size = K
        layer.register_parameter("cb_qweight", ModelWeightParameter(
            data=torch.empty(rows, self.fmt.row_bytes(K), dtype=torch.uint8),
            input_dim=1, output_dim=0, weight_loader=weight_loader))
        if self.has_static_fp4_activation:
            # one slot per logical shard; NaN until the checkpoint fills it, so a tensor that never
            # arrived is seen at the gate after loading instead of becoming an arbitrary scale
            layer.register_parameter("input_global_scale", PerTensorScaleParameter(
                data=torch.full((len(output_partition_sizes),), float("nan"), dtype=torch.float32),
                weight_loader=weight_loader))
        if not self.is_fp4:
            layer.register_parameter("weight_scale", ChannelQuantScaleParameter(
                data=torch.empty(rows, dtype=torch.float32), output_dim=0, weight_loader=weight_loader))

    def _finalize_static_activation_scale(self, layer) -> None:
        """Gate after loading for a contracted layer (gridbook/linear.py:348-372): the parameter
        exists and every logical shard loaded the same finite positive scale.  The value is kept on
        the layer for a caller that wants it."""
        if not self.has_static_fp4_activation:
            return
        p = getattr(layer, "input_global_scale", None)
        if p is None:
            raise ValueError(f"{self.prefix}: contracted FP4-CB layer has no input_global_scale parameter")
        layer._cb_fp4_input_global_scale_f32 = codec.loaded_static_activation_scale(p.data, self.prefix)

    # ------------------------------------------------------------------ post-load prep
    def _role_codebooks(self) -> list[list[torch.Tensor]]:
        """Codebook tables of every role of this (possibly fused) module, in shard order."""
        qc = self.quant_config
        if qc is None:
            raise NativeKernelUnavailableError(f"{self.prefix}: no quantization config to resolve codebooks")
        return qc.codebooks_for_prefix(self.prefix, self.scheme)

    def process_weights_after_loading(self, layer) -> None:
        """Build what the kernels keep resident: flat codebook block(s), per-row codebook
        offsets, the compose table, a packed buffer with tail slack, and the layer id.
        Everything that can fail does so here, never at the first forward."""
        self._finalize_static_activation_scale(layer)
        _native.load(f"{self.prefix}: CB Linear")
        qw = layer.cb_qweight.data
        dev = qw.device
        if not qw.is_cuda:
            raise NativeKernelUnavailableError(
                f"{self.prefix}: CB Linear weights must live on a CUDA device; there is no CPU path")
        _native.prepare(dev)
        N, K = qw.shape[0], layer._cb_input_size
        roles = self._role_codebooks()
        grid = self.fmt.grid
        blocks = [codec.build_flat_codebook(list(tabs),
                                            prefix=self.prefix, grid=grid) for tabs in roles]
        for b in blocks:
            if b.numel() != self.fmt.codebook_elems():
                raise ValueError(f"{self.prefix}: codebook has {b.numel()} entries, format "
                                 f"{self.fmt} wants {self.fmt.codebook_elems()}")
        widths = list(getattr(layer, "logical_widths", [N]))
        cb_row_offset = None
        if len(blocks) > 1:
            if len(blocks) != len(widths) or sum(widths) != N:
                raise ValueError(f"{self.prefix}: {len(blocks)} role codebooks for shard widths {widths}")
            cb_row_offset = torch.repeat_interleave(
                torch.arange(len(blocks), dtype=torch.int32) * self.fmt.codebook_elems(),
                torch.tensor(widths)).to(torch.int32).to(dev)
        flat = torch.cat(blocks)
        cb_dev = (flat if self.is_fp4 else codec.flat_codebook_fp8(flat, self.prefix)).to(dev)
        compose = codec.build_compose_table(self._sub_table).to(dev) if self.is_v2 else None
        fmt = self.fmt
        if (self.pad_two_tier_superblocks and fmt.is_fp4 and fmt.mode == "product" and fmt.k == 16 and fmt.n_sub == 2
                and fmt.scale_coding == "v2" and cb_row_offset is None and N >= 128 and K >= 1024):
            # 73-byte superblocks -> 80-byte slots, once: the rows become fetchable by TMA and every
            # batch size runs on the tensor-core decode kernel (the bytes themselves stay packed)
            fmt = fmt.padded(80)
            qw = codec.pad_superblocks(qw, self.fmt.type_size, 80)
        packed = codec.with_tail_slack(qw)
        layer.cb_qweight.data = packed          # same bytes, slack-backed storage
        ws = layer.weight_scale.data.float().contiguous() if not self.is_fp4 else None
        layer._cb_weight = kernels.make_weight(packed, cb_dev, fmt, K, cb_row_offset=cb_row_offset,
                                               compose=compose, weight_scale=ws,
                                               global_scale=self.global_scale)
        layer._cb_N, layer._cb_K = N, K
        layer._cb_workspace = torch.empty(
            _native.load().gb_gemv_workspace_bytes(DECODE_MAX_M, N, K), dtype=torch.uint8, device=dev)
        from .ops import register_cb_layer, warn_if_capture_sizes_exceed_the_decode_gates
        layer._cb_layer_id = register_cb_layer(self, layer)
        warn_if_capture_sizes_exceed_the_decode_gates()
        layer._cb_route = {"kernel": "gemv_kernel", "format": str(self.fmt), "N": N, "K": K}
        # one activation row of the literal format: the one-launch table kernel and its armed slots
        layer._cb_slots = (kernels.new_tab_slots([layer._cb_weight])
                           if kernels.table_kernel_applies(layer._cb_weight) else None)

    # ------------------------------------------------------------------ forward
    def apply(self, layer, x, bias=None):
        if bias is not None:
            raise NativeKernelUnavailableError(f"{self.prefix}: biased CB Linear has no native operator")
        lid = getattr(layer, "_cb_layer_id", None)
        if lid is None:
            raise NativeKernelUnavailableError(
                f"{self.prefix}: CB Linear was not registered during process_weights_after_loading")
        from .ops import cb_linear_forward
        return cb_linear_forward(x, lid)

    def _apply_inline(self, layer, x, bias=None):
        from . import ops
        w = layer._cb_weight
        N, K = layer._cb_N, layer._cb_K
        x2 = x.reshape(-1, K)
        M = x2.shape[0]
        if M == 0:
            return x.new_empty((*x.shape[:-1], N))
        if M == 1 and getattr(layer, "_cb_slots", None) is not None:
            outs = kernels.gemv_tab(x2, [w], layer._cb_slots, act=self.fmt.grid, scale_rule=ops.ACT_SCALE_RULE)
            if outs is not None:
                return outs[0].reshape(*x.shape[:-1], N)
        if M <= DECODE_MAX_M or M <= min(self.midm_max_rows, kernels.row_batch_max_rows(w)):
            # past sixteen rows: the literal format's tensor-core decode kernel, no decoded transient
            return kernels.gemv(x2, w, act=self.fmt.grid, scale_rule=ops.ACT_SCALE_RULE,
                                workspace=layer._cb_workspace).reshape(*x.shape[:-1], N)
        return self._apply_prefill(layer, x2).reshape(*x.shape[:-1], N)

    def _apply_prefill(self, layer, x2):
        """M > 16: expand the layer once into a transient decoded tile and run one tensor-core
        GEMM over it (tcgen05, accumulator in tensor memory).

        fp4 grid, route "nvfp4" (default): the rows are quantised to native NVFP4 (per-row scale,
        UE4M3 group scale factors, nearest-even E2M1), the layer is expanded to its native NVFP4
        view (packed E2M1 + E4M3 group scales, 0.56 bytes per weight) and the two meet in a
        block-scaled kind::mxf4nvf4 MMA — the reference's fused FP4 prefill lane
        (gridbook/csrc/cb_fused_fp4_gemm.cu:758-903); its activation bucket is NOT the decode
        contract's (UE4M3 scale factors instead of fp32 amax / 6).  Route "bf16": activations go
        through the group-16 bucket, the tile is the exact bf16 served weight, kind::f16 MMA —
        the reference's expand + bf16 GEMM route with the decode numerics
        (gridbook/linear.py:983-1023,1146-1152).  fp8 grid: activations are quantised per token to
        E4M3, the tile is the E4M3 value plane, kind::f8f6f4 MMA, and both scales multiply the
        fp32 accumulator — the reference's fp8 prefill lanes
        (gridbook/linear.py:1221-1264; epilogue of gridbook/csrc/cb_fused_gemm.cu:476-486)."""
        from . import ops
        w = layer._cb_weight
        if self.is_fp4 and self.prefill_route == "nvfp4":
            a, sfa, a_scale = kernels.nvfp4_quantize_rows(x2.contiguous())
            b, sfb = kernels.expand_fp4_nvfp4(w, operand=True)
            layer._cb_route["prefill"] = "nvfp4 activations + expand_fp4_nvfp4 + gemm_fp4(kind::mxf4nvf4)"
            return kernels.gemm_fp4(a, sfa, b, sfb, a_scale=a_scale, global_scale=w.global_scale)
        if self.is_fp4:
            xq = kernels.fp4_act_qdq(x2.contiguous(), ops.ACT_SCALE_RULE)
            wt = kernels.expand_fp4_bf16(w)
            layer._cb_route["prefill"] = "expand_fp4_bf16 + gemm_tn(kind::f16)"
            return kernels.gemm_tn(xq, wt, global_scale=w.global_scale)
        q, a_scale = kernels.fp8_quantize_rows(x2.contiguous(), ops.ACT_SCALE_RULE)
        wt = kernels.expand_fp8(w)
        layer._cb_route["prefill"] = "expand_fp8 + gemm_tn(kind::f8f6f4)"
        return kernels.gemm_tn(q, wt, a_scale=a_scale, b_scale=w.weight_scale, global_scale=w.global_scale)


def apply_shared_row(layers, x: torch.Tensor):
    """Several CB Linears that read the SAME activation row (q and kv of an attention block, gate
    and up kept as separate modules): one launch builds the inner-product tables once per CTA and
    streams all of them.  Falls back to one call per layer when the batch is not a single row or a
    layer's format has no table kernel.  -> list of outputs, in the order of ``layers``."""
    from . import ops
    layers = list(layers)
    ws = [l._cb_weight for l in layers]
    x2 = x.reshape(-1, ws[0].K)
    if (x2.shape[0] == 1 and 1 < len(layers) <= 4 and all(getattr(l, "_cb_slots", None) is not None for l in layers)
            and all(w.K == ws[0].K for w in ws)):
        key = tuple(l._cb_layer_id for l in layers)
        cache = layers[0].__dict__.setdefault("_cb_shared_slots", {})
        slots = cache.get(key)
        if slots is None:
            slots = cache[key] = kernels.new_tab_slots(ws)
        outs = kernels.gemv_tab(x2, ws, slots, act=ws[0].fmt.grid, scale_rule=ops.ACT_SCALE_RULE)
        if outs is not None:
            return [o.reshape(*x.shape[:-1], w.rows) for o, w in zip(outs, ws)]
    return [l(x) for l in layers]


def _scheme_of(fmt: CBFormat, global_scale: float = 1.0) -> dict:
    """The reference-style scheme dict of a format (docs/SPEC.md:408-440)."""
    scheme = {"grid": fmt.grid, "mode": fmt.mode, "k": fmt.k, "n_sub": fmt.n_sub,
              "type_size": fmt.type_size, "weight_global_scale": global_scale}
    if fmt.scale_coding == "v2":
        scheme["scale_coding"] = {"kind": "two_tier", "table": list(codec.TWO_TIER_SUB_TABLE)}
    return scheme


class CBLinear(torch.nn.Module):
    """Stand-alone module that drives PrismaQuantCBLinearMethod exactly as an engine does:
    create_weights -> copy the checkpoint tensors in -> process_weights_after_loading ->
    apply.  Used by the tests, the benchmark and anyone without an engine."""

    def __init__(self, fmt: CBFormat, in_features: int, out_partition_sizes, codebooks, *,
                 global_scale: float = 1.0, prefix: str = "cb_linear"):
        super().__init__()
        scheme = _scheme_of(fmt, global_scale)
        self.method = PrismaQuantCBLinearMethod(_InlineCodebooks(codebooks), scheme, prefix)
        sizes = list(out_partition_sizes)
        self.method.create_weights(self, in_features, sizes, in_features, sum(sizes), torch.bfloat16)

    def load(self, qw: torch.Tensor, weight_scale: torch.Tensor | None = None, device="cuda"):
        self.cb_qweight.data = qw.to(device)
        if weight_scale is not None:
            self.weight_scale.data = weight_scale.to(device)
        self.method.process_weights_after_loading(self)
        return self

    def forward(self, x):
        return self.method.apply(self, x)


class _InlineCodebooks:
    """Minimal codebook provider: ``roles`` is a list (one entry per fused role) of lists of
    tables.  Stands in for PrismaQuantConfig.codebooks_for_prefix."""

    def __init__(self, roles):
        self.roles = roles

    def codebooks_for_prefix(self, prefix, scheme):
        return self.roles
