"""Routed-experts (FusedMoE) method behind the plugin surface
(gridbook/moe.py:406-550,552-955,957-1055,2388-2504): stacked packed experts, device-side
routing, grouped codebook GEMV with fused SwiGLU, top-k weighted combine."""
from __future__ import annotations

import sys

import torch

from . import _native, codec, kernels
from ._native import NativeKernelUnavailableError
from ._vllm_compat import FusedMoEMethodBase
from .formats import CBFormat


# Route thresholds, in routed pairs (per expert where it says so).  They are crossovers measured on
# one B200 with 128 experts, hidden 2048, intermediate 768 (literal fp4 format); every method
# instance carries its own copy (attributes of the same lower-case names) that a caller may set
# for another shape.
PAIR_KERNEL_MAX_PAIRS = 768       # routed pairs up to which every pair runs as its own table GEMV
FUSED_BUCKET_MAX_PAIRS = 32       # routed pairs up to which the grouped kernel buckets its own rows
# From this many routed pairs per expert (on average) the routed layer decodes each stack once
# into a transient and runs grouped tensor-core GEMMs (sorted rows: 0.98 ms at 256 pairs per expert
# and +0.20 us per token; decoded stack + grouped GEMM: 1.12 ms and +0.13 us per token).
PREFILL_MIN_PAIRS_PER_EXPERT = 384
# Below that, from this many routed pairs per expert on, the rows are sorted by expert and every
# (expert, 128-row tile) decodes its weights once into tensor memory for a tensor-core MMA.  Literal
# fp4 stacks have the per-pair table kernel below it (measured at 128 experts, hidden 2048,
# intermediate 768: per-pair kernel 164 us against 157 us at 4 pairs per expert, decode kernel 280
# against 166 at 8).  Stacks without that kernel (two-tier k = 16, the fp8 grid) take the sorted
# rows from SORTED_MIN_PAIRS_OTHER routed pairs in all (two tokens at top-8: 223 us against 272 us
# on 32 experts of hidden 7168, intermediate 2048).
SORTED_MIN_PAIRS_PER_EXPERT = 4
SORTED_MIN_PAIRS_OTHER = 16
# Stacks the sorted-rows kernel does not decode (per-role codebooks, other widths and modes) go from
# the decode kernel's 16-row passes straight to the decoded stack + grouped GEMM, whose crossover
# with the decode kernel was measured at ~800 tokens of 128 experts top-8.
PREFILL_MIN_PAIRS_OTHER = 50


def _row_bytes(in_features: int, type_size: int) -> int:
    if in_features % codec.SUPERBLOCK:
        raise ValueError(f"in_features {in_features} not a multiple of {codec.SUPERBLOCK}")
    return (in_features // codec.SUPERBLOCK) * type_size


# Every stacked expert parameter carries a "was it filled" stamp (gridbook/cb_fill_guard.py:33-75):
# create_weights allocates uninitialised memory, and a model class whose loader never reaches the
# stacks would otherwise serve it without any error.
CB_FILLED_ATTR = "_pq_cb_filled"
CB_EXPERT_PARAM_NAMES = ("w13_cb_qweight", "w2_cb_qweight")


def mark_filled(param) -> None:
    """Record that checkpoint bytes were put into a stacked expert parameter.  Every fill path
    calls it: the load hook below, the artifact loader, CBMoE.load, and any loader of the caller's
    own that assigns the stacks directly."""
    setattr(param, CB_FILLED_ATTR, True)


def unfilled_cb_params(layer) -> list[str]:
    """Names of the registered, non-empty expert stacks that no fill path has marked.  A stack that
    is absent or has no experts on this rank proves nothing and is skipped; one without a stamp at
    all did not come from create_weights and counts as unfilled."""
    missing = []
    for name in CB_EXPERT_PARAM_NAMES:
        p = getattr(layer, name, None)
        if p is None or p.numel() == 0:
            continue
        if not getattr(p, CB_FILLED_ATTR, False):
            missing.append(name)
    return missing


class PrismaQuantCBMoEMethod(FusedMoEMethodBase):
    """CB decode for routed experts.  ``scheme`` is the gate_up format; ``scheme_down``
    (optional, not expressible in the reference: gridbook/config.py:1631-1640) gives the
    down projection its own format."""

    def __init__(self, quant_config, moe, scheme: dict, prefix: str, scheme_down: dict | None = None) -> None:
        super().__init__(moe)
        self.quant_config = quant_config
        self.scheme = scheme
        self.scheme_down = scheme_down or scheme
        self.prefix = prefix
        self.fmt13 = CBFormat.from_scheme(self.scheme)
        self.fmt2 = CBFormat.from_scheme(self.scheme_down)
        self.is_fp4 = self.fmt13.is_fp4
        # Stacks whose scheme declares the static NVFP4 activation contract ship one calibrated scale
        # per stage (gridbook/moe.py:423-427,492-500): the parameters are created and checked so the
        # checkpoint loads; the prefill route stays the per-row one.
        self.has_static_fp4_activation = {
            "w13": codec.static_activation_contract(self.scheme, f"{prefix}.w13"),
            "w2": codec.static_activation_contract(self.scheme_down, f"{prefix}.w2")}
        self.k, self.n_sub, self.type_size = self.fmt13.k, self.fmt13.n_sub, self.fmt13.type_size
        self.pair_kernel_max_pairs = PAIR_KERNEL_MAX_PAIRS
        self.sorted_min_pairs_per_expert = SORTED_MIN_PAIRS_PER_EXPERT
        self.sorted_min_pairs_other = SORTED_MIN_PAIRS_OTHER
        self.prefill_min_pairs_other = PREFILL_MIN_PAIRS_OTHER
        self.pad_two_tier_superblocks = True   # fp4 k = 16 two-tier stacks: 73-byte superblocks in 80-byte slots
        self.prefill_min_pairs_per_expert = PREFILL_MIN_PAIRS_PER_EXPERT

    # ------------------------------------------------------------------ parameters
    def create_weights(self, layer, num_experts: int, hidden_size: int,
                       intermediate_size_per_partition: int, params_dtype, **extra_weight_attrs):
        del params_dtype
        E, inter = num_experts, intermediate_size_per_partition
        layer._cb_hidden, layer._cb_inter = hidden_size, inter
        attrs = dict(extra_weight_attrs)

        def param_from(data):
            p = torch.nn.Parameter(data, requires_grad=False)
            for key, val in attrs.items():
                setattr(p, key, val)
            return p

        def param(shape, dtype):
            return param_from(torch.empty(*shape, dtype=dtype))

        # w13 = gate_up: out = 2*inter, in = hidden.  w2 = down: out = hidden, in = inter.
        layer.register_parameter("w13_cb_qweight", param(
            (E, 2 * inter, _row_bytes(hidden_size, self.fmt13.type_size)), torch.uint8))
        layer.register_parameter("w2_cb_qweight", param(
            (E, hidden_size, _row_bytes(inter, self.fmt2.type_size)), torch.uint8))
        for name in CB_EXPERT_PARAM_NAMES:
            setattr(getattr(layer, name), CB_FILLED_ATTR, False)
        if not self.fmt13.is_fp4:
            layer.register_parameter("w13_weight_scale", param((E, 2 * inter), torch.float32))
        if not self.fmt2.is_fp4:
            layer.register_parameter("w2_weight_scale", param((E, hidden_size), torch.float32))
        for which in ("w13", "w2"):
            if self.has_static_fp4_activation[which]:        # NaN until the checkpoint fills it
                layer.register_parameter(f"{which}_input_global_scale",
                                         param_from(torch.full((1,), float("nan"), dtype=torch.float32)))
        self._install_load_hook(layer)

    def _install_load_hook(self, layer) -> None:
        """Checkpoint tensors `<proj>.cb_qweight` / `<proj>.weight_scale` load straight into
        the stacked parameters; everything else goes to the layer's own loader
        (gridbook/moe.py:503-546)."""
        orig_load = getattr(layer, "load_weights", None)
        if orig_load is None or getattr(layer, "_cb_load_wrapped", False):
            return
        prefix = self.prefix
        cb_map = {"gate_up_proj.cb_qweight": "w13_cb_qweight", "down_proj.cb_qweight": "w2_cb_qweight",
                  "gate_up_proj.weight_scale": "w13_weight_scale", "down_proj.weight_scale": "w2_weight_scale",
                  "gate_up_proj.input_global_scale": "w13_input_global_scale",
                  "down_proj.input_global_scale": "w2_input_global_scale"}

        def _cb_load_weights(weights):
            deferred = []
            for name, w in weights:
                pname = cb_map.get(name)
                if pname is not None and hasattr(layer, pname):
                    p = getattr(layer, pname)
                    if tuple(p.shape) != tuple(w.shape):
                        raise ValueError(f"{prefix}.{name}: checkpoint shape {tuple(w.shape)} != param "
                                         f"{tuple(p.shape)} — stacked (E, out, bytes) contract violated")
                    p.data.copy_(w.to(p.dtype))
                    if pname in CB_EXPERT_PARAM_NAMES:
                        mark_filled(p)
                    yield pname
                else:
                    deferred.append((name, w))
            if deferred:
                yield from orig_load(deferred)

        layer.load_weights = _cb_load_weights
        layer._cb_load_wrapped = True

    def get_fused_moe_quant_config(self, layer):
        return None

    # ------------------------------------------------------------------ post-load prep
    def _stack_weight(self, layer, qw_name: str, scale_name: str, fmt: CBFormat, k_in: int, role: str):
        qc = self.quant_config
        if qc is None:
            raise NativeKernelUnavailableError(f"{self.prefix}: no quantization config to resolve codebooks")
        scheme = self.scheme if role == "w13" else self.scheme_down
        roles = qc.codebooks_for_prefix(f"{self.prefix}.{role}", scheme)
        # Per-role books (docs/SPEC.md:480-527; the reference serves them for FP8-CB only,
        # gridbook/moe.py:2252-2273): gate and up may carry their own book at the same rung, w13
        # splits at exactly `inter` rows, and every kernel selects the book by row.  w2 is a
        # one-role stack.
        if role == "w2" and len(roles) != 1:
            raise NativeKernelUnavailableError(
                f"{self.prefix}: the down projection is a one-role stack; got {len(roles)} codebooks")
        if role == "w13" and len(roles) not in (1, 2):
            raise NativeKernelUnavailableError(
                f"{self.prefix}: gate_up takes one shared codebook or one each for gate and up; got {len(roles)}")
        blocks = [codec.build_flat_codebook(list(tabs), prefix=self.prefix, grid=fmt.grid)
                  for tabs in roles]
        for b in blocks:
            if b.numel() != fmt.codebook_elems():
                raise ValueError(f"{self.prefix}: codebook has {b.numel()} entries, {fmt} wants {fmt.codebook_elems()}")
        flat = torch.cat(blocks)
        p = getattr(layer, qw_name)
        dev = p.device
        qw = p.data
        if (self.pad_two_tier_superblocks and fmt.is_fp4 and fmt.mode == "product" and fmt.k == 16 and fmt.n_sub == 2
                and fmt.scale_coding == "v2" and len(blocks) == 1 and qw.shape[1] % 128 == 0 and k_in >= 256):
            # 73-byte superblocks -> 80-byte slots, once (the sorted-rows kernel fetches rows by TMA)
            qw = codec.pad_superblocks(qw, fmt.type_size, 80)
            fmt = fmt.padded(80)
        packed = codec.with_tail_slack(qw)
        p.data = packed
        cb_dev = (flat if fmt.is_fp4 else codec.flat_codebook_fp8(flat, self.prefix)).to(dev)
        sc = scheme.get("scale_coding")
        table = (sc.get("table") if isinstance(sc, dict) else None) or codec.TWO_TIER_SUB_TABLE
        compose = codec.build_compose_table(table).to(dev) if fmt.scale_coding == "v2" else None
        ws = getattr(layer, scale_name).data.float().contiguous() if not fmt.is_fp4 else None
        cb_row_offset = None
        if len(blocks) == 2:
            inter = layer._cb_inter
            cb_row_offset = torch.cat([torch.zeros(inter, dtype=torch.int32),
                                       torch.full((inter,), fmt.codebook_elems(), dtype=torch.int32)]).to(dev)
        return kernels.make_weight(packed, cb_dev, fmt, k_in, cb_row_offset=cb_row_offset, compose=compose,
                                   weight_scale=ws, global_scale=float(scheme.get("weight_global_scale", 1.0)))

    def _require_served_contract(self, layer) -> None:
        """Fail closed at load on anything but SiLU-gated experts with router weights applied to the
        output (the reference resolves the activation and refuses weights-on-input the same way,
        gridbook/moe.py:920-921,972-974): the kernels fuse silu(gate) * up and nothing else."""
        act = getattr(layer, "activation", None)
        act = getattr(act, "value", act)
        if act is not None and str(act).lower() not in ("silu", "swiglu", "moeactivation.silu"):
            raise NativeKernelUnavailableError(
                f"{self.prefix} routed activation: activation {act!r} has no native Gridbook operator")
        if getattr(layer, "apply_router_weight_on_input", False):
            raise NativeKernelUnavailableError(
                f"{self.prefix}: apply_router_weight_on_input unsupported for CB MoE")

    def _finalize_static_activation_scales(self, layer) -> None:
        """Gate after loading for contracted stacks (gridbook/moe.py:560-594): each declared stage
        has its parameter and it was loaded with one finite positive scale."""
        for which in ("w13", "w2"):
            if not self.has_static_fp4_activation[which]:
                continue
            p = getattr(layer, f"{which}_input_global_scale", None)
            if p is None:
                raise ValueError(f"{self.prefix}: contracted FP4-CB MoE has no {which}_input_global_scale parameter")
            setattr(layer, f"_cb_fp4_input_global_scale_{which}_f32",
                    codec.loaded_static_activation_scale(p.data, f"{self.prefix}.{which}"))

    def _assert_experts_filled(self, layer) -> None:
        """No environment override, by design (gridbook/cb_fill_guard.py:121-140)."""
        missing = unfilled_cb_params(layer)
        if missing:
            raise RuntimeError(
                f"{self.prefix}: CB expert stack(s) {missing} were REGISTERED but never FILLED from the checkpoint: "
                f"the layer would serve uninitialised memory (plausible garbage, not a crash). The model class's "
                f"loader did not pass '<experts>.<proj>.cb_qweight' tensors to this layer's load_weights hook; "
                f"route them there, or call gridbook_b200.moe.mark_filled(param) after filling a stack directly.")

    def process_weights_after_loading(self, layer) -> None:
        self._require_served_contract(layer)
        self._assert_experts_filled(layer)
        self._finalize_static_activation_scales(layer)
        _native.load(f"{self.prefix}: CB routed experts")
        if not layer.w13_cb_qweight.is_cuda:
            raise NativeKernelUnavailableError(
                f"{self.prefix}: CB expert stacks must live on a CUDA device; there is no CPU path")
        _native.prepare(layer.w13_cb_qweight.device)
        layer._cb_w13 = self._stack_weight(layer, "w13_cb_qweight", "w13_weight_scale", self.fmt13,
                                           layer._cb_hidden, "w13")
        layer._cb_w2 = self._stack_weight(layer, "w2_cb_qweight", "w2_weight_scale", self.fmt2,
                                          layer._cb_inter, "w2")
        layer._cb_E = layer.w13_cb_qweight.shape[0]
        layer._cb_xrow_cache = {}
        from .ops import register_cb_layer
        layer._cb_layer_id = register_cb_layer(self, layer)
        print(f"[prismaquant-cb] {self.prefix}: decode=grouped-cuda (sm_100a) "
              f"w13={self.fmt13.grid}/k{self.fmt13.k} w2={self.fmt2.grid}/k{self.fmt2.k}",
              file=sys.stderr, flush=True)

    # ------------------------------------------------------------------ forward
    # keyword arguments an engine may pass that do not change what is computed
    _INERT_KWARGS = ("shared_experts", "shared_experts_input", "global_num_experts", "enable_eplb",
                     "expert_load_view", "logical_to_physical_map", "logical_replica_count")

    def apply(self, layer, x, topk_weights, topk_ids, shared_experts=None, shared_experts_input=None,
              apply_router_weight_on_input: bool = False, **kwargs):
        """Routed-only output; the shared expert is the engine's business
        (gridbook/moe.py:957-989)."""
        if apply_router_weight_on_input or getattr(layer, "apply_router_weight_on_input", False):
            raise NativeKernelUnavailableError(
                f"{self.prefix}: apply_router_weight_on_input unsupported for CB MoE")
        for key, val in kwargs.items():
            if key in self._INERT_KWARGS or val is None or val is False:
                continue
            if key == "activation" and str(getattr(val, "value", val)).lower() in ("silu", "swiglu"):
                continue
            # an expert_map, a different activation, a custom routing function ...: anything that
            # would change the result and that this method does not implement
            raise NativeKernelUnavailableError(
                f"{self.prefix}: argument {key}={val!r} changes the routed computation and has no native "
                "Gridbook operator")
        lid = getattr(layer, "_cb_layer_id", None)
        if lid is None:
            raise NativeKernelUnavailableError(
                f"{self.prefix}: CB experts were not registered during process_weights_after_loading")
        from .ops import cb_moe_forward
        return cb_moe_forward(x, topk_weights, topk_ids, lid)

    def _x_row(self, layer, T: int, topk: int, device):
        key = (T, topk)
        cached = layer._cb_xrow_cache.get(key)
        if cached is None:
            cached = (torch.arange(T * topk, device=device, dtype=torch.int32) // topk).contiguous()
            layer._cb_xrow_cache[key] = cached
        return cached

    def _apply_inline(self, layer, x, topk_weights, topk_ids):
        """route -> bucket -> grouped gate/up GEMV with SwiGLU -> bucket -> grouped down GEMV ->
        combine.  Four launches for small batches (the buckets fused into the grouped kernels), six
        otherwise; no host read, any token count (an expert's tokens are taken
        in passes of up to sixteen rows, its weights stream once per pass)."""
        from . import ops
        rule = ops.ACT_SCALE_RULE
        T, topk = topk_ids.shape
        if T == 0:
            return torch.empty_like(x)
        x2 = x.reshape(T, -1).to(torch.bfloat16).contiguous()
        ids = topk_ids.to(torch.int32).contiguous()
        sorted_ok = (kernels.moe_gemv_sorted_applies(layer._cb_w13) and kernels.moe_gemv_sorted_applies(layer._cb_w2)
                     and not (layer._cb_w2.fmt.is_fp4 and layer._cb_inter % 16))
        prefill_min = (self.prefill_min_pairs_per_expert if sorted_ok
                       else min(self.prefill_min_pairs_per_expert, self.prefill_min_pairs_other))
        if T * topk >= prefill_min * layer._cb_E:
            return self._apply_prefill(layer, x2, topk_weights, ids, rule).to(x.dtype).reshape(x.shape)
        pair_kernel = kernels.pair_kernel_applies(layer._cb_w13) and kernels.pair_kernel_applies(layer._cb_w2)
        if T * topk >= (self.sorted_min_pairs_per_expert * layer._cb_E if pair_kernel else self.sorted_min_pairs_other):
            out = self._apply_sorted(layer, x2, topk_weights, ids, rule)
            if out is not None:
                return out.to(x.dtype).reshape(x.shape)
        if T * topk <= self.pair_kernel_max_pairs and self.fmt13.is_fp4 and self.fmt2.is_fp4:
            out = self._apply_pairs(layer, x2, topk_weights, ids, rule)
            if out is not None:
                layer._cb_route = "per-pair table kernel"
                return out.to(x.dtype).reshape(x.shape)
        # the loop chain multiplies by the bf16-rounded router weight (gridbook/moe.py:2407-2408);
        # the routing launch writes it, zeroed for padded pairs
        _, offsets, order, pair_w = kernels.moe_route(ids, layer._cb_E, topk_weights)
        # Small batches: the fp4 bucket runs inside the grouped kernel while it stages the rows
        # (two launches fewer); large ones bucket once up front, since every row tile of an expert
        # would otherwise bucket the same rows again.
        fuse = T * topk <= FUSED_BUCKET_MAX_PAIRS
        x_row = self._x_row(layer, T, topk, x.device)
        if fuse and self.fmt13.is_fp4:
            a = kernels.moe_gemv(x2, layer._cb_w13, offsets, order, x_row=x_row, swiglu=True, clear=False,
                                 act="fp4", scale_rule=rule)
        else:
            bucket13 = kernels.fp4_act_qdq if self.fmt13.is_fp4 else kernels.fp8_act_qdq
            a = kernels.moe_gemv(bucket13(x2, rule), layer._cb_w13, offsets, order, x_row=x_row, swiglu=True,
                                 clear=False)
        if fuse and self.fmt2.is_fp4:
            y = kernels.moe_gemv(a, layer._cb_w2, offsets, order, clear=False, act="fp4", scale_rule=rule)
        else:
            bucket2 = kernels.fp4_act_qdq if self.fmt2.is_fp4 else kernels.fp8_act_qdq
            y = kernels.moe_gemv(bucket2(a, rule), layer._cb_w2, offsets, order, clear=False)
        out = kernels.moe_combine(y, pair_w, T, topk, topk_ids=ids, E=layer._cb_E)
        layer._cb_route = "grouped decode kernel"
        return out.to(x.dtype).reshape(x.shape)


    def _apply_prefill(self, layer, x2, topk_weights, ids, rule):
        """Many tokens per expert: decode each stack once into a transient bf16 tile of the exact
        served weights and run one grouped tensor-core GEMM over the expert segments per
        projection (tcgen05 kind::f16, accumulators in tensor memory; segment offsets stay on the
        device) - the reference's grouped bf16 route (gridbook/moe.py:2388-2504 with
        gridbook/ops.py:137-306).  Both grids keep the decode contract here (bucketed bf16 rows,
        per-weight bf16(value * scale)): the buckets between the two projections are coarse
        enough to turn a last-place difference of the first projection into whole quantisation
        steps, so the fp8 grid does not take the scales-in-the-epilogue E4M3 GEMM of the dense
        prefill."""
        T, topk = ids.shape
        E = layer._cb_E
        _, offsets, order, pair_w = kernels.moe_route(ids, E, topk_weights)
        x_row = self._x_row(layer, T, topk, x2.device)

        def bucket(rows, w):
            return (kernels.fp4_act_qdq if w.fmt.is_fp4 else kernels.fp8_act_qdq)(rows, rule)

        def stage(rows_sorted, w, row_map):
            wm = kernels.stack_rows(w)
            tile = kernels.expand_fp4_bf16(wm) if w.fmt.is_fp4 else kernels.expand_fp8_bf16(wm)
            return kernels.gemm_tn_grouped(rows_sorted, tile, offsets, w.rows, row_map=row_map,
                                           global_scale=w.global_scale)

        w13, w2 = layer._cb_w13, layer._cb_w2
        # bucket the T rows once, then bring them into expert order
        a = kernels.moe_gather_rows(bucket(x2, w13), order, offsets, x_row=x_row)
        if w2.fmt.is_fp4 and layer._cb_inter % 16 == 0:       # SwiGLU and the fp4 bucket in one launch
            h = kernels.moe_swiglu_rows(stage(a, w13, None), offsets, act="fp4", scale_rule=rule)
        else:
            h = bucket(kernels.moe_swiglu_rows(stage(a, w13, None), offsets), w2)
        y = stage(h, w2, order)                               # rows back in pair order
        layer._cb_route = "grouped prefill: expand + gemm_tn_grouped"
        return kernels.moe_combine(y, pair_w, T, topk, topk_ids=ids, E=E)

    def _apply_sorted(self, layer, x2, topk_weights, ids, rule):
        """Mid-size batches: route, bucket, bring the rows into expert order, then per projection one
        launch in which every (expert, 128-row tile) decodes its packed rows into tensor memory and
        multiplies them with the expert's rows on the tensor cores (tcgen05, 64 rows per pass);
        SwiGLU and the second bucket between them; the down projection stores its rows back in pair
        order for the combine.  The two stacks may be of different grids (an fp8-grid gate_up over an
        fp4-grid down): each projection's rows go through its own grid's bucket.  None when a stack
        is not of a format that kernel decodes (kernels.moe_gemv_sorted_applies)."""
        w13, w2 = layer._cb_w13, layer._cb_w2
        if not (kernels.moe_gemv_sorted_applies(w13) and kernels.moe_gemv_sorted_applies(w2)):
            return None
        if w2.fmt.is_fp4 and layer._cb_inter % 16:
            return None
        T, topk = ids.shape
        E = layer._cb_E
        _, offsets, order, pair_w = kernels.moe_route(ids, E, topk_weights)
        x_row = self._x_row(layer, T, topk, x2.device)
        xq = kernels.fp4_act_qdq(x2, rule) if w13.fmt.is_fp4 else kernels.fp8_act_qdq(x2, rule)
        a = kernels.moe_gather_rows(xq, order, offsets, x_row=x_row)
        h13 = kernels.moe_gemv_sorted(a, w13, offsets)
        if h13 is None:
            return None
        if w2.fmt.is_fp4:
            h = kernels.moe_swiglu_rows(h13, offsets, act="fp4", scale_rule=rule)
        else:
            h = kernels.fp8_act_qdq(kernels.moe_swiglu_rows(h13, offsets), rule)
        y = kernels.moe_gemv_sorted(h, w2, offsets, row_map=order)
        if y is None:
            return None
        layer._cb_route = "sorted rows: decode into tensor memory + tcgen05"
        return kernels.moe_combine(y, pair_w, T, topk, topk_ids=ids, E=E)

    def _apply_pairs(self, layer, x2, topk_weights, ids, rule):
        """Small batches of the literal format: every routed pair is its own M = 1 linear through
        the inner-product-table kernel (bucket fused; the down projection sums the gate/up K
        slices and applies SwiGLU while it stages its rows), then the combine.  Three launches, no
        routing tables.  None when the format has no such kernel."""
        T, topk = ids.shape
        x_row = self._x_row(layer, T, topk, x2.device)
        y = kernels.moe_mlp_pairs(x2, layer._cb_w13, layer._cb_w2, ids, x_row=x_row, act="fp4", scale_rule=rule)
        if y is None:
            return None
        return kernels.moe_combine(y, topk_weights, T, topk, topk_ids=ids, E=layer._cb_E, round_weights=True)


class CBMoE(torch.nn.Module):
    """Stand-alone driver of PrismaQuantCBMoEMethod (tests, benchmark): create_weights ->
    copy stacks in -> process_weights_after_loading -> apply."""

    def __init__(self, fmt13: CBFormat, fmt2: CBFormat, num_experts: int, hidden: int, inter: int,
                 codebooks13, codebooks2, *, prefix: str = "cb_moe"):
        super().__init__()
        from .linear import _scheme_of
        # codebooks13: the tables of one shared book, or [gate tables, up tables] for per-role books
        roles13 = list(codebooks13) if isinstance(codebooks13[0], (list, tuple)) else [codebooks13]
        books = {f"{prefix}.w13": roles13, f"{prefix}.w2": [codebooks2]}
        self.method = PrismaQuantCBMoEMethod(_PrefixCodebooks(books), None, _scheme_of(fmt13), prefix,
                                             scheme_down=_scheme_of(fmt2))
        self.method.create_weights(self, num_experts, hidden, inter, torch.bfloat16)

    def load(self, w13, w2, w13_scale=None, w2_scale=None, device="cuda"):
        self.w13_cb_qweight.data = w13.to(device)
        self.w2_cb_qweight.data = w2.to(device)
        mark_filled(self.w13_cb_qweight)
        mark_filled(self.w2_cb_qweight)
        if w13_scale is not None:
            self.w13_weight_scale.data = w13_scale.to(device)
        if w2_scale is not None:
            self.w2_weight_scale.data = w2_scale.to(device)
        self.method.process_weights_after_loading(self)
        return self

    def forward(self, x, topk_weights, topk_ids):
        return self.method.apply(self, x, topk_weights, topk_ids)


class _PrefixCodebooks:
    def __init__(self, books):
        self.books = books

    def codebooks_for_prefix(self, prefix, scheme):
        return self.books[prefix]
