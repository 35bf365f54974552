"""``PrismaQuantConfig`` — the quantization config vLLM instantiates for
``quant_method: gridbook`` (gridbook/config.py:484-531,803-957,1042-1106,1129-1204,
1422-1571,1605-1641).  Core paths only: pointer/inline resolution, target -> scheme map,
fused-shard roles, codebook sidecar, per-prefix method dispatch."""
from __future__ import annotations

import json
import os

import torch

from ._native import NativeKernelUnavailableError
from ._vllm_compat import HAVE_VLLM, QuantizationConfig

# fused module -> the checkpoint's per-role Linears, in shard order.  The engine publishes its own
# mapping by dispatch time; this table stays underneath it as the fallback (gridbook/config.py:115-132):
# the gated-delta-net projections, and the attention module that merges `wq_a` with `wkv` through its
# stacked-parameter table without declaring a packed mapping at all.
DEFAULT_PACKED_MODULES = {
    "qkv_proj": ["q_proj", "k_proj", "v_proj"],
    "gate_up_proj": ["gate_proj", "up_proj"],
    "in_proj_qkvz": ["in_proj_qkv", "in_proj_z"],
    "in_proj_ba": ["in_proj_b", "in_proj_a"],
    "fused_wqa_wkv": ["wq_a", "wkv"],
}
# Other checkpoint spellings of a served leaf (gridbook/config.py:134-158): a different fusion (`w1` /
# `w3` into the same `gate_up_proj`) or a plain rename (`w2` for `down_proj`).  Consulted only after
# the primary spelling found nothing; the first spelling with a hit wins whole, never mixed.
ALTERNATE_SHARD_SPELLINGS = {
    "gate_up_proj": (["w1", "w3"],),
    "gate_proj": (["w1"],),
    "up_proj": (["w3"],),
    "down_proj": (["w2"],),
}
_MOE_SUFFIXES = (".experts", ".mlp.experts", ".ffn.experts")

try:                                    # the engine's ignore lists are written for this engine
    import regex as _regex              # (Unicode properties); the stdlib one otherwise
except ImportError:                     # pragma: no cover - depends on the environment
    import re as _regex


def _canonical_prefix(name: str) -> str:
    """One namespace for the three spellings a module of the language model arrives in
    (gridbook/config.py:228-255): the wrapper-class serving form `language_model.model.X`, the
    older multimodal checkpoint form `model.language_model.X`, a bare `language_model.X`, and the
    source form `layers.N...` of checkpoints whose keys carry no `model.` at all - all become
    `model.X`.  Prefix-anchored; `visual.*`, `mtp.*`, `lm_head`, plain `model.layers.*` pass through."""
    for head, keep in (("language_model.model.", "model."), ("language_model.", "model."),
                       ("model.language_model.", "model.")):
        if name.startswith(head):
            return keep + name[len(head):]
    if name.startswith("layers."):
        return "model." + name
    return name


_canonical_target = _canonical_prefix     # stored targets and ignore entries: the same rewrite, once, at parse time


def _candidate_bases(name: str) -> list[str]:
    """The strings `name` may be matched as, most specific first: as given (the engine's mapper can
    move the stored keys into a namespace of its own after parsing), then canonical."""
    canonical = _canonical_prefix(name)
    return [name] if canonical == name else [name, canonical]


class PrismaQuantConfig(QuantizationConfig):
    """Holds the raw ``quantization_config`` and resolves it lazily (the sidecar files are
    read on first use, gridbook/config.py:803-957)."""

    def __init__(self, raw: dict, model_dir: str | None = None) -> None:
        super().__init__()
        self.raw = dict(raw)
        self.model_dir = model_dir or self.raw.get("_model_dir")
        self.packed_modules_mapping = dict(DEFAULT_PACKED_MODULES)
        self._resolved = False
        self.target_scheme: dict[str, dict] = {}
        self.ignore: list[str] = []
        self._codebooks: dict[str, torch.Tensor] | None = None

    # ---- vLLM QuantizationConfig surface (gridbook/config.py:1042-1074) -------------
    @classmethod
    def get_name(cls) -> str:
        return "gridbook"

    @classmethod
    def get_supported_act_dtypes(cls):
        return [torch.bfloat16]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100                      # sm_100a only (the reference says 80)

    @classmethod
    def get_config_filenames(cls):
        return []

    @classmethod
    def from_config(cls, config: dict) -> "PrismaQuantConfig":
        return cls(config)

    @classmethod
    def override_quantization_method(cls, hf_quant_cfg, user_quant):
        method = (hf_quant_cfg or {}).get("quant_method")
        return "gridbook" if method in ("gridbook", "prismaquant") else None

    def apply_vllm_mapper(self, hf_to_vllm_mapper) -> None:
        """The engine's checkpoint-to-module renaming, applied to the stored targets and to the literal
        ignore entries; patterns (`re:`) are never handed to it (gridbook/config.py:1761)."""
        self._ensure_resolved()
        if hasattr(hf_to_vllm_mapper, "apply_dict"):
            self.target_scheme = hf_to_vllm_mapper.apply_dict(self.target_scheme)
        if hasattr(hf_to_vllm_mapper, "apply_list"):
            literal = [ig for ig in self.ignore if not ig.startswith("re:")]
            mapped = iter(hf_to_vllm_mapper.apply_list(literal))
            self.ignore = [ig if ig.startswith("re:") else next(mapped) for ig in self.ignore]

    # ---- resolution -------------------------------------------------------------------
    def _ensure_resolved(self) -> None:
        if self._resolved:
            return
        full = self.raw
        if "config_groups" not in full:                          # pointer stub (docs/SPEC.md:388-399)
            if self.model_dir is None:
                raise ValueError("[prismaquant] pointer-style quantization_config needs the model directory")
            path = os.path.join(self.model_dir, full.get("config_file", "quant_config.json"))
            with open(path) as fh:
                full = json.load(fh)
        self.delegated_targets: dict[str, str] = {}
        for gname, group in full.get("config_groups", {}).items():
            raw_scheme = group.get("scheme")
            if not isinstance(raw_scheme, dict) or "grid" not in raw_scheme:
                # stock / passthrough groups carry no codebook scheme (the reference hands them to
                # other backends, gridbook/config.py:803-957): remembered so that a lookup can say
                # so instead of raising a bare KeyError or running them unquantized by accident
                for target in group.get("targets", []):
                    self.delegated_targets[_canonical_target(target)] = gname
                continue
            # v1 / v2 is decided by the group's OWN scale_coding: absent means v1 (E4M3-direct),
            # whatever the artifact's layout_version says (docs/SPEC.md:130-177; the reference's
            # linear method sets is_v2 = False when the key is missing, gridbook/linear.py:206-231)
            scheme = dict(raw_scheme)
            scheme.setdefault("_group", gname)
            for target in group.get("targets", []):
                self.target_scheme[_canonical_target(target)] = scheme
        # literal entries name one module (canonicalised like the targets); `re:` entries are patterns
        self.ignore = [ig if ig.startswith("re:") else _canonical_target(ig) for ig in full.get("ignore", [])]
        self.codebook_file = full.get("codebook_file", self.raw.get("codebook_file", "cb_codebooks.pqcb"))
        # artifact-external digests of the sidecar's tables (docs/SPEC.md:326-378); None = not declared
        prov = full.get("provenance")
        self.codebook_sha256 = prov.get("codebook_sha256") if isinstance(prov, dict) else None
        self._resolved = True

    def get_codebooks(self) -> dict[str, torch.Tensor]:
        """The codebook sidecar (a safetensors file, docs/SPEC.md:303-378), loaded once."""
        if self._codebooks is None:
            self._ensure_resolved()
            inline = self.raw.get("_codebooks")
            if inline is not None:
                self._codebooks = dict(inline)
            else:
                from safetensors.torch import load_file
                self._codebooks = load_file(os.path.join(self.model_dir, self.codebook_file))
            # declared digests are checked before any table is used; an undeclared mapping loads
            # without the check, an empty one does not equal absence
            from .artifact import verify_codebook_digests
            try:
                verify_codebook_digests(self._codebooks, self.codebook_sha256)
            except Exception:
                self._codebooks = None
                raise
        return self._codebooks

    def _tables(self, scheme: dict) -> list[torch.Tensor]:
        ref = scheme["codebook_ref"]
        names = ref if isinstance(ref, (list, tuple)) else [ref]
        books = self.get_codebooks()
        missing = [n for n in names if n not in books]
        if missing:
            raise KeyError(f"[prismaquant] codebook tensors {missing} are not in the sidecar")
        return [books[n] for n in names]

    # ---- fused shards (gridbook/config.py:1129-1204) ----------------------------------
    def _fused_roles(self, leaf: str) -> list[str] | None:
        live = getattr(self, "packed_modules_mapping", None) or {}
        return live.get(leaf) or DEFAULT_PACKED_MODULES.get(leaf)

    def shard_target_keys(self, prefix: str, unfused_fallback: bool = False) -> list[str]:
        """Checkpoint names whose rows make up the module `prefix`, in shard order: the roles of a
        fused module, the module itself, or another spelling of either."""
        self._ensure_resolved()
        head, _, leaf = prefix.rpartition(".")
        spellings = []
        roles = self._fused_roles(leaf)
        if roles:
            spellings.append(list(roles))
        spellings.append(None)                                  # the module under its own name
        spellings.extend(list(a) for a in ALTERNATE_SHARD_SPELLINGS.get(leaf, ()))
        for names in spellings:
            if names is None:
                if self._lookup(prefix) is not None:
                    return [prefix]
                continue
            keys = [f"{head}.{r}" if head else r for r in names]
            found = [k for k in keys if self._lookup(k) is not None]
            if found and len(found) != len(keys):
                raise ValueError(f"[prismaquant] {prefix}: only {found} of {keys} are CB targets; mixed "
                                 "fused modules are not served")
            if found:
                return keys
        return [prefix] if unfused_fallback else []

    # wrapper prefixes a serving class may put in front of (or strip from) the checkpoint's names
    _WRAPPERS = ("model", "language_model", "language_model.model", "model.language_model", "text_model")

    def _find(self, table: dict, key: str):
        """Entry of `table` (stored name -> value) that names the module `key`: the name as given,
        then its canonical form, then either side behind a known wrapper prefix.  Only a wrapper may
        separate the two names: a second tower whose modules end in the same tail
        (vision_tower.layers.0.mlp...) must not pick up this entry."""
        bases = _candidate_bases(key)
        for base in bases:
            if base in table:
                return table[base]
        wrapped = self._wrapped_index(table)
        for base in bases:
            if base in wrapped:
                return wrapped[base]
        return None

    def _wrapped_index(self, table: dict) -> dict:
        """name -> value for every stored name put behind, or freed from, one wrapper prefix; built
        once per table (a model has thousands of targets and asks once per module)."""
        cache = self.__dict__.setdefault("_wrapped_cache", [])
        for seen, size, index in cache:
            if seen is table and size == len(table):
                return index
        index: dict = {}
        for stored, value in table.items():
            for wrap in self._WRAPPERS:
                index.setdefault(f"{wrap}.{stored}", value)
                if stored.startswith(wrap + "."):
                    index.setdefault(stored[len(wrap) + 1:], value)
        cache[:] = [c for c in cache if c[0] is not table][-3:] + [(table, len(table), index)]
        return index

    def _lookup(self, key: str) -> dict | None:
        return self._find(self.target_scheme, key)

    def _delegated_group(self, key: str) -> str | None:
        return self._find(getattr(self, "delegated_targets", {}), key)

    def _name_ignored(self, name: str) -> bool:
        for base in _candidate_bases(name):
            for ig in self.ignore:
                if ig.startswith("re:"):
                    if _regex.match(ig[3:], base):           # start-anchored, not a full match
                        return True
                elif base == ig:
                    return True
        return False

    def _is_ignored(self, prefix: str) -> bool:
        """The `ignore` list with the exact / `re:` reading the engine's own compressed-tensors
        matcher gives it (the reference pins this in tests/test_target_namespace_compat.py:484-545): a
        literal entry names one module, nothing under it and nothing that merely starts the same; a
        pattern is `re.match`ed; a fused module is judged by its checkpoint shards, all of which
        must agree."""
        self._ensure_resolved()
        head, _, leaf = prefix.rpartition(".")
        roles = self._fused_roles(leaf)
        if roles:
            names = [f"{head}.{r}" if head else r for r in roles]
            flags = [self._name_ignored(n) for n in names]
            if any(flags) and not all(flags):
                hit = [n for n, f in zip(names, flags) if f]
                raise ValueError(f"[prismaquant] {prefix}: the shards of a fused module have different quantization "
                                 f"schemes: only {hit} of {names} are on the ignore list")
            return all(flags)
        return self._name_ignored(prefix)

    def _scheme_for_prefix(self, prefix: str) -> dict | None:
        keys = self.shard_target_keys(prefix)
        if not keys:
            return None
        schemes = [self._lookup(k) for k in keys]
        first = schemes[0]
        # the physical packed representation and the activation ABI one resident parameter set
        # shares; codebook refs may differ by role (gridbook/config.py:612-618)
        fields = ("grid", "mode", "k", "n_sub", "type_size", "group_size", "vec_dim", "scale_coding",
                  "activation_contract")
        for other in schemes[1:]:
            diff = [f for f in fields if other.get(f) != first.get(f)]
            if diff:
                raise ValueError(f"[prismaquant] {prefix}: fused roles differ in {diff}; one method cannot "
                                 "serve them")
        return first

    def codebooks_for_prefix(self, prefix: str, scheme: dict) -> list[list[torch.Tensor]]:
        """Tables of every role of ``prefix`` in shard order (one entry for a plain Linear or a
        routed stack).  Roles that share one ``codebook_ref`` collapse to a single entry."""
        base = prefix
        for tail in (".w13", ".w2"):
            if prefix.endswith(tail):
                refs = scheme.get("_role_refs")
                if tail == ".w13" and refs and json.dumps(refs[0]) != json.dumps(refs[1]):
                    return [self._tables(dict(scheme, codebook_ref=r)) for r in refs]
                return [self._tables(scheme)]
        keys = self.shard_target_keys(base, unfused_fallback=True)
        schemes = [self._lookup(k) or scheme for k in keys]
        refs = [json.dumps(s["codebook_ref"]) for s in schemes]
        if len(set(refs)) == 1:
            return [self._tables(schemes[0])]
        return [self._tables(s) for s in schemes]

    def _moe_scheme_for_prefix(self, prefix: str):
        """(gate_up scheme, down scheme) of a routed stack, or None
        (gridbook/config.py:1605-1641).  Unlike the reference, the two projections may differ.
        The gate_up scheme may come from a fused `gate_up_proj` target (one book for both roles)
        or from separate `gate_proj` / `up_proj` targets with their own books
        (docs/SPEC.md:480-527); then it carries `_role_refs`, the codebook_ref of each role."""
        self._ensure_resolved()
        # Per-expert format groups (targets ending in `.format_group_N`: some experts of the stack
        # in another format) are not served, and must be refused BY NAME: matching on the final
        # component would skip them in silence and resolve the stack from whatever else matched
        # (the reference refuses the same crossing, gridbook/config.py:1605-1641).
        for stored in self.target_scheme:
            tail = stored.rsplit(".format_group_", 1)
            if len(tail) == 2 and tail[1].isdigit():
                for leaf in ("gate_proj", "up_proj", "gate_up_proj", "down_proj"):
                    if self._find({tail[0]: True}, f"{prefix}.{leaf}"):
                        raise NativeKernelUnavailableError(
                            f"[prismaquant] {prefix}: target {stored!r} is a per-expert format group; stacks whose "
                            "experts differ in format are not served by gridbook_b200")
        fused = self._lookup(f"{prefix}.gate_up_proj")
        gate, up_role = self._lookup(f"{prefix}.gate_proj"), self._lookup(f"{prefix}.up_proj")
        down = self._lookup(f"{prefix}.down_proj")
        if fused is None and gate is None and up_role is None and down is None:
            return None
        if (gate is None) != (up_role is None):
            raise ValueError(f"[prismaquant] {prefix}: only one of gate_proj / up_proj is a CB target; a role "
                             "is left without a book")
        if fused is not None and gate is not None:
            for name, role in (("gate", gate), ("up", up_role)):
                if json.dumps(role.get("codebook_ref")) != json.dumps(fused.get("codebook_ref")):
                    raise ValueError(f"[prismaquant] {prefix}: gate_up_proj and {name}_proj claim the {name} role "
                                     "with different codebooks")
        up = fused
        if up is None and gate is not None:
            fields = ("grid", "mode", "k", "n_sub", "type_size", "scale_coding", "activation_contract")
            diff = [f for f in fields if gate.get(f) != up_role.get(f)]
            if diff:
                raise ValueError(f"[prismaquant] {prefix}: gate_proj and up_proj differ in {diff}; only the "
                                 "codebook may differ between the roles of a routed stack")
            up = dict(gate)
            up["_role_refs"] = [gate["codebook_ref"], up_role["codebook_ref"]]
        if up is None or down is None:
            raise ValueError(f"[prismaquant] {prefix}: only one of gate_up_proj / down_proj is a CB target")
        return up, down

    # ---- dispatch (gridbook/config.py:1422-1571) --------------------------------------
    def _require_single_gpu_engine(self) -> None:
        """The engine-facing methods serve tensor-parallel size 1 only, like the reference
        (gridbook/config.py:565-576): its loaders never shard the packed rows.  Sharding lives
        beside the engine (peer.py / parallel.py wrap the stand-alone modules)."""
        if getattr(self, "_tp_checked", False):
            return
        world = _engine_tensor_parallel_world_size()
        if world is None:
            return
        if world != 1:
            raise ValueError("[prismaquant] gridbook_b200's engine methods support tensor-parallel size 1 only; "
                             f"the live vLLM worker reports TP={world}")
        self._tp_checked = True

    def get_quant_method(self, layer, prefix: str):
        self._ensure_resolved()
        self._require_single_gpu_engine()
        if self._is_ignored(prefix):
            return _unquantized(layer)
        kind = type(layer).__name__
        if "MoE" in kind or "RoutedExperts" in kind or prefix.endswith(_MOE_SUFFIXES):
            pair = self._moe_scheme_for_prefix(prefix)
            if pair is None:
                return _unquantized(layer)
            from .moe import PrismaQuantCBMoEMethod
            return PrismaQuantCBMoEMethod(self, getattr(layer, "moe_config", None), pair[0], prefix,
                                          scheme_down=pair[1])
        scheme = self._scheme_for_prefix(prefix)
        if scheme is None:
            for key in self.shard_target_keys(prefix, unfused_fallback=True):
                gname = self._delegated_group(key)
                if gname is not None:
                    raise NativeKernelUnavailableError(
                        f"[prismaquant] {prefix}: group {gname!r} carries no codebook scheme (a stock or "
                        "passthrough group); delegated groups are not served by gridbook_b200")
            return _unquantized(layer)
        from .linear import PrismaQuantCBLinearMethod
        return PrismaQuantCBLinearMethod(self, scheme, prefix)


def _engine_tensor_parallel_world_size():
    """TP world size of a live vLLM worker, None when no engine (or no initialised group) is there."""
    if not HAVE_VLLM:
        return None
    try:
        from vllm.distributed import parallel_state
        if not parallel_state.model_parallel_is_initialized():
            return None
        return int(parallel_state.get_tensor_model_parallel_world_size())
    except Exception:            # pragma: no cover - depends on the installed vLLM
        return None


def _unquantized(layer):
    """Non-CB modules keep vLLM's own unquantized method (None lets the engine choose)."""
    if HAVE_VLLM:
        try:
            from vllm.model_executor.layers.linear import LinearBase, UnquantizedLinearMethod
            if isinstance(layer, LinearBase):
                return UnquantizedLinearMethod()
        except Exception:            # pragma: no cover
            pass
    return None
