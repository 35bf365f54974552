"""Target and ignore resolution across the namespaces a module name arrives in, on CPU: the cases the
reference pins in tests/test_target_namespace_compat.py.  A shipped artifact stores its targets as
`model.language_model.layers.N...`, newer ones as `model.layers.N...`, and a wrapper-class engine
model probes with `language_model.model.layers.N...`; all three must name the same Linear or routed
stack, without turning the match into a substring test.  The ignore list reads like the engine's
compressed-tensors matcher: literal entries are exact, `re:` entries are `re.match`ed, a fused
module is judged by its checkpoint shards."""
import pytest

from gridbook_b200.config import PrismaQuantConfig, _candidate_bases, _canonical_prefix, _canonical_target

SCHEME = {"grid": "fp8", "mode": "product", "k": 44, "n_sub": 4, "type_size": 176, "group_size": 0, "vec_dim": 8,
          "codebook_ref": ["cb.mlp.0", "cb.mlp.1", "cb.mlp.2", "cb.mlp.3"]}
NAMESPACES = ["language_model.model.", "model.", "model.language_model."]


def _config(groups, ignore=()):
    cfg = PrismaQuantConfig.from_config({
        "quant_method": "prismaquant", "format": "nvfp4_cb", "codebook_file": "cb_codebooks.pqcb",
        "config_groups": {name: {"format": "FP8_CB_K44", "targets": list(targets), "scheme": dict(SCHEME)}
                          for name, targets in groups.items()},
        "ignore": list(ignore)})
    cfg._ensure_resolved()
    return cfg


def _dense():
    return _config({"old_form": ["model.language_model.layers.0.mlp.gate_proj", "model.language_model.layers.0.mlp.up_proj",
                                 "model.language_model.layers.0.mlp.down_proj", "visual.blocks.0.mlp.down_proj"],
                    "new_form": ["model.layers.1.mlp.down_proj"]},
                   ignore=["model.language_model.layers.0.mlp.foo", "lm_head"])


def test_canonical_rules_and_agreement_of_both_sides():
    assert _canonical_target("model.language_model.layers.3.mlp.gate_proj") == "model.layers.3.mlp.gate_proj"
    assert _canonical_target("language_model.model.layers.3.mlp.gate_proj") == "model.layers.3.mlp.gate_proj"
    assert _canonical_prefix("language_model.layers.3.mlp.gate_proj") == "model.layers.3.mlp.gate_proj"
    assert _canonical_prefix("layers.3.ffn.experts") == "model.layers.3.ffn.experts"      # keys without `model.`
    for name in ("visual.blocks.0.mlp.down_proj", "mtp.layers.0.mlp.up_proj", "model.layers.0.mlp.up_proj", "lm_head"):
        assert _canonical_target(name) == name
    assert {_canonical_prefix(ns + "layers.0.mlp.gate_up_proj") for ns in NAMESPACES} == {"model.layers.0.mlp.gate_up_proj"}
    assert _candidate_bases("model.layers.0.x") == ["model.layers.0.x"]
    assert _candidate_bases("language_model.model.layers.0.x") == ["language_model.model.layers.0.x", "model.layers.0.x"]


def test_old_form_targets_are_normalised_at_parse():
    cfg = _dense()
    for key in ("model.layers.0.mlp.gate_proj", "model.layers.0.mlp.down_proj", "model.layers.1.mlp.down_proj",
                "visual.blocks.0.mlp.down_proj"):
        assert key in cfg.target_scheme
    assert not any(t.startswith("model.language_model.") for t in cfg.target_scheme)


@pytest.mark.parametrize("ns", NAMESPACES)
def test_dense_targets_resolve_in_every_namespace(ns):
    cfg = _dense()
    assert cfg._scheme_for_prefix(ns + "layers.0.mlp.gate_up_proj") is not None      # re-fused from its roles
    assert cfg._scheme_for_prefix(ns + "layers.0.mlp.down_proj") is not None
    assert cfg._scheme_for_prefix(ns + "layers.1.mlp.down_proj") is not None          # the new-form group
    assert cfg._scheme_for_prefix(ns + "layers.2.mlp.down_proj") is None
    assert cfg.shard_target_keys(ns + "layers.0.mlp.gate_up_proj") == [ns + "layers.0.mlp.gate_proj",
                                                                       ns + "layers.0.mlp.up_proj"]
    assert cfg._is_ignored(ns + "layers.0.mlp.foo") and not cfg._is_ignored(ns + "layers.0.mlp.down_proj")


def test_a_second_tower_with_the_same_tail_does_not_pick_up_the_scheme():
    cfg = _dense()
    assert cfg._scheme_for_prefix("vision_tower.layers.0.mlp.down_proj") is None
    assert cfg._scheme_for_prefix("visual.blocks.0.mlp.down_proj") is not None
    assert cfg._scheme_for_prefix("visual.blocks.1.mlp.down_proj") is None


@pytest.mark.parametrize("stored", ["model.language_model.", "model."])
@pytest.mark.parametrize("ns", NAMESPACES)
def test_routed_stack_resolves_across_namespaces(stored, ns):
    cfg = _config({"moe": [stored + "layers.1.mlp.experts.gate_up_proj", stored + "layers.1.mlp.experts.down_proj"]},
                  ignore=["lm_head"])
    pair = cfg._moe_scheme_for_prefix(ns + "layers.1.mlp.experts")
    assert pair is not None and pair[0]["k"] == SCHEME["k"] and pair[1]["k"] == SCHEME["k"]
    assert cfg._moe_scheme_for_prefix(ns + "layers.2.mlp.experts") is None
    assert cfg._moe_scheme_for_prefix(ns + "layers.1.mlp.shared_expert") is None      # a dense MLP beside it


@pytest.mark.parametrize("neighbour", ["experts2", "experts_backup"])
@pytest.mark.parametrize("ns", NAMESPACES)
def test_routed_lookup_needs_a_dotted_boundary(neighbour, ns):
    cfg = _config({"moe": [f"model.layers.1.mlp.{neighbour}.gate_up_proj", f"model.layers.1.mlp.{neighbour}.down_proj"]})
    assert cfg._moe_scheme_for_prefix(ns + "layers.1.mlp.experts") is None
    assert cfg._moe_scheme_for_prefix(ns + f"layers.1.mlp.{neighbour}") is not None


@pytest.mark.parametrize("ns", NAMESPACES)
def test_an_ignored_router_gate_does_not_swallow_the_gate_projections(ns):
    """Exporters collapse `.mlp.router.gate` to `.mlp.gate`, a raw substring of the quantised
    `.mlp.gate_proj` / `.mlp.gate_up_proj`."""
    cfg = _config({"cb": ["model.layers.0.mlp.down_proj"]}, ignore=["model.layers.1.mlp.gate"])
    assert cfg._is_ignored(ns + "layers.1.mlp.gate")
    assert not cfg._is_ignored(ns + "layers.1.mlp.gate_proj")
    assert not cfg._is_ignored(ns + "layers.1.mlp.gate_up_proj")


def test_literal_ignore_entries_are_exact():
    cfg = _config({"cb": ["model.layers.0.mlp.down_proj"]}, ignore=["model.layers.0.mlp", "lm_head"])
    assert cfg._is_ignored("model.layers.0.mlp") and cfg._is_ignored("lm_head")
    for name in ("model.layers.0.mlp.down_proj", "model.layers.0.mlp.shared_mlp.up_proj", "model.layers.01.mlp.down_proj",
                 "model.layers.0.mlp_extra.down_proj", "lm_head_proj", "model.lm_head"):
        assert not cfg._is_ignored(name), name


def test_regex_ignore_entries_are_matched_from_the_start_not_in_full():
    cfg = _config({"cb": ["model.layers.0.mlp.down_proj"]}, ignore=[r"re:model\.layers\.\d+\.mlp\.gate$"])
    assert cfg._is_ignored("model.layers.7.mlp.gate")
    assert not cfg._is_ignored("model.layers.7.mlp.gate_proj")
    assert not cfg._is_ignored("prefix.model.layers.7.mlp.gate")                 # anchored at the start ...
    tail = _config({"cb": ["model.layers.0.mlp.down_proj"]}, ignore=[r"re:model\.layers\.0"])
    assert tail._is_ignored("model.layers.0.mlp.down_proj")                      # ... but not at the end


def test_a_fused_module_is_judged_by_its_checkpoint_shards():
    cb = {"cb": ["model.layers.0.mlp.down_proj"]}
    assert not _config(cb, ignore=[r"re:.*gate_up_proj$"])._is_ignored("model.layers.0.mlp.gate_up_proj")
    assert _config(cb, ignore=[r"re:.*gate_proj$", r"re:.*up_proj$"])._is_ignored("model.layers.0.mlp.gate_up_proj")
    with pytest.raises(ValueError, match="different quantization schemes"):
        _config(cb, ignore=[r"re:.*gate_proj$"])._is_ignored("model.layers.0.mlp.gate_up_proj")


def test_the_engine_mapper_renames_literal_entries_and_never_sees_a_pattern():
    cfg = _config({"cb": ["model.layers.0.mlp.down_proj"]}, ignore=[r"re:.*\.mlp\.gate$", "model.layers.0.mlp.foo"])

    class LiteralOnlyMapper:
        def apply_list(self, names):
            assert all(not n.startswith("re:") for n in names)
            return ["mapped." + n for n in names]

        def apply_dict(self, values):
            return {"mapped." + k: v for k, v in values.items()}

    cfg.apply_vllm_mapper(LiteralOnlyMapper())
    assert cfg.ignore == [r"re:.*\.mlp\.gate$", "mapped.model.layers.0.mlp.foo"]
    assert cfg._scheme_for_prefix("mapped.model.layers.0.mlp.down_proj") is not None   # the string as given comes first
    assert cfg._is_ignored("mapped.model.layers.0.mlp.foo")
    assert cfg._is_ignored("language_model.model.layers.9.mlp.gate")
    assert not cfg._is_ignored("language_model.model.layers.9.mlp.gate_proj")


def test_get_quant_method_uses_the_same_resolution(monkeypatch):
    from gridbook_b200.linear import PrismaQuantCBLinearMethod
    from gridbook_b200.moe import PrismaQuantCBMoEMethod
    cfg = _config({"dense": ["model.language_model.layers.0.mlp.gate_proj", "model.language_model.layers.0.mlp.up_proj"],
                   "moe": ["model.language_model.layers.1.mlp.experts.gate_up_proj",
                           "model.language_model.layers.1.mlp.experts.down_proj"]},
                  ignore=["model.language_model.layers.0.mlp.gate"])

    class Linear:
        pass

    class RoutedExperts:
        pass

    m = cfg.get_quant_method(Linear(), "language_model.model.layers.0.mlp.gate_up_proj")
    assert isinstance(m, PrismaQuantCBLinearMethod)
    e = cfg.get_quant_method(RoutedExperts(), "language_model.model.layers.1.mlp.experts")
    assert isinstance(e, PrismaQuantCBMoEMethod)
    assert not isinstance(cfg.get_quant_method(Linear(), "language_model.model.layers.0.mlp.gate"),
                          PrismaQuantCBLinearMethod)
    assert not isinstance(cfg.get_quant_method(Linear(), "language_model.model.layers.5.mlp.gate_up_proj"),
                          PrismaQuantCBLinearMethod)


@pytest.mark.parametrize("leaf,members", [("qkv_proj", ("q_proj", "k_proj", "v_proj")), ("gate_up_proj", ("gate_proj", "up_proj")),
                                          ("in_proj_qkvz", ("in_proj_qkv", "in_proj_z")), ("in_proj_ba", ("in_proj_b", "in_proj_a")),
                                          ("fused_wqa_wkv", ("wq_a", "wkv"))])
def test_every_fused_family_is_refused_from_its_checkpoint_roles(leaf, members):
    """The fused modules the reference knows without the engine's help (gridbook/config.py:117-132),
    also when the engine's own mapping has replaced the default one."""
    base = "model.layers.7.mod."
    cfg = _config({"cb": [base + m for m in members]})
    for ns in ("", "language_model."):
        assert cfg._scheme_for_prefix(ns + base + leaf) is not None
        assert cfg.shard_target_keys(ns + base + leaf) == [ns + base + m for m in members]
    cfg.packed_modules_mapping = {"something_else": ["a", "b"]}                  # what an engine may publish
    assert cfg._scheme_for_prefix(base + leaf) is not None
    cfg.packed_modules_mapping = {leaf: list(reversed(members))}                 # the engine's order wins
    assert cfg.shard_target_keys(base + leaf) == [base + m for m in reversed(members)]


def test_alternate_checkpoint_spellings_are_tried_after_the_primary_one():
    """`w1` / `w3` fuse into the same gate_up_proj, `w2` is the down projection
    (gridbook/config.py:134-158): consulted only when the primary spelling finds nothing, and a
    spelling wins whole."""
    base = "model.layers.3.mlp.shared_experts."
    alt = _config({"cb": [base + "w1", base + "w3", base + "w2"]})
    assert alt.shard_target_keys(base + "gate_up_proj") == [base + "w1", base + "w3"]
    assert alt.shard_target_keys(base + "down_proj") == [base + "w2"]
    assert alt.shard_target_keys(base + "gate_proj") == [base + "w1"] and alt.shard_target_keys(base + "up_proj") == [base + "w3"]
    assert alt._scheme_for_prefix(base + "gate_up_proj") is not None
    both = _config({"cb": [base + "gate_proj", base + "up_proj", base + "w1", base + "w3"]})
    assert both.shard_target_keys(base + "gate_up_proj") == [base + "gate_proj", base + "up_proj"]
    with pytest.raises(ValueError, match="mixed fused modules"):
        _config({"cb": [base + "w1"]}).shard_target_keys(base + "gate_up_proj")
    assert _config({"cb": [base + "w9"]}).shard_target_keys(base + "gate_up_proj") == []
    assert _config({"cb": [base + "w9"]}).shard_target_keys(base + "gate_up_proj", unfused_fallback=True) == [base + "gate_up_proj"]
