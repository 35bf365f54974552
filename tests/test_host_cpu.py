"""Host-side logic that needs no GPU: the C-ABI library loads and exports every symbol the
header declares, the loader fails closed, config resolution, plugin registration with a
stubbed registry, the layer registry and the padding sentinel."""
import ctypes
import ctypes.util
import gc
import json
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "gridbook_b200.h")).read()
    return sorted(set(re.findall(r"GB_API\s+[\w\s\*]+?\b(gb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from gridbook_b200 import _native, build
    build.build()
    lib = ctypes.CDLL(_native.library_path())
    declared = _header_symbols()
    assert len(declared) >= 16
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(_native.REQUIRED_SYMBOLS) <= set(declared)
    assert _native.load().gb_abi_version() == _native.GB_ABI_VERSION


def test_loader_fails_closed(monkeypatch, tmp_path):
    from gridbook_b200 import _native
    monkeypatch.setattr(_native, "_LIB", None)
    monkeypatch.setenv("GRIDBOOK_B200_LIB", str(tmp_path / "missing.so"))
    with pytest.raises(_native.NativeKernelUnavailableError, match="missing"):
        _native.load("unit test")
    # a library without the required symbols is a stale extension
    monkeypatch.setenv("GRIDBOOK_B200_LIB", ctypes.util.find_library("m") and "/lib/x86_64-linux-gnu/libm.so.6")
    with pytest.raises(_native.NativeKernelUnavailableError):
        _native.load("unit test")
    monkeypatch.delenv("GRIDBOOK_B200_LIB")
    assert _native.load() is not None


def test_argument_validation_without_a_device():
    """Validation runs before any CUDA call, so bad descriptors are reported on a CPU box."""
    from gridbook_b200 import _native as nat
    lib = nat.load()
    fmt = nat.GbFormat(grid=0, mode=0, k_bits=16, n_sub=2, type_size=70, scale_coding=2)
    w = nat.GbWeight(qw=1, row_stride=73, codebook=1, cb_row_offset=None, compose=1, weight_scale=None,
                     global_scale=1.0, rows=8, K=256, fmt=fmt)
    rc = lib.gb_expand_fp4_bf16(ctypes.byref(w), 0, 8, ctypes.c_void_p(1), None)
    assert rc == 1 and b"type_size" in lib.gb_last_error()
    w.fmt.type_size = 73
    w.K = 250
    rc = lib.gb_expand_fp4_bf16(ctypes.byref(w), 0, 8, ctypes.c_void_p(1), None)
    assert rc == 1 and b"multiple of 256" in lib.gb_last_error()
    assert lib.gb_gemv_workspace_bytes(16, 1024, 512) == 16 * 512 * 2 + 16 * 1024 * 4
    assert lib.gb_gemv_workspace_bytes(1, 4096, 8192) == 8 * 4096 * 4      # M = 1: one slot per K slice


def test_kernels_refuse_cpu_tensors():
    from gridbook_b200 import kernels, ops
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernels.fp8_act_qdq(torch.zeros(2, 32, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        ops.fp4_act_qdq_or_codec(torch.zeros(2, 32, dtype=torch.bfloat16))


def _quant_config():
    two_tier = {"kind": "two_tier", "table": [1.0, 1.125, 1.25, 1.375, 1.5, 1.625, 1.75, 1.875,
                                              2.0, 2.25, 2.5, 2.75, 3.0, 3.25, 3.5, 3.75]}
    fp4 = {"grid": "fp4", "mode": "product", "k": 16, "n_sub": 2, "type_size": 73,
           "codebook_ref": ["cb.K16.sub0", "cb.K16.sub1"], "scale_coding": two_tier}
    fp4_b = dict(fp4, codebook_ref=["cb.K16b.sub0", "cb.K16b.sub1"])
    fp8 = {"grid": "fp8", "mode": "product", "k": 32, "n_sub": 4, "type_size": 128,
           "codebook_ref": [f"cb.F32.sub{i}" for i in range(4)]}
    return {
        "quant_method": "gridbook", "format": "nvfp4_cb", "layout_version": 2,
        "config_groups": {
            "g0": {"targets": ["model.layers.0.self_attn.q_proj", "model.layers.0.self_attn.k_proj",
                               "model.layers.0.self_attn.v_proj", "model.layers.0.mlp.gate_proj"], "scheme": fp4},
            "g1": {"targets": ["model.layers.0.mlp.up_proj"], "scheme": fp4_b},
            "g2": {"targets": ["model.layers.0.self_attn.o_proj", "model.layers.1.mlp.experts.gate_up_proj"],
                   "scheme": fp8},
            "g3": {"targets": ["model.layers.1.mlp.experts.down_proj"], "scheme": fp4},
        },
        "ignore": ["lm_head"],
    }


def test_config_resolution_inline_and_pointer(tmp_path):
    from gridbook_b200.config import PrismaQuantConfig
    from gridbook_b200.linear import PrismaQuantCBLinearMethod
    from gridbook_b200.moe import PrismaQuantCBMoEMethod
    assert PrismaQuantConfig.override_quantization_method({"quant_method": "prismaquant"}, None) == "gridbook"
    assert PrismaQuantConfig.override_quantization_method({"quant_method": "awq"}, None) is None
    assert PrismaQuantConfig.get_name() == "gridbook"

    full = _quant_config()
    books = {n: torch.zeros(256, 4) for n in ("cb.K16.sub0", "cb.K16.sub1", "cb.K16b.sub0", "cb.K16b.sub1")}
    books.update({f"cb.F32.sub{i}": torch.zeros(256, 2) for i in range(4)})
    cfg = PrismaQuantConfig.from_config(dict(full, _codebooks=books))

    class Linear(torch.nn.Module):
        pass

    class FusedMoE(torch.nn.Module):
        pass

    m = cfg.get_quant_method(Linear(), "model.layers.0.self_attn.qkv_proj")
    assert isinstance(m, PrismaQuantCBLinearMethod) and m.fmt.type_size == 73
    assert cfg.shard_target_keys("model.layers.0.self_attn.qkv_proj") == [
        "model.layers.0.self_attn.q_proj", "model.layers.0.self_attn.k_proj", "model.layers.0.self_attn.v_proj"]
    assert len(cfg.codebooks_for_prefix("model.layers.0.self_attn.qkv_proj", m.scheme)) == 1     # shared book
    gu = cfg.get_quant_method(Linear(), "model.layers.0.mlp.gate_up_proj")
    assert len(cfg.codebooks_for_prefix("model.layers.0.mlp.gate_up_proj", gu.scheme)) == 2      # per-role books
    assert cfg.get_quant_method(Linear(), "model.layers.0.self_attn.o_proj").fmt.grid == "fp8"
    assert cfg.get_quant_method(Linear(), "lm_head") is None
    assert cfg.get_quant_method(Linear(), "model.layers.7.mlp.down_proj") is None
    moe = cfg.get_quant_method(FusedMoE(), "model.layers.1.mlp.experts")
    assert isinstance(moe, PrismaQuantCBMoEMethod) and moe.fmt13.grid == "fp8" and moe.fmt2.grid == "fp4"
    # class-wrapper prefixes resolve to the stored keys
    assert cfg.get_quant_method(Linear(), "language_model.model.layers.0.self_attn.o_proj") is not None

    # pointer stub -> quant_config.json in the model directory
    (tmp_path / "quant_config.json").write_text(json.dumps(full))
    ptr = PrismaQuantConfig({"quant_method": "gridbook", "config_file": "quant_config.json"}, str(tmp_path))
    assert ptr.get_quant_method(Linear(), "model.layers.0.self_attn.o_proj").type_size == 128
    with pytest.raises(ValueError, match="model directory"):
        PrismaQuantConfig({"quant_method": "gridbook"}).get_quant_method(Linear(), "x")


def test_scheme_parsing_and_type_size_guard():
    from gridbook_b200.formats import CBFormat
    f = CBFormat.from_scheme({"grid": "fp4", "k": 13, "n_sub": 1, "type_size": 61,
                              "scale_coding": "two_tier"})
    assert f.mode == "signed" and f.scale_coding == "v2"
    assert CBFormat.from_scheme({"grid": "fp4", "mode": "full", "k": 8, "n_sub": 1}).type_size == 48
    assert CBFormat("fp8", 30, n_sub=4).widths() == [8, 8, 7, 7]
    with pytest.raises(ValueError, match="type_size"):
        CBFormat.from_scheme({"grid": "fp8", "k": 32, "n_sub": 4, "type_size": 120})


def test_codec_rejects_off_grid_codebooks():
    from gridbook_b200 import codec
    with pytest.raises(ValueError, match="off the E2M1 grid"):
        codec.build_flat_codebook([torch.tensor([[0.53125, 1.0, 2.0, 6.0]])], grid="fp4")
    with pytest.raises(ValueError, match="off the E4M3 grid"):
        codec.build_flat_codebook([torch.tensor([[0.3, 1.0]])], grid="fp8")
    flat = codec.build_flat_codebook([torch.tensor([[0.5, -6.0, 3.0, 0.0]])], grid="fp4")
    assert flat.dtype is torch.bfloat16 and flat.tolist() == [0.5, -6.0, 3.0, 0.0]
    assert codec.pad_qweight(torch.zeros(3, 73, dtype=torch.uint8)).shape == (3, 89)
    assert codec.build_compose_table()[127 * 16 + 9].item() == 2.25


@pytest.mark.parametrize("grid,name", [("fp4", "E2M1 grid"), ("fp8", "E4M3 grid")])
@pytest.mark.parametrize("value", [0.53125, float("nan"), float("inf")])
def test_codec_grid_validation_rejects_malformed_tables_at_load(grid, name, value):
    """Behaviour the reference pins in tests/test_fail_loud.py:224-246: an off-grid, NaN or infinite
    entry is refused at load with the grid or "non-finite" named; a learned table that sits on the
    grid is accepted even if it is not the deterministic lattice."""
    from gridbook_b200 import codec
    with pytest.raises(ValueError, match=f"{name}|non-finite"):
        codec.build_flat_codebook([torch.tensor([0.0, -0.5, value], dtype=torch.float32)], "some.layer", grid)
    ok = codec.build_flat_codebook([torch.tensor([-6.0, -1.5, -0.0, 0.5, 3.0])], "learned", grid)
    assert ok.dtype is torch.bfloat16


def test_codec_cast_check_names_layer_count_and_measured_errors(monkeypatch, capsys):
    """The lossy-cast error of the reference (tests/test_fail_loud.py:127-222): it names the layer and
    the cast, counts the entries that moved and prints the measured maximum absolute and relative
    error; float64 input is not rounded before the check; the environment override turns the error
    into a warning."""
    from gridbook_b200 import codec
    monkeypatch.delenv("PRISMAQUANT_SKIP_CB_CAST_CHECK", raising=False)
    on_grid = (torch.arange(64, dtype=torch.float32) / 64.0 - 0.5).to(torch.float8_e4m3fn).to(torch.bfloat16)
    codec.assert_cast_lossless(on_grid, on_grid.to(torch.float8_e4m3fn), "e4m3 flat", "t")
    assert codec.flat_codebook_fp8(on_grid).dtype is torch.uint8

    flat = on_grid[:8].float().clone()
    flat[3] = 0.53125                                  # between the E4M3 codes 0.5 and 0.5625
    cast = flat.to(torch.float8_e4m3fn)
    with pytest.raises(ValueError) as e:
        codec.assert_cast_lossless(flat, cast, "e4m3 flat", "model.layers.3.mlp.experts.w13")
    msg = str(e.value)
    got = float(cast.float()[3])
    for part in ("LOSSY", "model.layers.3.mlp.experts.w13", "e4m3 flat", "1 of 8 table values do not survive it",
                 f"max abs {abs(0.53125 - got):.3e}", f"max rel {abs(0.53125 - got) / 0.53125:.3e}",
                 "PRISMAQUANT_SKIP_CB_CAST_CHECK=1"):
        assert part in msg, part

    with pytest.raises(ValueError, match="bf16 flat"):
        codec.build_flat_codebook([torch.tensor([1.0000001], dtype=torch.float32)], "dense.layer")
    with pytest.raises(ValueError, match="bf16 flat"):                   # mixed dtypes, one lossy
        codec.build_flat_codebook([torch.tensor([[1.0000001, 2.0]]), torch.tensor([[0.5]], dtype=torch.bfloat16)])
    with pytest.raises(ValueError, match="bf16 flat"):
        codec.build_flat_codebook([torch.tensor([1.0 + 2.0 ** -40], dtype=torch.float64)], "float64.layer")
    with pytest.raises(ValueError, match="e4m3 flat"):
        codec.flat_codebook_fp8(torch.tensor([0.53125], dtype=torch.bfloat16), "dense.layer")

    monkeypatch.setenv("PRISMAQUANT_SKIP_CB_CAST_CHECK", "1")
    codec.assert_cast_lossless(flat, cast, "e4m3 flat", "t")             # must not raise
    err = capsys.readouterr().err
    assert "WARNING" in err and "LOSSY" in err


def test_plugin_registers_both_names():
    from gridbook_b200 import plugin
    from gridbook_b200.config import PrismaQuantConfig
    seen = {}

    def registry(name):
        def deco(cls):
            seen[name] = cls
            return cls
        return deco

    plugin.register(registry)
    assert seen == {"gridbook": PrismaQuantConfig, "prismaquant": PrismaQuantConfig}


def test_layer_registry_is_weak_and_monotonic():
    from gridbook_b200 import ops

    class Obj:
        pass

    m, l = Obj(), Obj()
    a = ops.register_cb_layer(m, l)
    b = ops.register_cb_layer(m, l)
    assert b > a and ops._lookup_cb_layer(a) == (m, l)
    del l
    gc.collect()
    with pytest.raises(RuntimeError, match="stale or unknown"):
        ops._lookup_cb_layer(a)


def test_padding_sentinel_is_neutralised():
    from gridbook_b200 import ops
    w = torch.tensor([[0.5, 0.5], [float("nan"), 1.0]])
    ids = torch.tensor([[3, -1], [-1, 2]])
    w2, ids2 = ops._neutralize_moe_padding_sentinel(w, ids)
    assert ids2.tolist() == [[3, 0], [0, 2]] and w2.tolist() == [[0.5, 0.0], [0.0, 1.0]]


def test_methods_fail_closed_before_load():
    from gridbook_b200._native import NativeKernelUnavailableError
    from gridbook_b200.formats import NVFP4_CB_K16
    from gridbook_b200.linear import CBLinear
    lin = CBLinear(NVFP4_CB_K16, 512, [16], [[torch.zeros(256, 4), torch.zeros(256, 4)]])
    assert lin.cb_qweight.shape == (16, 2 * 73)
    with pytest.raises(NativeKernelUnavailableError, match="not registered"):
        lin(torch.zeros(1, 512, dtype=torch.bfloat16))
    with pytest.raises(NativeKernelUnavailableError, match="biased"):
        lin.method.apply(lin, torch.zeros(1, 512), bias=torch.zeros(16))
    with pytest.raises(NativeKernelUnavailableError, match="CUDA device"):
        lin.method.process_weights_after_loading(lin)


def test_peer_role_slices_agree_with_the_gather_permutation():
    """The peer all-gather writes rank s's slice of every role at gcol + s * width; that must be
    the column order the NCCL path reaches through its permutation."""
    import torch
    from gridbook_b200 import parallel, peer
    for parts, world in (([6144], 2), ([1024, 1024], 4), ([512, 256, 256], 2), ([17408, 17408], 8)):
        roles = peer.role_slices(parts, world)
        n_local = sum(p // world for p in parts)
        full = torch.full((sum(parts),), -1, dtype=torch.int64)
        for s in range(world):
            for lcol, gcol, w in roles:
                full[gcol + s * w: gcol + (s + 1) * w] = s * n_local + lcol + torch.arange(w)
        assert torch.equal(full, parallel.gather_permutation(parts, world))
    with pytest.raises(ValueError):
        peer.role_slices([10], 4)


def _write_artifact(tmp_path, books, provenance="auto", tensors=None):
    """A minimal published directory: pointer stub, assignment, sidecar (+ optional tensors)."""
    from safetensors.torch import save_file
    from gridbook_b200.artifact import codebook_sha256
    full = _quant_config()
    if provenance == "auto":
        full["provenance"] = {"codebook_sha256": {n: codebook_sha256(t) for n, t in books.items()}}
    elif provenance is not None:
        full["provenance"] = {"codebook_sha256": provenance}
    (tmp_path / "config.json").write_text(json.dumps({"quantization_config": {"quant_method": "gridbook"}}))
    (tmp_path / "quant_config.json").write_text(json.dumps(full))
    save_file({n: t.to(torch.float16).contiguous() for n, t in books.items()}, str(tmp_path / "cb_codebooks.pqcb"))
    if tensors:
        save_file(tensors, str(tmp_path / "model.safetensors"))
    return full


def _books():
    g = torch.Generator().manual_seed(0)
    books = {n: torch.randint(-6, 7, (256, 4), generator=g).float() * 0.5
             for n in ("cb.K16.sub0", "cb.K16.sub1", "cb.K16b.sub0", "cb.K16b.sub1")}
    books.update({f"cb.F32.sub{i}": torch.randint(-8, 9, (256, 2), generator=g).float() for i in range(4)})
    return books


def test_artifact_codebook_digests(tmp_path):
    """Declared digests must cover the sidecar exactly and match; no declaration loads unchecked;
    an empty declaration is not the same as none (docs/SPEC.md:326-378)."""
    from gridbook_b200.artifact import Artifact, codebook_sha256
    books = _books()
    good = tmp_path / "good"
    good.mkdir()
    _write_artifact(good, books, tensors={"model.layers.0.self_attn.o_proj.cb_qweight":
                                          torch.zeros(4, 128, dtype=torch.uint8)})
    art = Artifact(str(good))
    assert art.has("model.layers.0.self_attn.o_proj.cb_qweight") and not art.has("nope")
    assert art.tensor("model.layers.0.self_attn.o_proj.cb_qweight").shape == (4, 128)
    assert art.config.get_quant_method(torch.nn.Identity(), "lm_head") is None
    # the digest is the SHA-256 of the fp16 row-major bytes
    import hashlib
    t = books["cb.K16.sub0"]
    assert codebook_sha256(t) == hashlib.sha256(t.to(torch.float16).numpy().tobytes()).hexdigest()

    undeclared = tmp_path / "undeclared"
    undeclared.mkdir()
    _write_artifact(undeclared, books, provenance=None)
    Artifact(str(undeclared))

    digests = {n: codebook_sha256(t) for n, t in books.items()}
    cases = {
        "wrong": dict(digests, **{"cb.K16.sub1": "0" * 64}),
        "missing": {n: d for n, d in digests.items() if n != "cb.F32.sub3"},
        "extra": dict(digests, **{"cb.ghost": "1" * 64}),
        "empty": {},
        "malformed": dict(digests, **{"cb.K16.sub0": "XYZ"}),
    }
    for tag, mapping in cases.items():
        d = tmp_path / tag
        d.mkdir()
        _write_artifact(d, books, provenance=mapping)
        with pytest.raises(ValueError, match="prismaquant"):
            Artifact(str(d))
    # a sidecar swapped for another intact one with the same names fails too
    swapped = tmp_path / "swapped"
    swapped.mkdir()
    _write_artifact(swapped, books, provenance=digests)
    from safetensors.torch import save_file
    other = {n: (t + 0.5).to(torch.float16) for n, t in books.items()}
    save_file(other, str(swapped / "cb_codebooks.pqcb"))
    with pytest.raises(ValueError, match="does not match"):
        Artifact(str(swapped))
    with pytest.raises(ValueError, match="no gridbook"):
        bad = tmp_path / "plain"
        bad.mkdir()
        (bad / "config.json").write_text("{}")
        Artifact(str(bad))


def test_scale_coding_comes_from_the_group_not_from_layout_version():
    """A layout_version-2 artifact may hold v1 groups: absence of scale_coding means E4M3-direct
    bytes (docs/SPEC.md:130-177), and mixed v1 / v2 groups resolve side by side."""
    from gridbook_b200.config import PrismaQuantConfig
    v1 = {"grid": "fp4", "mode": "product", "k": 16, "n_sub": 2, "type_size": 80, "codebook_ref": ["a", "b"]}
    v2 = {"grid": "fp4", "mode": "product", "k": 16, "n_sub": 2, "type_size": 73, "codebook_ref": ["a", "b"],
          "scale_coding": {"kind": "two_tier"}}
    cfg = PrismaQuantConfig({"quant_method": "gridbook", "layout_version": 2, "config_groups": {
        "old": {"targets": ["model.layers.0.mlp.down_proj"], "scheme": v1},
        "new": {"targets": ["model.layers.1.mlp.down_proj"], "scheme": v2}},
        "_codebooks": {"a": torch.zeros(256, 4), "b": torch.zeros(256, 4)}})

    class Linear(torch.nn.Module):
        pass

    old = cfg.get_quant_method(Linear(), "model.layers.0.mlp.down_proj")
    new = cfg.get_quant_method(Linear(), "model.layers.1.mlp.down_proj")
    assert old.fmt.scale_coding == "v1" and old.fmt.type_size == 80 and not old.is_v2
    assert new.fmt.scale_coding == "v2" and new.fmt.type_size == 73 and new.is_v2


def test_fused_roles_must_share_scale_coding_and_stock_groups_are_named():
    from gridbook_b200._native import NativeKernelUnavailableError
    from gridbook_b200.config import PrismaQuantConfig
    base = {"grid": "fp4", "mode": "product", "k": 16, "n_sub": 2, "codebook_ref": ["a", "b"]}
    v1 = dict(base, type_size=80)
    v2 = dict(base, type_size=73, scale_coding={"kind": "two_tier"})
    v2_other_table = dict(base, type_size=73, scale_coding={"kind": "two_tier", "table": [1.0] * 16})
    groups = {
        "g0": {"targets": ["model.layers.0.self_attn.q_proj", "model.layers.0.self_attn.k_proj"], "scheme": v2},
        "g1": {"targets": ["model.layers.0.self_attn.v_proj"], "scheme": v2_other_table},
        "g2": {"targets": ["model.layers.0.mlp.gate_proj"], "scheme": v2},
        "g3": {"targets": ["model.layers.0.mlp.up_proj"], "scheme": dict(v2, activation_contract="static_nvfp4")},
        "stock": {"targets": ["model.layers.0.self_attn.o_proj"], "format": "float-quantized"},
        "tower": {"targets": ["layers.3.mlp.down_proj"], "scheme": v1},
    }
    cfg = PrismaQuantConfig({"quant_method": "gridbook", "config_groups": groups})

    class Linear(torch.nn.Module):
        pass

    with pytest.raises(ValueError, match="scale_coding"):
        cfg.get_quant_method(Linear(), "model.layers.0.self_attn.qkv_proj")
    with pytest.raises(ValueError, match="activation_contract"):
        cfg.get_quant_method(Linear(), "model.layers.0.mlp.gate_up_proj")
    with pytest.raises(NativeKernelUnavailableError, match="delegated groups are not served"):
        cfg.get_quant_method(Linear(), "model.layers.0.self_attn.o_proj")
    # suffix matches need a known wrapper prefix: another tower with the same tail is not a target
    assert cfg.get_quant_method(Linear(), "model.layers.3.mlp.down_proj") is not None
    assert cfg.get_quant_method(Linear(), "vision_tower.layers.3.mlp.down_proj") is None


def test_routed_method_fails_closed_on_other_activations_and_weights_on_input():
    from gridbook_b200._native import NativeKernelUnavailableError
    from gridbook_b200.moe import PrismaQuantCBMoEMethod
    scheme = {"grid": "fp4", "mode": "full", "k": 8, "n_sub": 1, "type_size": 48}
    method = PrismaQuantCBMoEMethod(None, None, scheme, "model.layers.0.mlp.experts")

    class Act:
        def __init__(self, value):
            self.value = value

    class Layer(torch.nn.Module):
        pass

    gelu = Layer()
    gelu.activation = Act("gelu")
    with pytest.raises(NativeKernelUnavailableError, match="activation 'gelu'"):
        method.process_weights_after_loading(gelu)
    on_input = Layer()
    on_input.activation = Act("silu")
    on_input.apply_router_weight_on_input = True
    with pytest.raises(NativeKernelUnavailableError, match="apply_router_weight_on_input"):
        method.process_weights_after_loading(on_input)
    ok = Layer()
    ok.activation = Act("silu")
    ok._cb_layer_id = 1
    x, w, ids = torch.zeros(1, 8), torch.zeros(1, 2), torch.zeros(1, 2, dtype=torch.int32)
    with pytest.raises(NativeKernelUnavailableError, match="apply_router_weight_on_input"):
        method.apply(ok, x, w, ids, apply_router_weight_on_input=True)
    ok.apply_router_weight_on_input = True
    with pytest.raises(NativeKernelUnavailableError, match="apply_router_weight_on_input"):
        method.apply(ok, x, w, ids)
    ok.apply_router_weight_on_input = False
    with pytest.raises(NativeKernelUnavailableError, match="expert_map"):
        method.apply(ok, x, w, ids, expert_map=torch.arange(4))
    with pytest.raises(NativeKernelUnavailableError, match="activation"):
        method.apply(ok, x, w, ids, activation="gelu")


def test_per_role_routed_codebooks_resolve_and_conflicts_refuse():
    """gate_proj / up_proj / down_proj as separate targets with their own books
    (docs/SPEC.md:480-527): w13 gets two role books, w2 one; a role claimed twice with different
    books, or a role without a book, is refused."""
    from gridbook_b200.config import PrismaQuantConfig
    from gridbook_b200.moe import PrismaQuantCBMoEMethod

    def scheme(ref):
        return {"grid": "fp8", "mode": "product", "k": 32, "n_sub": 4, "type_size": 128,
                "codebook_ref": [f"{ref}.{i}" for i in range(4)]}

    books = {f"{r}.{i}": torch.full((256, 2), float(j)) for j, r in enumerate(("g", "u", "d")) for i in range(4)}
    pre = "model.layers.1.mlp.experts"
    groups = {"a": {"targets": [f"{pre}.gate_proj"], "scheme": scheme("g")},
              "b": {"targets": [f"{pre}.up_proj"], "scheme": scheme("u")},
              "c": {"targets": [f"{pre}.down_proj"], "scheme": scheme("d")}}
    cfg = PrismaQuantConfig({"quant_method": "gridbook", "config_groups": groups, "_codebooks": books})

    class FusedMoE(torch.nn.Module):
        pass

    m = cfg.get_quant_method(FusedMoE(), pre)
    assert isinstance(m, PrismaQuantCBMoEMethod)
    r13 = cfg.codebooks_for_prefix(f"{pre}.w13", m.scheme)
    r2 = cfg.codebooks_for_prefix(f"{pre}.w2", m.scheme_down)
    assert len(r13) == 2 and len(r2) == 1
    assert float(r13[0][0][0, 0]) == 0.0 and float(r13[1][0][0, 0]) == 1.0 and float(r2[0][0][0, 0]) == 2.0
    # the same book for both roles collapses to a uniform stack
    same = dict(groups, b={"targets": [f"{pre}.up_proj"], "scheme": scheme("g")})
    cfg2 = PrismaQuantConfig({"quant_method": "gridbook", "config_groups": same, "_codebooks": books})
    m2 = cfg2.get_quant_method(FusedMoE(), pre)
    assert len(cfg2.codebooks_for_prefix(f"{pre}.w13", m2.scheme)) == 1
    # a role left without a book / claimed twice with different books
    missing = {k: v for k, v in groups.items() if k != "b"}
    with pytest.raises(ValueError, match="without a book"):
        PrismaQuantConfig({"quant_method": "gridbook", "config_groups": missing}).get_quant_method(FusedMoE(), pre)
    twice = dict(groups, d={"targets": [f"{pre}.gate_up_proj"], "scheme": scheme("u")})
    with pytest.raises(ValueError, match="different codebooks"):
        PrismaQuantConfig({"quant_method": "gridbook", "config_groups": twice}).get_quant_method(FusedMoE(), pre)
    other_k = dict(groups, b={"targets": [f"{pre}.up_proj"], "scheme": dict(scheme("u"), k=28, type_size=112)})
    with pytest.raises(ValueError, match="differ in"):
        PrismaQuantConfig({"quant_method": "gridbook", "config_groups": other_k}).get_quant_method(FusedMoE(), pre)


def test_engine_methods_refuse_a_tensor_parallel_world(monkeypatch):
    """Like the reference (gridbook/config.py:565-576): the engine-facing methods serve TP = 1 only."""
    from gridbook_b200 import config as C
    v2 = {"grid": "fp4", "mode": "product", "k": 16, "n_sub": 2, "type_size": 73, "codebook_ref": ["a", "b"],
          "scale_coding": {"kind": "two_tier"}}
    raw = {"quant_method": "gridbook", "config_groups": {"g": {"targets": ["m.down_proj"], "scheme": v2}},
           "_codebooks": {"a": torch.zeros(256, 4), "b": torch.zeros(256, 4)}}

    class Linear(torch.nn.Module):
        pass

    monkeypatch.setattr(C, "_engine_tensor_parallel_world_size", lambda: 2)
    with pytest.raises(ValueError, match="tensor-parallel size 1 only"):
        C.PrismaQuantConfig(dict(raw)).get_quant_method(Linear(), "m.down_proj")
    monkeypatch.setattr(C, "_engine_tensor_parallel_world_size", lambda: 1)
    assert C.PrismaQuantConfig(dict(raw)).get_quant_method(Linear(), "m.down_proj") is not None
    monkeypatch.setattr(C, "_engine_tensor_parallel_world_size", lambda: None)       # no engine: stand-alone use
    assert C.PrismaQuantConfig(dict(raw)).get_quant_method(Linear(), "m.down_proj") is not None


def test_padded_superblock_layout_keeps_the_bytes_and_the_oracle_reads_it():
    """Two-tier superblocks moved into 80-byte slots (the resident layout the tensor-core decode kernel
    fetches by TMA): the format reports the stride as its type_size and the shipped size as its packed
    size, the padding is zero, and the oracle decodes the padded rows to the same weights."""
    import numpy as np
    from gridbook_b200 import codec, formats, synth
    from oracle import cb_oracle as O, oracle_kwargs
    fmt = formats.NVFP4_CB_K16
    pad = fmt.padded(80)
    assert (fmt.type_size, pad.type_size, pad.packed_type_size, pad.sb_pad) == (73, 80, 73, 7)
    assert pad.bits_per_weight() == fmt.bits_per_weight() and pad.packed_row_bytes(1024) == 4 * 73
    assert pad.row_bytes(1024) == 4 * 80 and pad.to_native().type_size == 80
    with pytest.raises(ValueError):
        fmt.padded(96)
    d = synth.make_linear(fmt, 6, 1024, seed=3)
    q80 = codec.pad_superblocks(torch.from_numpy(d["qw"]), 73, 80)
    assert q80.shape == (6, 320)
    blocks = q80.reshape(6, 4, 80)
    assert torch.equal(blocks[..., :73].reshape(6, -1), torch.from_numpy(d["qw"])) and int(blocks[..., 73:].sum()) == 0
    off = np.zeros(6, np.int32)
    w73 = O.reconstruct_weight(d["qw"], d["cb"], off, N=6, K=1024, compose=d["compose"], **oracle_kwargs(fmt))
    w80 = O.reconstruct_weight(q80.numpy(), d["cb"], off, N=6, K=1024, compose=d["compose"], **oracle_kwargs(pad))
    assert np.array_equal(w73, w80)
    with pytest.raises(ValueError):
        codec.pad_superblocks(torch.zeros(2, 100, dtype=torch.uint8), 73, 80)


def _cpu_weight(fmt, rows=256, K=1024, experts=1, offsets=False):
    """A PackedWeight over CPU tensors: enough for the route predicates, which look at formats,
    strides and alignment only."""
    from gridbook_b200.kernels import PackedWeight
    rb = fmt.row_bytes(K)
    qw = torch.zeros((experts, rows, rb) if experts > 1 else (rows, rb), dtype=torch.uint8)
    cb = torch.zeros(4096, dtype=torch.bfloat16 if fmt.is_fp4 else torch.uint8)
    return PackedWeight(qw, cb, fmt, K, rows, rb, torch.zeros(rows, dtype=torch.int32) if offsets else None, None,
                        None if fmt.is_fp4 else torch.ones(rows), 1.0, rows * rb if experts > 1 else 0, experts)


def test_route_predicates_follow_the_formats_the_kernels_decode():
    """Which stacks take the sorted-rows tensor-core route and which the per-pair table kernel: the
    literal fp4 format has both; the two-tier k = 16 format only in 80-byte superblock slots; the fp8
    product formats k = 32 / k = 16; nothing with per-role codebooks or rows that are not whole
    128-row tiles."""
    from gridbook_b200 import formats as F, kernels
    lit, k16, f32, f16 = F.NVFP4_LITERAL, F.NVFP4_CB_K16, F.FP8_CB_K32, F.FP8_LITERAL
    assert kernels.moe_gemv_sorted_applies(_cpu_weight(lit, experts=4))
    assert kernels.pair_kernel_applies(_cpu_weight(lit, experts=4))
    assert not kernels.moe_gemv_sorted_applies(_cpu_weight(k16, experts=4))            # 73-byte superblocks
    assert kernels.moe_gemv_sorted_applies(_cpu_weight(k16.padded(80), experts=4))
    assert not kernels.pair_kernel_applies(_cpu_weight(k16.padded(80), experts=4))
    assert kernels.moe_gemv_sorted_applies(_cpu_weight(f32, experts=4))
    assert kernels.moe_gemv_sorted_applies(_cpu_weight(f16, experts=4))
    assert not kernels.moe_gemv_sorted_applies(_cpu_weight(F.CBFormat("fp8", 30, n_sub=4), experts=4))
    assert not kernels.moe_gemv_sorted_applies(_cpu_weight(lit, rows=192, experts=4))   # not whole 128-row tiles
    assert not kernels.moe_gemv_sorted_applies(_cpu_weight(lit, experts=4, offsets=True))


def test_routed_method_thresholds_are_instance_attributes_with_the_measured_defaults():
    from gridbook_b200 import moe
    assert (moe.SORTED_MIN_PAIRS_PER_EXPERT, moe.SORTED_MIN_PAIRS_OTHER) == (4, 16)
    assert moe.PREFILL_MIN_PAIRS_PER_EXPERT > moe.PREFILL_MIN_PAIRS_OTHER > moe.SORTED_MIN_PAIRS_PER_EXPERT
    src = open(moe.__file__).read()
    for attr in ("pair_kernel_max_pairs", "sorted_min_pairs_per_expert", "sorted_min_pairs_other",
                 "prefill_min_pairs_per_expert", "prefill_min_pairs_other", "pad_two_tier_superblocks"):
        assert f"self.{attr} = " in src, attr


def _routed_cfg(groups, books=None):
    from gridbook_b200.config import PrismaQuantConfig
    raw = {"quant_method": "gridbook", "config_groups": {f"g{i}": {"targets": list(t), "scheme": s}
                                                          for i, (t, s) in enumerate(groups)}}
    if books is not None:
        raw["_codebooks"] = books
    return PrismaQuantConfig(raw)


def _k28(*refs):
    return {"grid": "fp8", "mode": "product", "k": 28, "n_sub": 4, "type_size": 112, "codebook_ref": list(refs)}


def test_uniform_routed_stack_is_one_role_however_its_targets_are_spelled():
    """The cases of the reference's tests/test_routed_per_role_codebooks.py:63-127 on this resolver:
    one book for the whole stack - written as gate_up_proj + down_proj in one group, or as the three
    unfused role names - is a uniform stack (one role for gate_up, one for down, the same book); a
    fused gate_up_proj target speaks for gate AND up while down carries its own book."""
    pre = "model.layers.1.mlp.experts"
    leaf = lambda n: f"{pre}.{n}"                                   # noqa: E731
    refs = [f"cb.routed.K28.sub{i}" for i in range(4)]
    books = {r: torch.full((128, 2), 3.0) for r in refs}
    for targets in ([leaf("gate_up_proj"), leaf("down_proj")], [leaf("gate_proj"), leaf("up_proj"), leaf("down_proj")]):
        cfg = _routed_cfg([(targets, _k28(*refs))], books)
        up, down = cfg._moe_scheme_for_prefix(pre)
        assert up["codebook_ref"] == refs and down["codebook_ref"] == refs
        assert len(cfg.codebooks_for_prefix(f"{pre}.w13", up)) == 1
        assert len(cfg.codebooks_for_prefix(f"{pre}.w2", down)) == 1
    w13 = [f"cb.l1.w13.sub{i}" for i in range(4)]
    dn = [f"cb.l1.down.sub{i}" for i in range(4)]
    books = {**{r: torch.full((128, 2), 1.0) for r in w13}, **{r: torch.full((128, 2), 2.0) for r in dn}}
    cfg = _routed_cfg([([leaf("gate_up_proj")], _k28(*w13)), ([leaf("down_proj")], _k28(*dn))], books)
    up, down = cfg._moe_scheme_for_prefix(pre)
    r13, r2 = cfg.codebooks_for_prefix(f"{pre}.w13", up), cfg.codebooks_for_prefix(f"{pre}.w2", down)
    assert len(r13) == 1 and float(r13[0][0][0, 0]) == 1.0 and float(r2[0][0][0, 0]) == 2.0


@pytest.mark.parametrize("leaf_name", ["gate_proj", "gate_up_proj", "down_proj"])
def test_role_crossed_with_a_per_expert_format_group_is_refused_by_name(leaf_name):
    """tests/test_routed_per_role_codebooks.py:165-182 of the reference: a `...<leaf>.format_group_0`
    target must not be skipped in silence.  A neighbouring stack's group does not trip the guard."""
    from gridbook_b200._native import NativeKernelUnavailableError
    pre = "model.layers.1.mlp.experts"
    refs = [f"r{i}" for i in range(4)]
    cfg = _routed_cfg([([f"{pre}.gate_up_proj", f"{pre}.down_proj"], _k28(*refs)),
                       ([f"{pre}.{leaf_name}.format_group_0"], _k28(*refs))])
    with pytest.raises(NativeKernelUnavailableError, match="per-expert format group"):
        cfg._moe_scheme_for_prefix(pre)
    other = _routed_cfg([([f"{pre}.gate_up_proj", f"{pre}.down_proj"], _k28(*refs)),
                         ([f"model.layers.2.mlp.experts.{leaf_name}.format_group_0"], _k28(*refs))])
    assert other._moe_scheme_for_prefix(pre) is not None


def test_codebook_digest_known_answers():
    """The reference's own known-answer vectors for the table digest (tests/test_codebook_digest.py:94-120):
    SHA-256 of the fp16 row-major bytes, whatever the dtype and the strides of the tensor handed in."""
    import hashlib
    import struct
    from gridbook_b200.artifact import codebook_sha256
    table = torch.tensor([0.0, 1.0, -2.0, 0.5], dtype=torch.float32)
    assert struct.pack("<4e", 0.0, 1.0, -2.0, 0.5).hex() == "0000003c00c00038"
    assert codebook_sha256(table) == "58e0b63dabbfe62f04be297478992b1c1d301fc4c3c4c1c8abe3f431b322cce5"
    source = torch.arange(24, dtype=torch.float32).reshape(4, 6).t()        # not contiguous
    want = hashlib.sha256(struct.pack("<24e", *source.to(torch.float16).contiguous().reshape(-1).tolist())).hexdigest()
    assert codebook_sha256(source) == want == codebook_sha256(source.to(torch.float64))
    assert codebook_sha256(torch.empty(0)) == hashlib.sha256(b"").hexdigest()


def test_routed_method_parameter_shapes_and_checkpoint_hook():
    """The stacked-parameter contract the reference pins in tests/test_moe_stacked.py:77-106 and the
    instance load hook of gridbook/moe.py:503-546: w13 = [E, 2I, row_bytes(H)], w2 = [E, H, row_bytes(I)],
    per-(expert, row) fp32 scales on the fp8 grid only; checkpoint tensors named <proj>.cb_qweight /
    <proj>.weight_scale go straight into the stacked parameters, a shape that breaks the contract is
    refused by name, everything else reaches the layer's own loader."""
    from gridbook_b200.moe import PrismaQuantCBMoEMethod, _row_bytes
    E, hidden, inter, k, ts = 8, 512, 1024, 44, 176
    scheme = {"grid": "fp8", "mode": "product", "k": k, "n_sub": 4, "type_size": ts, "codebook_ref": ["cb.x"]}
    method = PrismaQuantCBMoEMethod(None, None, scheme, "model.layers.0.mlp.experts")
    seen = []

    class Layer(torch.nn.Module):
        def load_weights(self, weights):
            for name, _ in weights:
                seen.append(name)
                yield name

    layer = Layer()
    method.create_weights(layer, E, hidden, inter, torch.bfloat16, weight_loader=None)
    assert layer.w13_cb_qweight.shape == (E, 2 * inter, _row_bytes(hidden, ts)) and layer.w13_cb_qweight.dtype is torch.uint8
    assert layer.w2_cb_qweight.shape == (E, hidden, _row_bytes(inter, ts))
    assert layer.w13_weight_scale.shape == (E, 2 * inter) and layer.w13_weight_scale.dtype is torch.float32
    assert layer.w2_weight_scale.shape == (E, hidden)
    assert not layer.w13_cb_qweight.requires_grad
    with pytest.raises(ValueError, match="multiple of 256"):
        _row_bytes(300, ts)

    w13 = torch.randint(0, 256, tuple(layer.w13_cb_qweight.shape), dtype=torch.uint8)
    s2 = torch.rand(E, hidden)
    loaded = list(layer.load_weights([("gate_up_proj.cb_qweight", w13), ("down_proj.weight_scale", s2),
                                      ("gate.weight", torch.zeros(2))]))
    assert loaded == ["w13_cb_qweight", "w2_weight_scale", "gate.weight"] and seen == ["gate.weight"]
    assert torch.equal(layer.w13_cb_qweight.data, w13) and torch.equal(layer.w2_weight_scale.data, s2)
    with pytest.raises(ValueError, match=r"down_proj\.cb_qweight.*stacked"):
        list(layer.load_weights([("down_proj.cb_qweight", torch.zeros(E, hidden, 3, dtype=torch.uint8))]))

    fp4 = PrismaQuantCBMoEMethod(None, None, {"grid": "fp4", "mode": "product", "k": 16, "n_sub": 2, "type_size": 73,
                                              "scale_coding": "two_tier"}, "model.layers.1.mlp.experts")
    l4 = Layer()
    fp4.create_weights(l4, 4, 512, 256, torch.bfloat16)
    assert l4.w13_cb_qweight.shape == (4, 512, 2 * 73) and l4.w2_cb_qweight.shape == (4, 512, 73)
    assert not hasattr(l4, "w13_weight_scale") and not hasattr(l4, "w2_weight_scale")


def test_linear_method_parameter_shapes():
    """create_weights of the linear method (gridbook/linear.py:233-273): one packed parameter of
    [sum of the fused shards' rows, row_bytes(K)] bytes, a per-row fp32 scale on the fp8 grid only,
    in_features a multiple of the superblock."""
    from gridbook_b200.linear import PrismaQuantCBLinearMethod
    fp8 = PrismaQuantCBLinearMethod(None, {"grid": "fp8", "mode": "product", "k": 32, "n_sub": 4, "type_size": 128},
                                    "model.layers.0.self_attn.qkv_proj")
    layer = torch.nn.Module()
    fp8.create_weights(layer, 1024, [64, 16, 16], 1024, 96, torch.bfloat16, weight_loader=None)
    assert layer.cb_qweight.shape == (96, 4 * 128) and layer.cb_qweight.dtype is torch.uint8
    assert layer.weight_scale.shape == (96,) and layer.weight_scale.dtype is torch.float32
    assert layer.logical_widths == [64, 16, 16]
    fp4 = PrismaQuantCBLinearMethod(None, {"grid": "fp4", "mode": "product", "k": 16, "n_sub": 2, "type_size": 73,
                                           "scale_coding": "two_tier"}, "model.layers.0.mlp.down_proj")
    l4 = torch.nn.Module()
    fp4.create_weights(l4, 768, [32], 768, 32, torch.bfloat16)
    assert l4.cb_qweight.shape == (32, 3 * 73) and not hasattr(l4, "weight_scale")
    with pytest.raises(ValueError, match="multiple of 256"):
        fp4.create_weights(torch.nn.Module(), 300, [32], 300, 32, torch.bfloat16)


def test_static_activation_contract_parameters_load_and_the_gate_fails_closed():
    """A scheme that declares the static NVFP4 activation contract ships `input_global_scale`
    tensors (gridbook/linear.py:214-218,252-267,348-372; gridbook/moe.py:423-427,492-500,560-594):
    the parameters exist so the checkpoint loads, start as NaN so a tensor that never arrived is
    seen, and the gate after loading wants one finite positive scale per module, bit-identical
    across the logical shards.  The declaration is fp4-only and names one known contract."""
    from gridbook_b200 import codec
    from gridbook_b200.linear import PrismaQuantCBLinearMethod
    from gridbook_b200.moe import PrismaQuantCBMoEMethod
    fp4 = {"grid": "fp4", "mode": "product", "k": 16, "n_sub": 2, "type_size": 73, "scale_coding": "two_tier",
           "activation_contract": "nvfp4_w4a4"}
    m = PrismaQuantCBLinearMethod(None, fp4, "model.layers.0.self_attn.qkv_proj")
    layer = torch.nn.Module()
    m.create_weights(layer, 512, [32, 16, 16], 512, 64, torch.bfloat16, weight_loader=None)
    assert layer.input_global_scale.shape == (3,) and layer.input_global_scale.dtype is torch.float32
    assert bool(torch.isnan(layer.input_global_scale).all())
    with pytest.raises(ValueError, match="finite positive"):            # nothing was loaded
        m.process_weights_after_loading(layer)
    layer.input_global_scale.data.copy_(torch.tensor([0.5, 0.5, 0.25]))
    with pytest.raises(ValueError, match="non-identical input_global_scale"):
        m.process_weights_after_loading(layer)
    layer.input_global_scale.data.fill_(0.5)
    m._finalize_static_activation_scale(layer)
    assert layer._cb_fp4_input_global_scale_f32 == 0.5
    del layer.input_global_scale
    with pytest.raises(ValueError, match="no input_global_scale parameter"):
        m._finalize_static_activation_scale(layer)
    plain = PrismaQuantCBLinearMethod(None, {k: v for k, v in fp4.items() if k != "activation_contract"}, "p")
    l2 = torch.nn.Module()
    plain.create_weights(l2, 512, [32], 512, 32, torch.bfloat16)
    assert not hasattr(l2, "input_global_scale")
    plain._finalize_static_activation_scale(l2)                          # nothing to check

    with pytest.raises(ValueError, match="fp4-only"):
        PrismaQuantCBLinearMethod(None, {"grid": "fp8", "mode": "product", "k": 32, "n_sub": 4, "type_size": 128,
                                         "activation_contract": "nvfp4_w4a4"}, "x")
    with pytest.raises(ValueError, match="unsupported activation_contract 'other'"):
        PrismaQuantCBLinearMethod(None, dict(fp4, activation_contract="other"), "x")
    with pytest.raises(ValueError, match="nonempty 1-D float32"):
        codec.loaded_static_activation_scale(torch.zeros(2, 2), "x")
    with pytest.raises(ValueError, match="finite positive"):
        codec.loaded_static_activation_scale(torch.tensor([-0.0, 0.0]), "x")  # equal values, different bits

    moe = PrismaQuantCBMoEMethod(None, None, fp4, "model.layers.1.mlp.experts")

    class Layer(torch.nn.Module):
        def load_weights(self, weights):
            yield from (name for name, _ in weights)

    ml = Layer()
    moe.create_weights(ml, 4, 512, 256, torch.bfloat16)
    assert ml.w13_input_global_scale.shape == (1,) and bool(torch.isnan(ml.w2_input_global_scale).all())
    with pytest.raises(ValueError, match=r"experts\.w13\.input_global_scale.*finite positive"):
        moe._finalize_static_activation_scales(ml)
    loaded = list(ml.load_weights([("gate_up_proj.input_global_scale", torch.tensor([2.0])),
                                   ("down_proj.input_global_scale", torch.tensor([4.0]))]))
    assert loaded == ["w13_input_global_scale", "w2_input_global_scale"]
    moe._finalize_static_activation_scales(ml)
    assert (ml._cb_fp4_input_global_scale_w13_f32, ml._cb_fp4_input_global_scale_w2_f32) == (2.0, 4.0)
    with pytest.raises(ValueError, match="stacked"):
        list(ml.load_weights([("down_proj.input_global_scale", torch.tensor(4.0))]))   # a 0-d tensor breaks the contract


def test_expert_stacks_that_were_never_filled_are_refused_after_loading():
    """The guard the reference pins in tests/test_cb_fill_guard.py: create_weights allocates
    uninitialised stacks, and a model class whose loader never hands them to this layer would serve
    that memory without any error.  Every fill path stamps the parameter; after loading, a registered
    non-empty stack without the stamp is refused by name - before any native library is touched, with
    no override.  Absent or empty stacks prove nothing and are skipped."""
    from gridbook_b200 import moe as M
    scheme = {"grid": "fp4", "mode": "full", "k": 8, "n_sub": 1, "type_size": 48}
    method = M.PrismaQuantCBMoEMethod(None, None, scheme, "model.layers.0.mlp.experts")

    class Layer(torch.nn.Module):
        def load_weights(self, weights):
            yield from (name for name, _ in weights)

    layer = Layer()
    method.create_weights(layer, 2, 256, 256, torch.bfloat16)
    assert M.unfilled_cb_params(layer) == ["w13_cb_qweight", "w2_cb_qweight"]
    with pytest.raises(RuntimeError, match=r"\['w13_cb_qweight', 'w2_cb_qweight'\] were REGISTERED but never FILLED"):
        method.process_weights_after_loading(layer)
    list(layer.load_weights([("gate_up_proj.cb_qweight", torch.zeros(2, 512, 48, dtype=torch.uint8))]))
    assert M.unfilled_cb_params(layer) == ["w2_cb_qweight"]                 # the hook stamps what it fills
    with pytest.raises(RuntimeError, match=r"\['w2_cb_qweight'\] were REGISTERED"):
        method.process_weights_after_loading(layer)
    layer.w2_cb_qweight.data = torch.zeros(2, 256, 48, dtype=torch.uint8)   # a direct fill ...
    assert M.unfilled_cb_params(layer) == ["w2_cb_qweight"]
    M.mark_filled(layer.w2_cb_qweight)                                      # ... has to say so
    assert M.unfilled_cb_params(layer) == []
    method._assert_experts_filled(layer)

    empty = Layer()
    method.create_weights(empty, 0, 256, 256, torch.bfloat16)               # no experts on this rank
    assert M.unfilled_cb_params(empty) == [] and M.unfilled_cb_params(Layer()) == []
    foreign = Layer()
    foreign.w13_cb_qweight = torch.nn.Parameter(torch.zeros(1, 4, 48, dtype=torch.uint8), requires_grad=False)
    assert M.unfilled_cb_params(foreign) == ["w13_cb_qweight"]              # no stamp at all: not ours, not filled

    # the stand-alone module's load() stamps both stacks: it gets past the guard and stops at the
    # next gate (no CPU path)
    from gridbook_b200._native import NativeKernelUnavailableError
    from gridbook_b200.formats import CBFormat
    fmt = CBFormat.from_scheme(scheme)
    tabs = [torch.zeros(256, 8)]
    alone = M.CBMoE(fmt, fmt, 2, 256, 256, tabs, tabs)
    with pytest.raises(NativeKernelUnavailableError, match="CUDA device"):
        alone.load(torch.zeros(2, 512, 48, dtype=torch.uint8), torch.zeros(2, 256, 48, dtype=torch.uint8), device="cpu")
    assert M.unfilled_cb_params(alone) == []
