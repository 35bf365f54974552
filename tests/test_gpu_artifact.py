"""A published directory (pointer stub, assignment with codebook digests, safetensors, sidecar)
loaded without an engine and checked against the oracle: a fused gate/up module whose roles use
different codebooks, and a routed expert stack with an FP8 gate/up and an FP4 down projection."""
import json

import numpy as np
import pytest
import torch

from oracle import cb_oracle as O
from oracle import oracle_kwargs
from tests.helpers import assert_close_bf16, f32_of, oracle_linear

pytestmark = pytest.mark.gpu


def _tables(fmt, flat):
    out, pos = [], 0
    for r, d in fmt.table_shapes():
        out.append(torch.from_numpy(np.ascontiguousarray(flat[pos:pos + r * d].reshape(r, d))))
        pos += r * d
    return out


def test_directory_round_trip(tmp_path):
    from safetensors.torch import save_file
    from gridbook_b200 import _native, codec, synth
    from gridbook_b200.artifact import Artifact, codebook_sha256
    from gridbook_b200.formats import FP8_CB_K32, NVFP4_CB_K16
    _native.prepare(0)
    dev = torch.device("cuda:0")
    two_tier = {"kind": "two_tier", "table": list(codec.TWO_TIER_SUB_TABLE)}
    fp4 = NVFP4_CB_K16
    books, tensors, groups = {}, {}, {}

    def scheme(fmt, refs):
        s = {"grid": fmt.grid, "mode": fmt.mode, "k": fmt.k, "n_sub": fmt.n_sub, "type_size": fmt.type_size,
             "codebook_ref": refs}
        if fmt.is_fp4:
            s["scale_coding"] = two_tier
        return s

    # ---- dense: gate_proj and up_proj with their own role codebooks, served as one fused module ----
    N, K = 512, 1024
    d = synth.make_linear(fp4, N, K, seed=4, n_books=2)
    per = fp4.codebook_elems()
    for i, role in enumerate(("gate_proj", "up_proj")):
        refs = [f"cb_codebook.{role}.NVFP4_CB_K16.sub{j}" for j in range(2)]
        for ref, t in zip(refs, _tables(fp4, d["cb"][i * per:(i + 1) * per])):
            books[ref] = t
        tensors[f"model.layers.0.mlp.{role}.cb_qweight"] = torch.from_numpy(d["qw"][i * N // 2:(i + 1) * N // 2].copy())
        groups[f"dense_{role}"] = {"targets": [f"model.layers.0.mlp.{role}"], "scheme": scheme(fp4, refs)}

    # ---- routed stack: FP8 gate/up, FP4 down ----
    E, hidden, inter, T, topk = 8, 512, 256, 6, 2
    w13d, w2d = synth.make_moe(FP8_CB_K32, fp4, E, hidden, inter, seed=6)
    refs13 = [f"cb_codebook.experts_up.FP8_CB_K32.sub{j}" for j in range(4)]
    refs2 = [f"cb_codebook.experts_down.NVFP4_CB_K16.sub{j}" for j in range(2)]
    for ref, t in zip(refs13, _tables(FP8_CB_K32, w13d["cb"])):
        books[ref] = t
    for ref, t in zip(refs2, _tables(fp4, w2d["cb"])):
        books[ref] = t
    pre = "model.layers.1.mlp.experts"
    tensors[f"{pre}.gate_up_proj.cb_qweight"] = torch.from_numpy(w13d["qw"].copy())
    tensors[f"{pre}.gate_up_proj.weight_scale"] = torch.from_numpy(w13d["scale"].copy())
    tensors[f"{pre}.down_proj.cb_qweight"] = torch.from_numpy(w2d["qw"].copy())
    groups["moe_up"] = {"targets": [f"{pre}.gate_up_proj"], "scheme": scheme(FP8_CB_K32, refs13)}
    groups["moe_down"] = {"targets": [f"{pre}.down_proj"], "scheme": scheme(fp4, refs2)}

    full = {"quant_method": "gridbook", "format": "nvfp4_cb", "layout_version": 2, "config_groups": groups,
            "ignore": ["lm_head"],
            "provenance": {"codebook_sha256": {n: codebook_sha256(t) for n, t in books.items()}}}
    (tmp_path / "config.json").write_text(json.dumps({"quantization_config": {"quant_method": "gridbook"}}))
    (tmp_path / "quant_config.json").write_text(json.dumps(full))
    save_file({n: t.to(torch.float16).contiguous() for n, t in books.items()}, str(tmp_path / "cb_codebooks.pqcb"))
    save_file(tensors, str(tmp_path / "model-00001-of-00001.safetensors"))

    art = Artifact(str(tmp_path))
    lin = art.load_linear("model.layers.0.mlp.gate_up_proj", dev)
    x = synth.make_activations(3, K, seed=1)
    y = lin(synth.bf16_tensor(x, dev))
    assert_close_bf16(f32_of(y), oracle_linear(x, d, bucket=True, scale_rule="recip"), "fused module from disk")
    one = art.load_linear("model.layers.0.mlp.up_proj", dev)            # a single role on its own
    y_up = one(synth.bf16_tensor(x, dev))
    assert torch.equal(y_up, y[:, N // 2:])

    moe = art.load_experts(pre, dev)
    ids, tw = synth.make_routing(T, E, topk, seed=3)
    xm = synth.make_activations(T, hidden, seed=2)
    out = moe(synth.bf16_tensor(xm, dev), torch.from_numpy(tw).to(dev), torch.from_numpy(ids).to(dev))
    ref = O.moe_loop_chain(xm, ids, tw, w13d, w2d, E=E, hidden=hidden, inter=inter,
                           fmt13=oracle_kwargs(FP8_CB_K32), fmt2=oracle_kwargs(fp4), scale_rule="recip")
    got = f32_of(out)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-2
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()
    with pytest.raises(KeyError):
        art.load_linear("lm_head", dev)
