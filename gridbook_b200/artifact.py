"""Loading a published artifact without an engine (docs/SPEC.md:271-399): a directory with
``config.json`` (pointer stub under ``quantization_config``), ``quant_config.json`` (the
assignment), ``*.safetensors`` (``<q>.cb_qweight`` uint8 streams, fp8 ``<q>.weight_scale``) and
the codebook sidecar ``cb_codebooks.pqcb`` (itself a safetensors file).

What an engine does through the plugin surface - resolve the scheme of a prefix, create the
parameters, copy the checkpoint tensors in, prepare after loading - happens here for one Linear
or one routed expert stack at a time, through the same method classes.  The sidecar's tables
are checked against ``provenance.codebook_sha256`` when the assignment carries it
(docs/SPEC.md:326-378; the reference's cb_digest.py)."""
from __future__ import annotations

import glob
import hashlib
import json
import os

import torch

from .config import PrismaQuantConfig


def codebook_sha256(table: torch.Tensor) -> str:
    """The normative digest of one sidecar table: SHA-256 over its fp16, row-major, little-endian
    bytes (docs/SPEC.md:352-362)."""
    raw = table.to(torch.float16).cpu().contiguous().numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()


def verify_codebook_digests(books: dict, expected) -> None:
    """``expected`` is ``provenance.codebook_sha256`` or None.  Absent: nothing to check.  Present:
    it must name the sidecar's tables exactly and every digest must match; an empty mapping is
    not the same as absence (docs/SPEC.md:368-373)."""
    if expected is None:
        return
    if not isinstance(expected, dict):
        raise ValueError("[prismaquant] provenance.codebook_sha256 must be a mapping of table name to digest")
    names, want = set(books), set(expected)
    if names != want:
        raise ValueError(f"[prismaquant] codebook digests do not cover the sidecar exactly: "
                         f"missing {sorted(names - want)}, unknown {sorted(want - names)}")
    for name in sorted(names):
        digest = expected[name]
        if not (isinstance(digest, str) and len(digest) == 64 and all(c in "0123456789abcdef" for c in digest)):
            raise ValueError(f"[prismaquant] malformed digest for {name}")
        got = codebook_sha256(books[name])
        if got != digest:
            raise ValueError(f"[prismaquant] codebook {name} does not match its recorded digest "
                             f"(sidecar {got[:12]}..., config {digest[:12]}...)")


class Artifact:
    """One model directory: its resolved quantization config and a name -> file index of its
    tensors (read lazily, tensor by tensor)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        with open(os.path.join(model_dir, "config.json")) as fh:
            hf = json.load(fh)
        stub = hf.get("quantization_config")
        if not stub or stub.get("quant_method") not in ("gridbook", "prismaquant"):
            raise ValueError(f"[prismaquant] {model_dir}/config.json carries no gridbook quantization_config")
        self.config = PrismaQuantConfig(stub, model_dir)
        self.config.get_codebooks()                 # resolves, reads the sidecar, checks the digests
        self._index: dict[str, str] = {}
        from safetensors import safe_open
        for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
            with safe_open(path, framework="pt") as f:
                for key in f.keys():
                    self._index[key] = path

    def tensor(self, name: str) -> torch.Tensor:
        from safetensors import safe_open
        path = self._index.get(name)
        if path is None:
            raise KeyError(f"[prismaquant] tensor {name} is not in {self.model_dir}")
        with safe_open(path, framework="pt") as f:
            return f.get_tensor(name)

    def has(self, name: str) -> bool:
        return name in self._index

    # ------------------------------------------------------------------ modules
    def load_linear(self, prefix: str, device="cuda") -> torch.nn.Module:
        """The Linear (or fused module: its roles' rows concatenated in shard order) under
        ``prefix`` as a callable module on ``device``."""
        from .linear import PrismaQuantCBLinearMethod
        cfg = self.config
        scheme = cfg._scheme_for_prefix(prefix)
        if scheme is None:
            raise KeyError(f"[prismaquant] {prefix} is not a codebook target of this artifact")
        keys = cfg.shard_target_keys(prefix)
        parts = [self.tensor(f"{k}.cb_qweight") for k in keys]
        method = PrismaQuantCBLinearMethod(cfg, scheme, prefix)
        in_features = parts[0].shape[1] // method.fmt.type_size * 256
        sizes = [int(p.shape[0]) for p in parts]
        module = _Loaded(method)
        method.create_weights(module, in_features, sizes, in_features, sum(sizes), torch.bfloat16)
        module.cb_qweight.data = torch.cat(parts, dim=0).to(device)
        if not method.fmt.is_fp4:
            module.weight_scale.data = torch.cat([self.tensor(f"{k}.weight_scale") for k in keys]).to(device)
        if method.has_static_fp4_activation:     # one calibrated scale per role; the gate wants them identical
            module.input_global_scale.data = torch.cat(
                [self.tensor(f"{k}.input_global_scale").reshape(-1).float() for k in keys]).to(device)
        method.process_weights_after_loading(module)
        return module

    def load_experts(self, prefix: str, device="cuda") -> torch.nn.Module:
        """The routed expert stack under ``prefix`` (``<prefix>.gate_up_proj`` / ``.down_proj``
        stacked tensors, docs/SPEC.md:281-289) as a module taking (x, topk_weights, topk_ids)."""
        from .moe import PrismaQuantCBMoEMethod, mark_filled
        cfg = self.config
        pair = cfg._moe_scheme_for_prefix(prefix)
        if pair is None:
            raise KeyError(f"[prismaquant] {prefix} holds no codebook expert stack")
        w13 = self.tensor(f"{prefix}.gate_up_proj.cb_qweight")
        w2 = self.tensor(f"{prefix}.down_proj.cb_qweight")
        method = PrismaQuantCBMoEMethod(cfg, None, pair[0], prefix, scheme_down=pair[1])
        E, two_inter = int(w13.shape[0]), int(w13.shape[1])
        hidden = int(w2.shape[1])
        module = _Loaded(method)
        method.create_weights(module, E, hidden, two_inter // 2, torch.bfloat16)
        module.w13_cb_qweight.data = w13.to(device)
        module.w2_cb_qweight.data = w2.to(device)
        mark_filled(module.w13_cb_qweight)
        mark_filled(module.w2_cb_qweight)
        if not method.fmt13.is_fp4:
            module.w13_weight_scale.data = self.tensor(f"{prefix}.gate_up_proj.weight_scale").to(device)
        if not method.fmt2.is_fp4:
            module.w2_weight_scale.data = self.tensor(f"{prefix}.down_proj.weight_scale").to(device)
        for which, proj in (("w13", "gate_up_proj"), ("w2", "down_proj")):
            if method.has_static_fp4_activation[which]:
                getattr(module, f"{which}_input_global_scale").data = self.tensor(
                    f"{prefix}.{proj}.input_global_scale").reshape(-1).float().to(device)
        method.process_weights_after_loading(module)
        return module


class _Loaded(torch.nn.Module):
    """A bare module the method hangs its parameters on; forward = the method's apply."""

    def __init__(self, method):
        super().__init__()
        self.method = method

    def forward(self, *args):
        return self.method.apply(self, *args)
