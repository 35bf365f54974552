"""Base classes and parameter types of the vLLM plugin surface.

Inside a vLLM process (vllm already imported by the engine that is loading this
plugin) the real classes are used, so the methods are drop-ins.  Standalone (tests,
benchmarks, the GPU box without an engine) light stand-ins with the same call
surface are used instead, so the hot path can be driven without importing vLLM."""
from __future__ import annotations

import sys

import torch

HAVE_VLLM = False
if "vllm" in sys.modules:
    try:
        from vllm.model_executor.layers.fused_moe import FusedMoEMethodBase  # type: ignore
        from vllm.model_executor.layers.linear import (LinearMethodBase,  # type: ignore
                                                       register_weight_loader_v2_supported_method)
        from vllm.model_executor.layers.quantization.base_config import QuantizationConfig  # type: ignore
        from vllm.model_executor.parameter import (ChannelQuantScaleParameter,  # type: ignore
                                                   ModelWeightParameter, PerTensorScaleParameter)
        HAVE_VLLM = True
    except Exception:       # pragma: no cover - depends on the installed vLLM
        HAVE_VLLM = False

if not HAVE_VLLM:
    class LinearMethodBase:                       # noqa: D401 - stand-in
        """Stand-in for vllm.model_executor.layers.linear.LinearMethodBase."""

    class FusedMoEMethodBase:
        """Stand-in for vllm...fused_moe.FusedMoEMethodBase."""
        def __init__(self, moe=None):
            self.moe = moe

    class QuantizationConfig:
        """Stand-in for vllm...quantization.base_config.QuantizationConfig."""
        def __init__(self):
            self.packed_modules_mapping = {}

    def register_weight_loader_v2_supported_method(cls):
        return cls

    def _plain(data, **_ignored):
        return torch.nn.Parameter(data, requires_grad=False)

    ModelWeightParameter = ChannelQuantScaleParameter = PerTensorScaleParameter = _plain
