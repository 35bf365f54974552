"""vLLM plugin registration (gridbook/plugin.py:142-166): one quantization config class
under both registry keys.  Nothing else of the reference's plugin module (per-architecture
loader wraps, extension preloading) is part of this path."""
from __future__ import annotations

_REGISTERED = False
QUANT_METHOD_NAMES = ("gridbook", "prismaquant")


def register(registry=None) -> None:
    """Register PrismaQuantConfig.  ``registry`` (a callable ``name -> class decorator``) is
    for tests; by default vLLM's ``register_quantization_config`` is used."""
    global _REGISTERED
    engine = registry is None
    if _REGISTERED and engine:
        return
    from . import _native
    _native.load("gridbook_b200 plugin")           # fail closed at start-up, not at first forward
    if registry is None:
        from vllm.model_executor.layers.quantization import register_quantization_config as registry
    from .config import PrismaQuantConfig
    for name in QUANT_METHOD_NAMES:
        try:
            registry(name)(PrismaQuantConfig)
        except (ValueError, AssertionError) as exc:      # already registered by an earlier load
            if "already" not in str(exc).lower():
                raise
    if engine:
        _REGISTERED = True
