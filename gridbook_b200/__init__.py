"""gridbook_b200 — sm_100a kernels for the gridbook codebook-decode linear and
routed-MoE hot path, behind the reference's vLLM plugin surface."""
__version__ = "0.2.0"


def register() -> None:
    """vLLM ``general_plugins`` entry point (gridbook/__init__.py:20-22)."""
    from .plugin import register as _register
    _register()
