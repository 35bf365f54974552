"""Static ratchet in the manner of the reference's tests/test_no_triton_runtime.py: the product package
is native-only.  Every module of gridbook_b200 is parsed and must not (a) import the CPU oracle,
Triton, tilelang or another kernel library, (b) call torch.compile, (c) compute a linear with a
torch GEMM (F.linear, matmul, mm, bmm, einsum, the @ operator) - a missing library or kernel has to
fail closed, never fall back - and (d) read a working file or the reference checkout.  The CUDA
sources must not name a bulk load that is shared out over a cluster.  No GPU needed."""
import ast
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "gridbook_b200")
MODULES = sorted(f for f in os.listdir(PKG) if f.endswith(".py"))

FORBIDDEN_IMPORTS = ("oracle", "triton", "tilelang", "flash_attn", "flashinfer", "cutlass", "vllm._custom_ops",
                     "jax", "numba")
GEMM_CALLS = {"linear", "matmul", "mm", "bmm", "einsum", "addmm", "baddbmm", "tensordot"}
# host-side generators of synthetic inputs may use numpy freely; they never produce a served result
DATA_ONLY = {"synth.py"}


def _tree(name):
    with open(os.path.join(PKG, name)) as f:
        return ast.parse(f.read(), filename=name)


@pytest.mark.parametrize("name", MODULES)
def test_module_imports_no_checker_and_no_other_kernel_library(name):
    for node in ast.walk(_tree(name)):
        mods = []
        if isinstance(node, ast.Import):
            mods = [a.name for a in node.names]
        elif isinstance(node, ast.ImportFrom) and node.level == 0 and node.module:
            mods = [node.module]
        for m in mods:
            for bad in FORBIDDEN_IMPORTS:
                assert not (m == bad or m.startswith(bad + ".")), f"{name}:{node.lineno} imports {m}"


@pytest.mark.parametrize("name", [m for m in MODULES if m not in DATA_ONLY])
def test_module_has_no_torch_gemm_and_no_compile(name):
    for node in ast.walk(_tree(name)):
        if isinstance(node, ast.BinOp) and isinstance(node.op, ast.MatMult):
            raise AssertionError(f"{name}:{node.lineno} uses the @ operator")
        if isinstance(node, ast.Call):
            fn = node.func
            attr = fn.attr if isinstance(fn, ast.Attribute) else (fn.id if isinstance(fn, ast.Name) else "")
            assert attr not in GEMM_CALLS, f"{name}:{node.lineno} calls {attr}(): a torch GEMM on the product path"
            assert attr != "compile" or not (isinstance(fn, ast.Attribute) and isinstance(fn.value, ast.Name)
                                              and fn.value.id == "torch"), f"{name}:{node.lineno} calls torch.compile"


@pytest.mark.parametrize("name", MODULES)
def test_module_reads_no_working_file_and_no_reference_checkout(name):
    with open(os.path.join(PKG, name)) as f:
        text = f.read()
    for needle in ("_work/", "_work\\\\", "oracle/_ref", "baseline/_ref"):
        assert needle not in text, f"{name} names {needle}"
    assert not re.search(r"[\"']/root/", text), f"{name} holds a path of one machine"


def test_cuda_sources_name_no_bulk_load_shared_over_a_cluster():
    """Every bulk or tensor copy instruction in the CUDA sources is written without the qualifier that
    delivers one load to several CTAs of a cluster (spelled in two halves here, so that this file
    does not name it either)."""
    qualifier = "multi" + "cast"
    bulk = "cp" + r"\.async\." + "bulk" + r"[.\w:]*"
    csrc = os.path.join(PKG, "csrc")
    for f in sorted(os.listdir(csrc)):
        with open(os.path.join(csrc, f)) as fh:
            text = fh.read()
        assert qualifier + "::cluster" not in text, f
        for m in re.finditer(bulk, text):
            assert qualifier not in m.group(0), f"{f}: {m.group(0)}"


def test_no_except_clause_swallows_a_missing_kernel():
    """Nothing in the package catches NativeKernelUnavailableError (or everything) around a kernel
    call and carries on: the only broad handlers allowed are the ones that re-raise or that guard an
    optional import."""
    for name in MODULES:
        for node in ast.walk(_tree(name)):
            if not isinstance(node, ast.ExceptHandler):
                continue
            caught = ast.unparse(node.type) if node.type is not None else "BaseException"
            assert "NativeKernelUnavailableError" not in caught, f"{name}:{node.lineno} catches the fail-closed error"
            assert "StaleExtensionError" not in caught, f"{name}:{node.lineno} catches the stale-library error"
