"""The package installs, and vLLM's plugin loader would find it: after a plain `pip install`
into a scratch directory the `vllm.general_plugins` group holds `gridbook = gridbook_b200:register`
(the reference's pyproject.toml:74-75), the entry point loads, and calling it registers the
quantization config under both names."""
import importlib.metadata as md
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def installed(tmp_path_factory):
    target = tmp_path_factory.mktemp("site")
    # install from a copy, so that pip's build folders do not land in the checkout
    src = tmp_path_factory.mktemp("src")
    for name in ("pyproject.toml", "README.md"):
        shutil.copy(os.path.join(ROOT, name), src / name)
    shutil.copytree(os.path.join(ROOT, "gridbook_b200"), src / "gridbook_b200",
                    ignore=shutil.ignore_patterns("build", "__pycache__", "*.digest"))
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-deps", "--no-build-isolation", "--quiet",
           "--target", str(target), str(src)]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if done.returncode != 0:
        pytest.fail("pip install failed:\n" + done.stdout[-2000:] + done.stderr[-2000:])
    return str(target)


def test_entry_point_is_discoverable_and_registers(installed):
    dists = [d for d in md.distributions(path=[installed]) if d.metadata["Name"] == "gridbook-b200"]
    assert len(dists) == 1
    eps = [e for e in dists[0].entry_points if e.group == "vllm.general_plugins"]
    assert [(e.name, e.value) for e in eps] == [("gridbook", "gridbook_b200:register")]
    register = eps[0].load()                       # resolves against the checkout on sys.path
    import gridbook_b200
    assert register is gridbook_b200.register
    # the installed copy carries the package and, when it was built before installing, the library
    assert os.path.exists(os.path.join(installed, "gridbook_b200", "plugin.py"))
    assert os.path.exists(os.path.join(installed, "gridbook_b200", "csrc", "gb_gemv.cu"))
    if os.path.exists(os.path.join(ROOT, "gridbook_b200", "libgridbook_b200.so")):
        assert os.path.exists(os.path.join(installed, "gridbook_b200", "libgridbook_b200.so"))


def test_register_against_the_installed_engine():
    """With vLLM importable, register() lands in its quantization registry under both names.  Runs
    in a fresh interpreter, as the engine's plugin loader runs it: vLLM is imported first, so the
    config class derives from the engine's own QuantizationConfig."""
    pytest.importorskip("vllm")
    code = (
        "import vllm\n"
        "from vllm.model_executor.layers.quantization import get_quantization_config\n"
        "import gridbook_b200\n"
        "gridbook_b200.register()\n"
        "from gridbook_b200.config import PrismaQuantConfig\n"
        "assert get_quantization_config('gridbook') is PrismaQuantConfig\n"
        "assert get_quantization_config('prismaquant') is PrismaQuantConfig\n"
        "print('registered')\n")
    done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT)
    if done.returncode != 0 and "get_quantization_config" in done.stderr and "ImportError" in done.stderr:
        pytest.skip("this vLLM build has no quantization registry helpers")
    assert done.returncode == 0 and "registered" in done.stdout, done.stderr[-2000:]
