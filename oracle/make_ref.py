"""Recipe for oracle/_ref: the reference's OWN CPU implementation of the path, for validating the
restatement and for the reference arm of the benchmark.

The reference's path is two self-contained torch files (its independent decoder
tests/cb_torch_reference.py and its codec gridbook/codec.py).  Where the reference checkout is
present they are copied, unmodified, into oracle/_ref/ - a folder that is never committed (it is
listed in .gitignore) but travels with the working tree to the machine that runs the benchmark.
Nothing in the product package reads it; bench.py --impl reference times it when it is there."""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = (("tests/cb_torch_reference.py", "cb_torch_reference.py"), ("gridbook/codec.py", "codec.py"))


def default_reference_root() -> str:
    """Where the reference checkout is looked for: $GRIDBOOK_REFERENCE, else a folder named
    `reference` beside this repository."""
    return os.environ.get("GRIDBOOK_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def make(reference_root: str | None = None) -> bool:
    """Copies the files when `reference_root` holds them; returns whether oracle/_ref is complete."""
    reference_root = reference_root or default_reference_root()
    if all(os.path.exists(os.path.join(reference_root, src)) for src, _ in FILES):
        os.makedirs(REF_DIR, exist_ok=True)
        for src, dst in FILES:
            shutil.copyfile(os.path.join(reference_root, src), os.path.join(REF_DIR, dst))
    return available()


def available() -> bool:
    return all(os.path.exists(os.path.join(REF_DIR, dst)) for _, dst in FILES)


def load():
    """(cb_torch_reference module, codec module) from oracle/_ref."""
    import importlib.util
    mods = []
    for _, dst in FILES:
        spec = importlib.util.spec_from_file_location("gridbook_ref_" + dst[:-3], os.path.join(REF_DIR, dst))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods.append(mod)
    return tuple(mods)


if __name__ == "__main__":
    ok = make(sys.argv[1] if len(sys.argv) > 1 else None)
    print("oracle/_ref", "ready" if ok else "not available (no reference checkout here)")
