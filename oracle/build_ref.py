"""Build recipe of `oracle/_ref`: the reference's own modules of the hot path, compiled.

TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline; the shipped package never loads it).

    python oracle/build_ref.py --reference <checkout of the reference>

The reference's path is plain Python, so "building" it means byte-compiling its modules from
where they lie: `bigptq.py`, `binary.py`, `modelutils.py` and `utils/{__init__,autosearch,mask,
structure}.py` are compiled with `py_compile` into `oracle/_ref/*.pyc` (sourceless modules that
the same interpreter imports like any other).  No source file is copied; `oracle/_ref/` is build
output and is not tracked.  `load()` imports the compiled reference with the shims it needs on a
machine without the packages it imports but never uses (`exceptiongroup`, `pyparsing`) and, on a
CUDA-less host, with `torch.cuda.synchronize` made a no-op (bigptq.py:272 calls it).
"""
from __future__ import annotations

import argparse
import importlib
import os
import py_compile
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
MODULES = ("bigptq.py", "binary.py", "modelutils.py", "utils/__init__.py", "utils/autosearch.py",
           "utils/mask.py", "utils/structure.py")


def build(reference: str, quiet: bool = False) -> str:
    """Compiles the reference modules of the path into oracle/_ref (outputs only; nothing is copied)."""
    for rel in MODULES:
        src = os.path.join(reference, rel)
        dst = os.path.join(REF_DIR, rel[:-3] + ".pyc")
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        py_compile.compile(src, cfile=dst, dfile=rel, doraise=True)
    with open(os.path.join(REF_DIR, "BUILT_FROM"), "w") as f:
        f.write(f"byte-compiled by oracle/build_ref.py with Python {sys.version.split()[0]}\n")
    if not quiet:
        print("built", REF_DIR)
    return REF_DIR


def available() -> bool:
    return all(os.path.exists(os.path.join(REF_DIR, rel[:-3] + ".pyc")) for rel in MODULES)


def load():
    """Imports the compiled reference: returns its (bigptq, binary, utils.autosearch) modules."""
    import torch
    if not available():
        raise RuntimeError("oracle/_ref is not built (python oracle/build_ref.py --reference <checkout>)")
    for name, attr in (("exceptiongroup", "catch"), ("pyparsing", "line")):
        try:
            importlib.import_module(name)
        except ImportError:
            mod = types.ModuleType(name)
            setattr(mod, attr, None)
            sys.modules[name] = mod
    if not torch.cuda.is_available():
        torch.cuda.synchronize = lambda *a, **k: None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    bigptq = importlib.import_module("bigptq")
    binary = importlib.import_module("binary")
    autosearch = importlib.import_module("utils.autosearch")
    if not getattr(bigptq, "__file__", "").startswith(REF_DIR):
        raise RuntimeError("another module named bigptq shadows oracle/_ref")
    return bigptq, binary, autosearch


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of an unmodified checkout of the reference project")
    a = ap.parse_args()
    build(a.reference)
    mods = load()
    print("import ok:", [m.__name__ for m in mods])
