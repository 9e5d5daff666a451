"""Build recipe of `oracle/_ref`: the reference's own modules of the hot path, compiled.

TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline; the shipped package never loads it).

    python oracle/build_ref.py --reference <checkout of the reference>

The reference's path is plain Python, so "building" it means byte-compiling its modules from
where they lie: `bigptq.py`, `binary.py`, `modelutils.py` and `utils/{__init__,autosearch,mask,
structure}.py` are compiled and the code objects written (marshal) to `oracle/_ref/*.pycode`.
No source file is copied; `oracle/_ref/` is build output and is not tracked.  `load()` turns the
code objects back into modules (same interpreter version as the one that built them) with the
shims the reference needs on a machine without the packages it imports but never uses
(`exceptiongroup`, `pyparsing`) and, on a CUDA-less host, with `torch.cuda.synchronize` made a
no-op (bigptq.py:272 calls it).
"""
from __future__ import annotations

import argparse
import importlib
import os
import marshal
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
MODULES = ("bigptq.py", "binary.py", "modelutils.py", "utils/__init__.py", "utils/autosearch.py",
           "utils/mask.py", "utils/structure.py")


def _artifact(rel: str) -> str:
    return os.path.join(REF_DIR, rel[:-3] + ".pycode")


def build(reference: str, quiet: bool = False) -> str:
    """Compiles the reference modules of the path into oracle/_ref (outputs only; nothing is copied)."""
    for rel in MODULES:
        with open(os.path.join(reference, rel), "rb") as f:
            code = compile(f.read(), rel, "exec", dont_inherit=True)
        dst = _artifact(rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        with open(dst, "wb") as f:
            marshal.dump(code, f)
    with open(os.path.join(REF_DIR, "BUILT_FROM"), "w") as f:
        f.write(f"{sys.version_info[0]}.{sys.version_info[1]}\n")
    if not quiet:
        print("built", REF_DIR)
    return REF_DIR


def available() -> bool:
    tag = os.path.join(REF_DIR, "BUILT_FROM")
    if not (os.path.exists(tag) and all(os.path.exists(_artifact(rel)) for rel in MODULES)):
        return False
    with open(tag) as f:                                  # code objects are tied to the interpreter version
        return f.read().strip() == f"{sys.version_info[0]}.{sys.version_info[1]}"


_loaded = None


def load():
    """Imports the compiled reference: returns its (bigptq, binary, utils.autosearch) modules."""
    global _loaded
    if _loaded is not None:
        return _loaded
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
    # dependency order: binary <- utils.mask <- utils.autosearch <- utils.structure <- bigptq
    order = ("binary.py", "utils/__init__.py", "utils/mask.py", "utils/autosearch.py", "utils/structure.py",
             "bigptq.py", "modelutils.py")
    mods = {}
    for rel in order:
        name = rel[:-3].replace("/", ".")
        is_pkg = name.endswith(".__init__")
        if is_pkg:
            name = name[: -len(".__init__")]
        mod = types.ModuleType(name)
        mod.__file__ = _artifact(rel)
        if is_pkg:
            mod.__path__ = []
        with open(_artifact(rel), "rb") as f:
            code = marshal.load(f)
        sys.modules[name] = mod
        exec(code, mod.__dict__)
        if "." in name:
            setattr(sys.modules[name.rsplit(".", 1)[0]], name.rsplit(".", 1)[1], mod)
        mods[name] = mod
    _loaded = (mods["bigptq"], mods["binary"], mods["utils.autosearch"])
    return _loaded


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of an unmodified checkout of the reference project")
    a = ap.parse_args()
    build(a.reference)
    mods = load()
    print("import ok:", [m.__name__ for m in mods])
