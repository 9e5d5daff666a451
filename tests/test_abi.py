"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from crb_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "crb_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(crb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("crb_hessian_accumulate", "crb_hinv_upper_factor", "crb_block_step",
                 "crb_trailing_update", "crb_quantize_linear", "crb_binarize_group"):
        assert must in names


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        pytest.fail(f"{_lib.LIB_PATH} not built: run `python -m crb_b200.build`")
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(handle, name), f"missing export {name}"


def test_python_binding_covers_the_header():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_host_only_calls():
    L = _lib.lib()
    assert L.crb_version() >= 1
    assert L.crb_arch() == b"sm_100a"
    assert L.crb_status_string(0) == b"ok"
    assert L.crb_status_string(-2) == b"workspace too small"
    # workspace sizing is pure host arithmetic
    assert L.crb_block_workspace_bytes(4096) > 4096 * 128 * 4
    assert L.crb_linear_workspace_bytes(4096) >= L.crb_block_workspace_bytes(4096) + 4096 * 128 * 4
    assert L.crb_factor_workspace_bytes(256) >= 256 * 256 * 4
    assert L.crb_hessian_workspace_bytes(256, 1024, 0) > L.crb_hessian_workspace_bytes(256, 1024, 1)
    assert L.crb_block_workspace_bytes(0) == 0


def test_product_path_refuses_cpu_tensors():
    import torch
    import torch.nn as nn
    from crb_b200 import BRAGPTQ, Binarization, ops
    lin = nn.Linear(128, 8, bias=False)
    with pytest.raises(_lib.CrbError):
        BRAGPTQ(lin, Binarization(lin.weight, method="crb", groupsize=128), "hessian")
    with pytest.raises(_lib.CrbError):
        ops.hessian_accumulate(torch.zeros(128, 128), torch.zeros(16, 128))
    with pytest.raises(NotImplementedError):
        Binarization(lin.weight, method="2bit")


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "crb_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, f"{f} mentions the oracle"
