"""crb_b200: the CRB / BiLLM calibration-time binarization path on B200 (sm_100a).

Public surface (mirrors the reference's `bigptq.BRAGPTQ` and `binary.Binarization`):

    from crb_b200 import BRAGPTQ, Binarization

The CUDA kernels live in `crb_b200/csrc`, built in-tree into
`crb_b200/_lib/libcrb_b200.so` by `python -m crb_b200.build`; the C ABI is
declared in `include/crb_b200.h`.
"""
from .binary import Binarization
from .bigptq import BRAGPTQ

__all__ = ["BRAGPTQ", "Binarization"]
__version__ = "0.1.0"
