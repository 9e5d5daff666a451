"""crb_b200: the CRB / BiLLM calibration-time binarization path on B200 (sm_100a).

Public surface (mirrors the reference's `bigptq.BRAGPTQ` and `binary.Binarization`):

    from crb_b200 import BRAGPTQ, Binarization

The CUDA kernels live in `crb_b200/csrc`, built in-tree into
`crb_b200/_lib/libcrb_b200.so` by `python -m crb_b200.build`; the C ABI is
declared in `include/crb_b200.h`.
"""
import os as _os

# The layer loop keeps more than eight streams busy at once (one per linear, the factorisation's
# side streams, copies, the lanes of the re-propagation pass).  With the CUDA default of eight
# hardware work queues, streams share queues and pick up ordering from each other: a short block
# loop then waits behind another linear's long factorisation.  The setting is read when the
# process creates its CUDA context, so it only takes effect when this package is imported before
# the first CUDA call; a value the user has set is left alone.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

from .binary import Binarization
from .bigptq import BRAGPTQ

__all__ = ["BRAGPTQ", "Binarization"]
__version__ = "0.1.0"
