"""`Binarization`: drop-in for the reference class of the same name (binary.py:2850-2980).

It carries the technique and its hyper-parameters to `BRAGPTQ.fasterquant`, where
the block kernel applies the binarizer to the three groups of every block.  The
techniques implemented are the three of the calibration path:

    braq   residual binary expansion            (binary.py:18-39)
    crbog  coupled expansion, float64 2x2 solve  (binary.py:577-687)
    crb    CRB v7: Tikhonov-regularised joint scale solve, correlation damping,
           two-way sign refinement                (binary.py:1544-1638)
    crb_norefine, crb_symdamp, crb_symdamp_norefine
           the same function with skip_refinement / symmetric_damp set (binary.py:2885-2890)
"""
from __future__ import annotations

import math

import torch.nn as nn

SUPPORTED_METHODS = ("braq", "crbog", "crb", "crb_norefine", "crb_symdamp", "crb_symdamp_norefine")


class Binarization(nn.Module):
    def __init__(self, weight, method="2bit", groupsize=-1, corr_damp=0.1, lam=1e-5, coupling=0.5):
        super().__init__()
        oc, ic = weight.shape[0], int(weight.shape[1:].numel())
        if groupsize == -1:
            groupsize = ic
        self.groupsize = groupsize
        self.n_groups = math.ceil(ic / groupsize)
        self.method = str(method).lower()       # the README spells the techniques in upper case
        if self.method not in SUPPORTED_METHODS:
            raise NotImplementedError(
                f"method {method!r}: this build implements {', '.join(SUPPORTED_METHODS)} only")
        self.corr_damp = corr_damp
        self.lam = lam
        self.coupling = coupling

    def quantize(self, w, mask, order=2, groupi=0, col_weights=None):
        """Binarizes `w` on `mask` with the configured technique (binary.py:2868-2884).

        Runs the same device code as the block step on a [R, 128] block.
        """
        from . import ops
        return ops.binarize_group(w, mask, order, self.method, self.lam, self.corr_damp)
