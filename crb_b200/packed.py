"""Packed form of a binarized linear and its way back to float32 weights.

The reference never stores the binarized result: `fasterquant` writes the de-quantized weights
into the layer (bigptq.py:276-280) and `--save` is commented out (run.py:1033-1039).  The block
step here can also emit, per weight, its group and its two signs (`codes`) and, per row and
128-column block, the eight scales (`scales`); this module squeezes those into bit planes

    b1      [R, C/8]   first sign                       1 bit / weight
    lm      [R, C/8]   low / mid group                  1 bit / weight
    salcol  [C]        salient columns per block        1 byte / column
    b2      per block  second sign of the salient columns only
    scales  [C/128, R, 8] float32

(about 2 bits per weight plus 2 bits per weight of float32 scales), lists the handful of
elements a bit cannot describe (a sign of exactly 0, an element outside every group) with
their values, and rebuilds the float32 weights with the `crb_dequantize` kernel — bit for bit
the numbers the block step wrote.  `save` / `load` move a packed linear to and from an .npz file.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import numpy as np
import torch

from . import _lib
from ._lib import BLOCK, CrbError, check, lib, ptr, stream_ptr


@dataclass
class PackedLinear:
    rows: int
    cols: int
    technique: str
    b1: torch.Tensor          # uint8 [R, C/8]
    lm: torch.Tensor          # uint8 [R, C/8]
    salcol: torch.Tensor      # uint8 [C]
    b2: torch.Tensor          # uint8 [sum_b R * pitch_b]
    b2_off: torch.Tensor      # int64 [C/128]
    b2_pitch: torch.Tensor    # int32 [C/128]
    scales: torch.Tensor      # float32 [C/128, R, 8]
    patch_index: torch.Tensor  # int64 [n]  flat indices r * C + c of the listed elements
    patch_value: torch.Tensor  # float32 [n]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors().values())

    def bits_per_weight(self) -> float:
        return 8.0 * self.nbytes() / (self.rows * self.cols)

    def tensors(self) -> Dict[str, torch.Tensor]:
        return dict(b1=self.b1, lm=self.lm, salcol=self.salcol, b2=self.b2, b2_off=self.b2_off,
                    b2_pitch=self.b2_pitch, scales=self.scales, patch_index=self.patch_index,
                    patch_value=self.patch_value)

    def to(self, device) -> "PackedLinear":
        return PackedLinear(self.rows, self.cols, self.technique,
                            **{k: v.to(device) for k, v in self.tensors().items()})


def _pack_bits(mask: torch.Tensor) -> torch.Tensor:
    """[R, n] bool -> [R, ceil(n / 8)] uint8, LSB first."""
    R, n = mask.shape
    pad = (-n) % 8
    if pad:
        mask = torch.cat([mask, torch.zeros(R, pad, dtype=torch.bool, device=mask.device)], 1)
    w = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.int32, device=mask.device)
    return (mask.reshape(R, -1, 8).to(torch.int32) * w).sum(-1).to(torch.uint8)


def pack_linear(codes: torch.Tensor, scales: torch.Tensor, W_q: torch.Tensor, technique: str) -> PackedLinear:
    """Packs the outputs of `ops.quantize_linear(..., want_codes=True)`.

    codes [R, C] uint8 (bits 0-1 first sign + 1, bits 2-3 second sign + 1, bits 4-5 group: 0 low,
    1 mid, 2 salient, 3 none), scales [C/128, R, 8] float32, W_q [R, C] the weights the block loop
    left behind (only read for the listed elements).  Works on the tensors' own device.
    """
    if technique not in _lib.TECHNIQUES:
        raise CrbError(f"unknown technique {technique!r}")
    R, C = codes.shape
    if C % BLOCK or scales.shape != (C // BLOCK, R, 8):
        raise CrbError("codes [R, C] and scales [C/128, R, 8] do not belong together")
    dev = codes.device
    s1 = (codes & 3).to(torch.int16) - 1
    s2 = ((codes >> 2) & 3).to(torch.int16) - 1
    grp = (codes >> 4) & 3
    sal = grp == 2
    b1 = _pack_bits(s1 > 0)
    lm = _pack_bits(grp == 1)
    # salient columns are whole columns of a block (bigptq.py:143-145): read them off any row
    nblk = C // BLOCK
    sal_cols = sal.any(0)
    if bool((sal != sal_cols.unsqueeze(0)).any()):
        raise CrbError("the salient group is not column structured")
    within = sal_cols.reshape(nblk, BLOCK)
    pos = torch.cumsum(within.to(torch.int32), 1) - 1
    salcol = torch.where(within, pos, torch.full_like(pos, 255)).to(torch.uint8).reshape(C)
    counts = within.sum(1).to(torch.int32)
    pitch = (counts + 7) // 8
    off = torch.zeros(nblk, dtype=torch.int64, device=dev)
    if nblk > 1:
        off[1:] = torch.cumsum(pitch[:-1].to(torch.int64) * R, 0)
    planes = []
    for b in range(nblk):
        cols = torch.nonzero(within[b], as_tuple=False).flatten() + b * BLOCK
        planes.append(_pack_bits(s2[:, cols] > 0).reshape(-1) if cols.numel() else
                      torch.zeros(0, dtype=torch.uint8, device=dev))
    b2 = torch.cat(planes) if planes else torch.zeros(0, dtype=torch.uint8, device=dev)
    if b2.numel() == 0:
        b2 = torch.zeros(16, dtype=torch.uint8, device=dev)       # a valid pointer for the kernel
    odd = (s1 == 0) | (sal & (s2 == 0)) | (grp == 3)
    idx = torch.nonzero(odd.reshape(-1), as_tuple=False).flatten()
    val = W_q.reshape(-1)[idx].float() if W_q.is_contiguous() else W_q.contiguous().reshape(-1)[idx].float()
    return PackedLinear(R, C, technique, b1.contiguous(), lm.contiguous(), salcol.contiguous(), b2.contiguous(),
                        off, pitch.to(torch.int32).contiguous(), scales.contiguous().float(), idx, val)


def dequantize(p: PackedLinear, out: torch.Tensor = None) -> torch.Tensor:
    """float32 weights [R, C] of a packed linear (CUDA only; there is no CPU path)."""
    dev = p.b1.device
    if dev.type != "cuda":
        raise CrbError("dequantize needs the packed linear on a CUDA device (no CPU fallback)")
    if out is None:
        out = torch.empty(p.rows, p.cols, dtype=torch.float32, device=dev)
    if out.shape != (p.rows, p.cols) or out.dtype != torch.float32 or out.stride(1) != 1 or out.device != dev:
        raise CrbError("out must be a float32 [R, C] CUDA tensor with unit column stride")
    check(lib().crb_dequantize(ptr(out), p.rows, p.cols, out.stride(0), _lib.TECHNIQUES[p.technique], ptr(p.b1),
                               ptr(p.lm), ptr(p.salcol), ptr(p.b2), ptr(p.b2_off), ptr(p.b2_pitch), ptr(p.scales),
                               stream_ptr()), "crb_dequantize")
    if p.patch_index.numel():
        if out.is_contiguous():
            out.view(-1)[p.patch_index] = p.patch_value
        else:
            out[p.patch_index // p.cols, p.patch_index % p.cols] = p.patch_value
    return out


def save(path: str, p: PackedLinear) -> None:
    np.savez_compressed(path, rows=p.rows, cols=p.cols, technique=p.technique,
                        **{k: v.detach().cpu().numpy() for k, v in p.tensors().items()})


def load(path: str, device="cpu") -> PackedLinear:
    with np.load(path, allow_pickle=False) as z:
        t = {k: torch.from_numpy(z[k]).to(device) for k in
             ("b1", "lm", "salcol", "b2", "b2_off", "b2_pitch", "scales", "patch_index", "patch_value")}
        return PackedLinear(int(z["rows"]), int(z["cols"]), str(z["technique"]), **t)
