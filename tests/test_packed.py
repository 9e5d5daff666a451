"""The packed form of a binarized linear: bit planes + scales -> exactly the weights the block
loop wrote (GPU), and the file round trip of the container (CPU)."""
import os

import numpy as np
import pytest
import torch

import helpers as Hh  # noqa: F401  (keeps the tests directory on the path the same way the other files do)


def _synthetic_codes(R=24, C=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    s1 = torch.randint(0, 3, (R, C), generator=g)
    s2 = torch.randint(0, 3, (R, C), generator=g)
    grp = torch.randint(0, 2, (R, C), generator=g)
    for b in range(C // 128):
        cols = torch.randperm(128, generator=g)[: 3 + 5 * b] + 128 * b
        grp[:, cols] = 2
    grp[1, 5] = 3 if grp[1, 5] != 2 else 2
    codes = (s1 | (s2 << 2) | (grp << 4)).to(torch.uint8)
    scales = torch.randn(C // 128, R, 8, generator=g)
    Wq = torch.randn(R, C, generator=g)
    return codes, scales, Wq


def test_pack_layout_and_file_round_trip(tmp_path):
    from crb_b200 import packed
    from crb_b200._lib import CrbError
    codes, scales, Wq = _synthetic_codes()
    p = packed.pack_linear(codes, scales, Wq, "crb")
    R, C = codes.shape
    s1 = (codes & 3).int() - 1
    s2 = ((codes >> 2) & 3).int() - 1
    grp = (codes >> 4) & 3
    bits = np.unpackbits(p.b1.numpy(), axis=1, bitorder="little")[:, :C]
    assert np.array_equal(bits.astype(bool), (s1 > 0).numpy())
    bits = np.unpackbits(p.lm.numpy(), axis=1, bitorder="little")[:, :C]
    assert np.array_equal(bits.astype(bool), (grp == 1).numpy())
    for b in range(C // 128):
        cols = torch.nonzero(grp[0, 128 * b:128 * (b + 1)] == 2).flatten()
        assert p.salcol[128 * b:128 * (b + 1)][cols].tolist() == list(range(len(cols)))
        assert int((p.salcol[128 * b:128 * (b + 1)] != 255).sum()) == len(cols)
        pitch = int(p.b2_pitch[b])
        assert pitch == (len(cols) + 7) // 8
        plane = p.b2[int(p.b2_off[b]): int(p.b2_off[b]) + R * pitch].reshape(R, pitch).numpy()
        got = np.unpackbits(plane, axis=1, bitorder="little")[:, :len(cols)].astype(bool)
        assert np.array_equal(got, (s2[:, cols + 128 * b] > 0).numpy())
    odd = (s1 == 0) | ((grp == 2) & (s2 == 0)) | (grp == 3)
    assert torch.equal(p.patch_index, torch.nonzero(odd.reshape(-1)).flatten())
    assert torch.equal(p.patch_value, Wq.reshape(-1)[p.patch_index])
    path = os.path.join(tmp_path, "lin.npz")
    packed.save(path, p)
    q = packed.load(path)
    assert (q.rows, q.cols, q.technique) == (p.rows, p.cols, p.technique)
    for k, v in p.tensors().items():
        assert torch.equal(v, q.tensors()[k]), k
    with pytest.raises(CrbError):
        packed.dequantize(p)                       # no CPU path
    bad = codes.clone()
    bad[0, 0] = (bad[0, 0] & 15) | (2 << 4)
    bad[1, 0] = (bad[1, 0] & 15)
    with pytest.raises(CrbError):
        packed.pack_linear(bad, scales, Wq, "crb")   # salient group must be whole columns


@pytest.mark.gpu
@pytest.mark.parametrize("tech", ("braq", "crbog", "crb"))
def test_dequantize_reproduces_the_block_loop(tech, tmp_path):
    from crb_b200 import ops, packed
    dev = "cuda:0"
    g = torch.Generator().manual_seed(5)
    R, C = 200, 128 * 5
    W = torch.randn(R, C, generator=g) * 0.02
    W[::9, 40] = 0.0
    W[:, 300] = 0.0                                   # a dead input channel
    U = torch.triu(torch.randn(C, C, generator=g) * (0.05 / C ** 0.5), 1) + torch.diag(0.5 + torch.rand(C, generator=g))
    Wd = W.to(dev).clone()
    out = ops.quantize_linear(Wd, U.to(dev).contiguous(), tech, want_codes=True)
    p = packed.pack_linear(out["codes"], out["scales"], Wd, tech)
    assert torch.equal(packed.dequantize(p), Wd)      # bit for bit
    path = os.path.join(tmp_path, "lin.npz")
    packed.save(path, p)
    back = packed.dequantize(packed.load(path, dev))
    assert torch.equal(back, Wd)
    assert p.bits_per_weight() < 5.0
    # listed elements are rare on ordinary data
    assert p.patch_index.numel() < 0.02 * R * C


@pytest.mark.gpu
def test_bragptq_keeps_the_packed_result():
    import torch.nn as nn
    from crb_b200 import BRAGPTQ, Binarization, packed
    dev = "cuda:0"
    g = torch.Generator().manual_seed(6)
    lin = nn.Linear(256, 96, bias=False)
    lin.weight.data = torch.randn(96, 256, generator=g) * 0.02
    lin = lin.half().to(dev)
    q = BRAGPTQ(lin, Binarization(lin.weight, method="crb", groupsize=128), salient_metric="hessian")
    q.verbose = False
    q.pack = True
    for _ in range(4):
        q.add_batch(torch.randn(1, 512, 256, generator=g).half().to(dev), None)
    q.fasterquant(blocksize=128, percdamp=0.01)
    assert q.packed is not None
    W32 = packed.dequantize(q.packed)
    assert torch.equal(W32.to(torch.float16), lin.weight.data)
