"""Pins the CPU oracle to outputs of the unmodified reference (tests/golden/*.npz).

The fixtures were produced by tests/golden/make_golden.py, which imports the
reference and records its masks, candidate errors, group outputs and final
weights on seeded inputs.  The oracle must reproduce them: exactly for masks
and for the braq / crb arithmetic, to 1e-6 for crbog (whose reference sums run
over compacted rows).
"""
import os

import numpy as np
import pytest
import torch

from oracle import crb_oracle as O


def unpack(bits, shape):
    n = int(np.prod(shape))
    return torch.from_numpy(np.unpackbits(bits)[:n].reshape(shape).astype(bool))


@pytest.fixture(scope="module")
def blocks(golden_dir):
    return np.load(os.path.join(golden_dir, "blocks.npz"))


@pytest.fixture(scope="module")
def linear(golden_dir):
    return np.load(os.path.join(golden_dir, "linear.npz"))


def test_quantile_restated_matches_numpy():
    probs = torch.linspace(0.10, 0.90, 81).numpy()
    for n, seed in ((7, 0), (1000, 1), (64 * 128, 2), (2048 * 128, 3)):
        rng = np.random.default_rng(seed)
        a = rng.standard_normal(n).astype(np.float32) ** 2
        a[rng.integers(0, n, n // 5)] = 0.0
        assert np.array_equal(O.quantile_linear_f32(a, probs), np.quantile(a, q=probs))


@pytest.mark.parametrize("ci", range(4))
def test_block_search_matches_reference(blocks, ci):
    W = torch.from_numpy(blocks[f"c{ci}_W"])
    d = torch.from_numpy(blocks[f"c{ci}_d"])
    m1, m2, m3, tr = O.partition_block(W, d)
    for name, m in (("m1", m1), ("m2", m2), ("m3", m3)):
        assert torch.equal(m, unpack(blocks[f"c{ci}_{name}"], W.shape)), name
    ref = blocks[f"c{ci}_errs"]
    got = np.asarray(tr.salient_err + tr.split_err)
    assert ref.shape == (130,)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("tech", O.TECHNIQUES)
@pytest.mark.parametrize("ci", range(4))
def test_block_binarizers_match_reference(blocks, ci, tech):
    W = torch.from_numpy(blocks[f"c{ci}_W"])
    masks = [unpack(blocks[f"c{ci}_{n}"], W.shape) for n in ("m1", "m2", "m3")]
    for g, (m, order) in enumerate(zip(masks, (1, 1, 2))):
        q = O.binarize(tech, W, m, order)
        ref = torch.from_numpy(blocks[f"c{ci}_{tech}_q{g}"])
        if tech == "crbog" and order == 2:
            assert torch.allclose(q, ref, rtol=1e-6, atol=1e-9)
        else:
            assert torch.equal(q, ref), (tech, g)


def test_hessian_matches_reference(linear):
    X = torch.from_numpy(linear["X"])
    H = O.hessian_from_tokens(X, int(linear["nseq"]))
    assert torch.equal(H, torch.from_numpy(linear["H"]))


@pytest.mark.parametrize("tech", O.TECHNIQUES)
def test_linear_matches_reference(linear, tech):
    W = torch.from_numpy(linear["W"])
    H = torch.from_numpy(linear["H"]).clone()
    res = O.quantize_linear(W, H, tech)
    ref = torch.from_numpy(linear[f"{tech}_Wq"])
    for bi, blk in enumerate(res.blocks):
        shape = blk.Q.shape
        assert torch.equal(torch.diag(res.U[bi * 128:(bi + 1) * 128, bi * 128:(bi + 1) * 128]),
                           torch.from_numpy(linear[f"{tech}_b{bi}_d"]))
        for name, m in zip(("m1", "m2", "m3"), blk.masks):
            assert torch.equal(m, unpack(linear[f"{tech}_b{bi}_{name}"], shape)), (bi, name)
    if tech == "crbog":
        assert torch.allclose(res.W, ref, rtol=1e-5, atol=1e-8)
        assert abs(res.error - float(linear[f"{tech}_error"])) <= 1e-5 * abs(res.error)
    else:
        assert torch.equal(res.W, ref)
        assert res.error == float(linear[f"{tech}_error"])


def test_codes_and_scales_rebuild_q(blocks):
    """The oracle's sign codes and scales are a complete description of Q."""
    W = torch.from_numpy(blocks["c1_W"])
    d = torch.from_numpy(blocks["c1_d"])
    for tech in O.TECHNIQUES:
        blk = O.block_step(W, d, tech)
        grp = (blk.codes >> 4).long()
        b1 = (blk.codes & 3).float() - 1
        b2 = ((blk.codes >> 2) & 3).float() - 1
        s = blk.scales
        low = s[:, 0:1] + s[:, 1:2] * b1
        mid = s[:, 2:3] + s[:, 3:4] * b1
        if tech == "braq":
            sal = (s[:, 4:5] + s[:, 5:6] * b1) + (s[:, 6:7] + s[:, 7:8] * b2)
        else:
            sal = s[:, 4:5] + s[:, 5:6] * b1 + s[:, 6:7] * b2
        rebuilt = torch.where(grp == 0, low, torch.where(grp == 1, mid, sal))
        assert torch.allclose(rebuilt, blk.Q, rtol=1e-5, atol=1e-8), tech


@pytest.fixture(scope="module")
def variants(golden_dir):
    return np.load(os.path.join(golden_dir, "variants.npz"))


@pytest.mark.parametrize("tech", ("crb_norefine", "crb_symdamp", "crb_symdamp_norefine"))
@pytest.mark.parametrize("ci", (0, 3))
def test_crb_flag_variants_match_reference(blocks, variants, ci, tech):
    """skip_refinement / symmetric_damp of the v7 binarizer (binary.py:2885-2890)."""
    W = torch.from_numpy(blocks[f"c{ci}_W"])
    masks = [unpack(blocks[f"c{ci}_{n}"], W.shape) for n in ("m1", "m2", "m3")]
    for g, m in enumerate(masks):
        for order in (1, 2):
            ref = torch.from_numpy(variants[f"c{ci}_{tech}_g{g}_o{order}"])
            assert torch.equal(O.binarize(tech, W, m, order), ref), (tech, g, order)
    ragged = masks[0].clone()
    ragged[::7] = False
    assert torch.equal(O.binarize(tech, W, ragged, 2), torch.from_numpy(variants[f"c{ci}_{tech}_ragged_o2"]))


@pytest.mark.parametrize("tech,orders", [("braq", (2, 2, 2)), ("crb", (2, 2, 2)), ("crb", (2, 1, 1)),
                                         ("crb_symdamp_norefine", (1, 1, 2))])
def test_linear_with_other_orders_matches_reference(linear, variants, tech, orders):
    """`orders` reaches the quantizer per group (bigptq.py:246-247); the searches do not depend on it."""
    tag = f"{tech}_{''.join(map(str, orders))}"
    W = torch.from_numpy(linear["W"])
    H = torch.from_numpy(linear["H"]).clone()
    res = O.quantize_linear(W, H, tech, orders=orders)
    for bi, blk in enumerate(res.blocks):
        got = np.asarray(blk.trace.salient_err + blk.trace.split_err)
        assert np.array_equal(got, variants[f"{tag}_b{bi}_errs"]), bi
    assert torch.equal(res.W, torch.from_numpy(variants[f"{tag}_Wq"]))
    assert res.error == float(variants[f"{tag}_error"])


@pytest.mark.parametrize("ci", (0, 1, 3))
def test_magnitude_metric_block_search_matches_reference(blocks, variants, ci):
    """salient_metric="magnitude": the searches run on the signed weights (utils/structure.py:11-12)."""
    W = torch.from_numpy(blocks[f"c{ci}_W"])
    d = torch.from_numpy(blocks[f"c{ci}_d"])
    m1, m2, m3, tr = O.partition_block(W, d, "magnitude")
    for name, m in (("m1", m1), ("m2", m2), ("m3", m3)):
        assert torch.equal(m, unpack(variants[f"mag_c{ci}_{name}"], W.shape)), name
    assert np.array_equal(np.asarray(tr.salient_err + tr.split_err), variants[f"mag_c{ci}_errs"])
    assert torch.equal(O.block_step(W, d, "crb", metric="magnitude").Q, torch.from_numpy(variants[f"mag_c{ci}_crb_Q"]))


@pytest.mark.parametrize("tech", ("braq", "crb"))
def test_magnitude_metric_linear_matches_reference(linear, variants, tech):
    W = torch.from_numpy(linear["W"])
    H = torch.from_numpy(linear["H"]).clone()
    res = O.quantize_linear(W, H, tech, metric="magnitude")
    for bi, blk in enumerate(res.blocks):
        got = np.asarray(blk.trace.salient_err + blk.trace.split_err)
        assert np.array_equal(got, variants[f"mag_{tech}_b{bi}_errs"]), bi
        assert torch.equal(blk.masks[0], unpack(variants[f"mag_{tech}_b{bi}_m1"], blk.Q.shape))
        assert torch.equal(blk.masks[2], unpack(variants[f"mag_{tech}_b{bi}_m3"], blk.Q.shape))
    assert torch.equal(res.W, torch.from_numpy(variants[f"mag_{tech}_Wq"]))
    assert res.error == float(variants[f"mag_{tech}_error"])
