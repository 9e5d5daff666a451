"""Parity at the shapes the benchmark runs: the single-linear workload end to end against the
reference's golden outputs, tall blocks (16384 and 36864 rows) against the oracle, and the
sensitivity of the block decisions to the summation order of partial Hessians."""
import os

import numpy as np
import pytest
import torch

from oracle import crb_oracle as O
from tests import helpers as Hh

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from crb_b200 import ops as _ops
    return _ops


def test_single_linear_workload_end_to_end(golden_dir):
    """W 2048x2048, 128 sequences of 2048 float32 tokens (1 % of the channels x20), crb: the
    whole path add_batch x 128 -> factor -> 16 block steps with grouped trailing updates, against
    what the unmodified reference produced on the same seeded inputs (bigptq.py:37-54, 56-291)."""
    import torch.nn as nn
    from crb_b200 import BRAGPTQ, Binarization
    from crb_b200.synth import single_linear_case
    ref = np.load(os.path.join(golden_dir, "config1.npz"))
    W, ch, sequences = single_linear_case(device=DEV)
    assert np.array_equal(ch.numpy(), ref["channels"])
    R, C = W.shape
    lin = nn.Linear(C, R, bias=False)
    lin.weight.data = W.clone()
    lin = lin.to(DEV)
    g = BRAGPTQ(lin, Binarization(lin.weight, method="crb", groupsize=128), salient_metric="hessian")
    g.verbose = False
    G = torch.zeros(C, C, dtype=torch.float64, device=DEV)
    for x in sequences():
        g.add_batch(x.unsqueeze(0), None)
        xd = x.double()
        G += xd.t() @ xd
    assert g.nsamples == 128
    H = g.H
    h_diag, h_row0 = torch.diag(H).cpu().numpy(), H[0].cpu().numpy()
    # float32 activations go through two fp16 planes (about 22 significand bits per product)
    np.testing.assert_allclose(h_diag, ref["H_diag"], rtol=2e-5)
    np.testing.assert_allclose(h_row0, ref["H_row0"], rtol=2e-5, atol=2e-5 * float(np.abs(ref["H_row0"]).max()))
    info = g.fasterquant(blocksize=128, percdamp=0.01)
    Wq = lin.weight.data.float().cpu()
    trace = g.last_trace.cpu()
    # block decisions: every block must follow the reference until (if ever) a decision differs inside
    # the tie band; after such a tie the two runs work on different inputs and only the aggregate
    # figures below can be compared
    outcomes = []
    for bi in range(C // 128):
        tf = Hh.trace_fields(trace[bi])
        outcome = Hh.check_search_against_reference(tf, ref[f"b{bi}_errs"], f"block {bi}", rtol=2e-4)
        outcomes.append(outcome)
        if outcome != "exact":
            break
        cols = np.sort(tf["top_cols"][:tf["n_salient"]])
        assert np.array_equal(cols, ref[f"b{bi}_m3cols"]), f"block {bi}: salient columns"
    n_exact = sum(o == "exact" for o in outcomes)
    print(f"single-linear workload: {n_exact} of {C // 128} blocks decided exactly like the reference, "
          f"outcomes {outcomes}")
    cols_ok = n_exact * 128
    if cols_ok:
        rows = torch.from_numpy(ref["Wq_rows"])[:, :cols_ok]
        got = Wq[:32, :cols_ok]
        close = torch.isclose(got, rows, rtol=1e-3, atol=1e-6).float().mean().item()
        assert close >= Hh.SIGN_AGREEMENT, f"only {close:.5f} of the first rows' weights agree"
        norm = torch.linalg.norm(Wq.double(), dim=0).numpy()[:cols_ok]
        np.testing.assert_allclose(norm, ref["Wq_colnorm"][:cols_ok], rtol=1e-3)
    D = (W.to(DEV).double() - Wq.to(DEV).double())
    out_err = float(torch.sqrt(torch.clamp(((D @ G) * D).sum(), min=0)))
    assert abs(out_err - float(ref["out_err"])) <= Hh.OUTPUT_ERR_RTOL * float(ref["out_err"]), (out_err, float(ref["out_err"]))
    assert abs(info["error"] - float(ref["error"])) <= Hh.OUTPUT_ERR_RTOL * float(ref["error"]), (info["error"], float(ref["error"]))


def _tall_block(R, seed):
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(R, 128, generator=g) * 0.02
    d = 0.5 + torch.rand(128, generator=g)
    hot = torch.randperm(128, generator=g)[:4]
    d[hot] *= 0.25
    W[::97, 5] = 0.0                      # exact zeros in the metric
    return W, d


@pytest.mark.parametrize("R", (16384, 36864))
def test_tall_block_matches_oracle(ops, R):
    """Row counts of the benchmark's tallest linears (fc1 of the 6.7b and of the 66b shape): above
    8192 rows the search kernels take several row tiles per CTA and the float32 quantile index of
    numpy starts to matter.  Search decisions, the 81 split values, masks and Q for braq and crb."""
    W, d = _tall_block(R, 1000 + R)
    m1, m2, m3, tr = O.partition_block(W, d)
    ref_errs = np.asarray(tr.salient_err + tr.split_err)
    for tech in ("crb", "braq"):
        Wd = W.to(DEV).clone()
        out = ops.block_step(Wd, torch.diag(d).to(DEV), 0, tech)
        torch.cuda.synchronize()
        tf = Hh.trace_fields(out["trace"])
        outcome = Hh.check_search_against_reference(tf, ref_errs, f"R={R} {tech}")
        assert np.array_equal(tf["top_cols"], tr.top_cols.numpy())
        g1, g2, g3 = Hh.masks_from_codes(out["codes"].cpu())
        assert bool(((g1.int() + g2.int() + g3.int()) == 1).all())
        if tf["n_salient"] == tr.n_salient:
            # the split candidates are the quantiles numpy computes, bit for bit
            assert np.array_equal(tf["split_values"], tr.split_values.astype(np.float32)), f"R={R}: split values"
        if outcome != "exact":
            continue
        assert np.float32(tf["split_value"]) == np.float32(tr.split_value)
        assert torch.equal(g3, m3) and torch.equal(g1, m1) and torch.equal(g2, m2), f"R={R} {tech}: masks"
        Q = torch.zeros_like(W)
        for mask, order in zip((m1, m2, m3), (1, 1, 2)):
            Q += O.binarize(tech, W, mask, order) * mask
        assert torch.allclose(Wd.cpu(), Q, rtol=2e-5, atol=1e-7), f"R={R} {tech}: Q max diff {(Wd.cpu() - Q).abs().max()}"
        Err = (W - Q) / d.reshape(1, -1)
        assert torch.allclose(out["Err"].cpu(), Err, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("inputs", ("gaussian", "relu_features"))
def test_summation_order_of_partial_hessians_only_moves_ties(ops, inputs):
    """Several GPUs sum their partial Hessians in an order that depends on the GPU count.  Quantize
    one 4096 x 4096 linear from the same four partial sums added in three different orders: the
    runs may only part ways at a block whose decision is a near tie, and the layer's output error
    must agree far inside the 0.5 % contract either way.  `relu_features` mimics the input of an
    MLP's second linear (rectified, strongly correlated features: a badly conditioned Hessian)."""
    C = R = 4096
    g = torch.Generator(device=DEV).manual_seed(31)
    if inputs == "gaussian":
        X = torch.randn(4 * 4096, C, generator=g, device=DEV)
        X[:, torch.randperm(C, generator=g, device=DEV)[:40]] *= 20
    else:
        Z = torch.randn(4 * 4096, 1024, generator=g, device=DEV)
        X = torch.relu(Z @ (torch.randn(1024, C, generator=g, device=DEV) / 32.0) - 0.5)
    X = X.half()
    W = (torch.randn(R, C, generator=g, device=DEV) * 0.02)
    parts = []
    for k in range(4):
        S = torch.zeros(C, C, device=DEV)
        ops.hessian_accumulate(S, X[k * 4096:(k + 1) * 4096])
        parts.append(S)
    sums = [((parts[0] + parts[1]) + parts[2]) + parts[3], ((parts[3] + parts[2]) + parts[1]) + parts[0],
            (parts[0] + parts[2]) + (parts[1] + parts[3])]
    assert not torch.equal(sums[0], sums[1])
    runs = []
    for S in sums:
        H = S.clone()
        ops.hessian_finalize(H, 2.0 / 8)
        Wq = W.clone()
        U = ops.hinv_upper_factor(H, Wq, 0.01)
        udiag = torch.diagonal(U).double().cpu()
        out = ops.quantize_linear(Wq, U, "crb")
        assert ops.read_status(out["workspace"]) == 0
        D = (W - Wq).double()
        out_err = float(torch.linalg.norm(D @ X.double().t()))
        runs.append(dict(trace=out["trace"].cpu(), error=float(out["losses"].sum()), out_err=out_err, udiag=udiag))
    base = runs[0]
    nblk = C // 128
    report, failures = [], []
    for other in runs[1:]:
        # how far the two factors are apart: the block step divides by diag(U)
        u_rel = float(((other["udiag"] - base["udiag"]).abs() / base["udiag"]).max())
        differing, first = 0, None
        for b in range(nblk):
            ta, tb = Hh.trace_fields(base["trace"][b]), Hh.trace_fields(other["trace"][b])
            if (ta["n_salient"], ta["split_index"]) == (tb["n_salient"], tb["split_index"]):
                continue
            differing += 1
            if first is not None:
                continue                 # after the first difference the two runs work on different weights
            # which decision moved, how close it was, and how far apart the two runs' candidate errors are
            if ta["n_salient"] != tb["n_salient"]:
                ea, eb, ia, ib = ta["salient_err"], tb["salient_err"], ta["n_salient"] - 1, tb["n_salient"] - 1
            else:
                ea, eb, ia, ib = ta["split_err"], tb["split_err"], ta["split_index"], tb["split_index"]
            gap = float(abs(ea[ib] - ea[ia]) / ea[ia])
            moved = float(max(abs(ea[ia] - eb[ia]) / ea[ia], abs(ea[ib] - eb[ib]) / ea[ib]))
            tied = (Hh.score_tied_candidates(ta, max(Hh.SCORE_TIE, u_rel)) |
                    Hh.score_tied_candidates(tb, max(Hh.SCORE_TIE, u_rel))) & {ia, ib}
            first = dict(block=b, gap=gap, moved=moved, kind="column-score tie" if tied else "candidate tie")
            # a decision can only change hands if the inputs moved the two candidates by about their
            # gap; the inputs differ by float32 rounding amplified by the factorisation (u_rel).  Two
            # columns with (nearly) equal scores ranked the other way round move one candidate by a
            # finite amount: the documented metric tie.
            if not tied and gap > max(Hh.TIE_GAP, 4.0 * moved):
                failures.append(("decision moved without a tie", first))
        d_out = abs(other["out_err"] - base["out_err"]) / base["out_err"]
        d_sum = abs(other["error"] - base["error"]) / base["error"]
        report.append(dict(u_diag_rel=u_rel, first=first, differing_blocks=differing, out_err_rel=d_out, error_sum_rel=d_sum))
        if differing == 0:
            # identical decisions: the results agree to rounding
            if d_out > 1e-5:
                failures.append(("same decisions, different output error", d_out))
        elif d_out > 2 * Hh.OUTPUT_ERR_RTOL:
            failures.append(("output error moved by more than twice the contract's tolerance", d_out))
    print(f"summation order ({inputs}), {nblk} blocks:", *report, sep="\n  ")
    assert not failures, failures


def test_bounded_wait_runs_out_cleanly(ops):
    """A wait that nothing satisfies ends after its time limit: the kernel raises CRB_FLAG_WAIT_LIMIT and
    returns, and the context keeps working."""
    from crb_b200 import _lib
    flags = ops.selftest_wait_limit(DEV, limit_us=500)
    assert flags & _lib.FLAG_WAIT_LIMIT
    a = torch.randn(256, 128, device=DEV)
    b = torch.randn(128, 256, device=DEV)
    c = torch.zeros(256, 256, device=DEV)
    ops.gemm_f32(a, b, c)                                  # the same kernel, healthy again
    assert torch.allclose(c, a @ b, rtol=1e-4, atol=1e-4)


def test_wait_limit_flag_stops_fasterquant(ops):
    """The host side refuses to go on when the Hessian kernel reported an expired wait (injected here by
    setting the flag in its status word; nothing on the GPU is made to stall)."""
    import torch.nn as nn
    from crb_b200 import BRAGPTQ, Binarization, _lib
    lin = nn.Linear(256, 64, bias=False).to(DEV)
    g = BRAGPTQ(lin, Binarization(lin.weight, method="crb", groupsize=128), salient_metric="hessian")
    g.verbose = False
    g.add_batch(torch.randn(1, 512, 256, device=DEV), None)
    g._hess_ws[:4].view(torch.int32).fill_(_lib.FLAG_WAIT_LIMIT)
    with pytest.raises(_lib.CrbError, match="WAIT_LIMIT"):
        g.fasterquant()
    g._hess_ws[:4].zero_()
