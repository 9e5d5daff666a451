"""Parity of the CUDA path (through the C ABI) with the reference's golden outputs and
with the CPU oracle on identical seeded inputs.  All tests here need a B200."""
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


@pytest.fixture(scope="module")
def blocks(golden_dir):
    return np.load(os.path.join(golden_dir, "blocks.npz"))


@pytest.fixture(scope="module")
def linear(golden_dir):
    return np.load(os.path.join(golden_dir, "linear.npz"))


@pytest.fixture(scope="module")
def config1(golden_dir):
    return np.load(os.path.join(golden_dir, "config1.npz"))


def run_block(ops, W, d, tech):
    """Runs the device block step on one [R,128] block with diag(U) = d."""
    Wd = W.to(DEV).clone()
    U = torch.diag(d).to(DEV)
    out = ops.block_step(Wd, U, 0, tech)
    torch.cuda.synchronize()
    return Wd.cpu(), {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in out.items()}


def compare_block(Wq, out, ref_masks, ref_errs, ref_Q, W, d, tech, what):
    tf = Hh.trace_fields(out["trace"])
    outcome = Hh.check_search_against_reference(tf, ref_errs, what)
    m1, m2, m3 = Hh.masks_from_codes(out["codes"])
    if outcome == "exact":
        assert torch.equal(m3, ref_masks[2]), f"{what}: salient mask"
        # elements whose metric equals the split value to the last bit may fall on either side
        diff = (m1 != ref_masks[0]).float().mean().item()
        assert diff == 0.0, f"{what}: low/mid masks differ on {diff:.2e} of the block"
        tol = 2e-5 if tech != "crbog" else 5e-5
        assert torch.allclose(Wq, ref_Q, rtol=tol, atol=1e-7), f"{what}: Q max diff {(Wq - ref_Q).abs().max()}"
    # partition property, Err and loss definitions hold regardless of ties
    assert bool(((m1.int() + m2.int() + m3.int()) == 1).all())
    assert bool((m3 == m3[0:1]).all()), "salient mask must be column structured"
    Err = (W - Wq) / d.reshape(1, -1)
    assert torch.allclose(out["Err"], Err, rtol=1e-6, atol=1e-9)
    loss = (((W - Wq) ** 2) / d.reshape(1, -1) ** 2).sum(1) / 2
    assert torch.allclose(out["losses"], loss, rtol=1e-5, atol=1e-12)
    return outcome


@pytest.mark.parametrize("tech", O.TECHNIQUES)
@pytest.mark.parametrize("ci", range(4))
def test_block_step_matches_reference(ops, blocks, ci, tech):
    W = torch.from_numpy(blocks[f"c{ci}_W"])
    d = torch.from_numpy(blocks[f"c{ci}_d"])
    ref_masks = [Hh.unpack(blocks[f"c{ci}_{n}"], W.shape) for n in ("m1", "m2", "m3")]
    ref_Q = torch.from_numpy(blocks[f"c{ci}_{tech}_Q"])
    Wq, out = run_block(ops, W, d, tech)
    compare_block(Wq, out, ref_masks, blocks[f"c{ci}_errs"], ref_Q, W, d, tech, f"case {ci} {tech}")


@pytest.mark.parametrize("tech", O.TECHNIQUES)
def test_block_codes_and_scales_match_oracle(ops, blocks, tech):
    """Sign planes and per-row scales against the oracle (signs >= 99.9 %, scales 1e-3)."""
    W = torch.from_numpy(blocks["c1_W"])
    d = torch.from_numpy(blocks["c1_d"])
    ref = O.block_step(W, d, tech)
    Wq, out = run_block(ops, W, d, tech)
    tf = Hh.trace_fields(out["trace"])
    if tf["n_salient"] != ref.trace.n_salient or tf["split_index"] != ref.trace.split_index:
        pytest.skip("search tie on this block; covered by test_block_step_matches_reference")
    assert Hh.sign_agreement(out["codes"], ref.codes) >= Hh.SIGN_AGREEMENT
    # second-pass means are rounding noise around zero: absolute floor tied to the block's scale
    atol = 1e-5 * float(ref.scales.abs().max())
    assert torch.allclose(out["scales"], ref.scales, rtol=Hh.SCALE_RTOL, atol=atol)
    assert abs(tf["split_value"] - ref.trace.split_value) <= 1e-7 * abs(ref.trace.split_value)
    assert np.array_equal(tf["top_cols"], ref.trace.top_cols.numpy())


@pytest.mark.parametrize("tech", O.TECHNIQUES)
@pytest.mark.parametrize("ci", (0, 3))
def test_binarize_group_matches_reference(ops, blocks, ci, tech):
    W = torch.from_numpy(blocks[f"c{ci}_W"])
    masks = [Hh.unpack(blocks[f"c{ci}_{n}"], W.shape) for n in ("m1", "m2", "m3")]
    for g, (m, order) in enumerate(zip(masks, (1, 1, 2))):
        q = ops.binarize_group(W.to(DEV), m.to(DEV), order, tech).cpu()
        ref = torch.from_numpy(blocks[f"c{ci}_{tech}_q{g}"])
        assert torch.allclose(q, ref, rtol=5e-5, atol=1e-7), (tech, g, (q - ref).abs().max())
    # element-structured mask with order 2 and empty rows (not produced by the block loop)
    m = masks[0].clone()
    m[::7] = False
    q = ops.binarize_group(W.to(DEV), m.to(DEV), 2, tech).cpu()
    ref = O.binarize(tech, W, m, 2)
    assert torch.allclose(q, ref, rtol=5e-5, atol=1e-7)
    assert bool((q[::7] == 0).all())


def test_gemm_f32_keeps_float32_accuracy(ops):
    """The split-TF32 tensor-core GEMM against float64, in every operand layout the path uses."""
    g = torch.Generator().manual_seed(11)
    cases = [(96, 384, 128, False, False), (300, 256, 256, True, False), (512, 512, 128, True, True),
             (128, 640, 384, False, False), (33, 128, 128, True, False)]
    for M, N, K, b_is_nk, lower in cases:
        A = torch.randn(M, K, generator=g) * torch.logspace(-3, 3, K)[None, :]      # wide dynamic range
        B = (torch.randn(N, K, generator=g) if b_is_nk else torch.randn(K, N, generator=g))
        C0 = torch.randn(M, N, generator=g)
        ref = (-0.5 * (A.double() @ (B.double().t() if b_is_nk else B.double())) + 2.0 * C0.double())
        mag = (A.double().abs() @ (B.double().abs().t() if b_is_nk else B.double().abs())) + C0.double().abs()
        Cd = C0.to(DEV).clone()
        ops.gemm_f32(A.to(DEV), B.to(DEV), Cd, alpha=-0.5, beta=2.0, b_is_nk=b_is_nk, lower_only=lower)
        got = Cd.cpu().double()
        err = ((got - ref).abs() / mag)
        if lower:   # 128 x 128 blocks above the diagonal are left untouched
            keep = torch.zeros(M, N, dtype=torch.bool)
            for mi in range(0, M, 128):
                keep[mi:mi + 128, mi + 128:] = True
            assert torch.equal(Cd.cpu()[keep], C0[keep])
            err = err[~keep]
        assert float(err.max()) < 3e-6, (M, N, K, b_is_nk, lower, float(err.max()))


def test_gemm_f32_triangular_operands_and_long_k(ops):
    """Operands promised lower triangular (their zero half is skipped), a rectangular lower-only
    update as the factorisation's outer panels issue it, and K = 1024 with beta = 1."""
    g = torch.Generator().manual_seed(12)
    for M, N, K, kind in [(384, 512, 512, "b"), (640, 256, 640, "a"), (512, 768, 768, "b"), (128, 128, 128, "a"),
                          (768, 384, 128, "rect"), (384, 640, 1024, "longk")]:
        A = torch.randn(M, K, generator=g)
        B = torch.randn(K, N, generator=g)
        C0 = torch.randn(M, N, generator=g)
        kw = {}
        if kind == "b":
            B = torch.tril(B)
            kw["b_lower"] = True
        if kind == "a":
            A = torch.tril(A)
            kw["a_lower"] = True
        beta = 1.0 if kind in ("rect", "longk") else 0.0
        if kind == "rect":
            kw["lower_only"] = True
        ref = 0.75 * (A.double() @ B.double()) + beta * C0.double()
        mag = A.double().abs() @ B.double().abs() + C0.double().abs()
        Cd = C0.to(DEV).clone()
        ops.gemm_f32(A.to(DEV), B.to(DEV), Cd, alpha=0.75, beta=beta, **kw)
        got = Cd.cpu().double()
        err = (got - ref).abs() / mag
        if kind == "rect":
            keep = torch.zeros(M, N, dtype=torch.bool)
            for mi in range(0, M, 128):
                keep[mi:mi + 128, mi + 128:] = True
            assert torch.equal(Cd.cpu()[keep], C0[keep])
            err = err[~keep]
        assert float(err.max()) < 3e-6, (M, N, K, kind, float(err.max()))


def test_grouped_linear_loop_matches_per_block_calls(ops):
    """crb_quantize_linear (updates grouped by 8 blocks) against block step + trailing update per block."""
    g = torch.Generator().manual_seed(21)
    R, C = 192, 128 * 11                    # one full group and a partial one
    W = torch.randn(R, C, generator=g) * 0.02
    U = torch.triu(torch.randn(C, C, generator=g) * (0.05 / C ** 0.5), 1) + torch.diag(0.5 + torch.rand(C, generator=g))
    Wa, Wb, Ud = W.to(DEV).clone(), W.to(DEV).clone(), U.to(DEV).contiguous()
    out = ops.quantize_linear(Wa, Ud, "braq", want_trace=True)
    loss_b = torch.zeros(R, device=DEV)
    agree = C // 128                       # blocks decided alike by both paths
    for b in range(C // 128):
        o = ops.block_step(Wb, Ud, b, "braq")
        loss_b += o["losses"]
        ops.trailing_update(Wb, o["Err"], Ud, b)
        ta, tb = Hh.trace_fields(out["trace"][b]), Hh.trace_fields(o["trace"])
        if (ta["n_salient"], ta["split_index"]) != (tb["n_salient"], tb["split_index"]):
            # only a near tie may be decided differently by the two association orders
            assert min(ta["salient_gap"], tb["salient_gap"], ta["split_gap"], tb["split_gap"]) < Hh.TIE_GAP
            agree = b
            break
    # every block up to the first such tie holds the same values (all of them without a tie)
    assert agree >= 8, "the first group (per-block updates on both paths) cannot differ"
    assert torch.allclose(Wa[:, :agree * 128], Wb[:, :agree * 128], rtol=1e-4, atol=1e-6)
    if agree == C // 128:
        assert torch.allclose(out["losses"], loss_b, rtol=1e-4)


def test_trailing_lookahead_gives_the_same_bits(ops):
    """The far part of a group's trailing update on a side stream beside the next group's block steps:
    every element receives the same products in the same order, so nothing may change."""
    g = torch.Generator().manual_seed(23)
    R, C = 320, 128 * 27                    # three full groups and a partial one
    W = torch.randn(R, C, generator=g) * 0.02
    U = torch.triu(torch.randn(C, C, generator=g) * (0.05 / C ** 0.5), 1) + torch.diag(0.5 + torch.rand(C, generator=g))
    Ud = U.to(DEV).contiguous()
    outs = []
    for mode in (0, 2, 2):
        old = ops.set_trailing_lookahead(mode)
        try:
            Wd = W.to(DEV).clone()
            o = ops.quantize_linear(Wd, Ud, "crb", want_trace=True)
            torch.cuda.synchronize()
        finally:
            ops.set_trailing_lookahead(old)
        assert ops.read_status(o["workspace"]) == 0
        outs.append((Wd.cpu(), o["losses"].cpu(), o["trace"].cpu()))
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.equal(a, b)


def test_trailing_update_matches_fp32_matmul(ops):
    g = torch.Generator().manual_seed(3)
    for R, C, blk in ((96, 384, 0), (257, 512, 2), (128, 256, 1)):
        W = torch.randn(R, C, generator=g)
        Err = torch.randn(R, 128, generator=g)
        U = torch.triu(torch.randn(C, C, generator=g))
        ref = W.clone()
        ed = (blk + 1) * 128
        ref[:, ed:] -= Err.matmul(U[blk * 128:ed, ed:])
        Wd = W.to(DEV)
        ops.trailing_update(Wd, Err.to(DEV), U.to(DEV), blk)
        assert torch.allclose(Wd.cpu(), ref, rtol=1e-5, atol=1e-4)
        assert torch.equal(Wd.cpu()[:, :ed], W[:, :ed])


def test_factor_lookahead_gives_the_same_bits(ops):
    """The rank-1024 updates split into the next panel's columns (caller's stream) and the rest (side
    stream) apply the same products to every element in the same order: U must not change by a bit."""
    C = 4096 + 1024                                          # five outer panels
    g = torch.Generator().manual_seed(11)
    X = torch.randn(2 * C, C, generator=g)
    H0 = ((X.t() @ X) / C).to(DEV)
    outs = []
    for enable in (False, True, True):
        old = ops.set_factor_lookahead(enable)
        try:
            H = H0.clone()
            ops.hinv_upper_factor(H, None, 0.01, restore=lambda h: h.copy_(H0))
            torch.cuda.synchronize()
        finally:
            ops.set_factor_lookahead(old)
        outs.append(H.cpu())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert torch.isfinite(outs[0]).all() and float(outs[0].diagonal().min()) > 0


@pytest.mark.parametrize("C", (128, 384, 1024, 4096))      # 4096: four outer panels, two levels of merges across them
def test_factor_matches_reference_chain(ops, C):
    g = torch.Generator().manual_seed(C)
    X = torch.randn(4 * C, C, generator=g)
    X[:, :3] *= 20
    H = (X.t() @ X) * (2.0 / 8)
    H[5, :] = 0
    H[:, 5] = 0                                   # a dead column
    W = torch.randn(64, C, generator=g)
    Wr, Hr = W.clone(), H.clone()
    U_ref = O.hinv_upper_factor(Hr, Wr, 0.01)     # float32 library chain, as the reference
    # float64 ground truth
    Hd = H.double().clone()
    Hd[5, 5] = 1
    Hd += 0.01 * torch.diag(Hd).mean() * torch.eye(C, dtype=torch.float64)
    U_true = torch.linalg.cholesky(torch.linalg.inv(Hd), upper=True)
    Hg, Wg = H.to(DEV).clone(), W.to(DEV).clone()
    U = ops.hinv_upper_factor(Hg, Wg, 0.01).cpu()
    assert torch.equal(Wg.cpu(), Wr)              # dead column zeroed
    assert bool((torch.tril(U, -1) == 0).all())
    err_dev = (U.double() - U_true).norm() / U_true.norm()
    err_ref = (U_ref.double() - U_true).norm() / U_true.norm()
    assert err_dev <= max(4 * err_ref, 1e-5), (float(err_dev), float(err_ref))
    d_dev = torch.diag(U).double()
    assert torch.allclose(d_dev, torch.diag(U_true), rtol=1e-4)


def test_factor_accuracy_on_ill_conditioned_hessian(ops):
    """Two outer panels of the blocked factorisation (C = 2048), a Hessian with a decaying spectrum
    (condition number ~4e4 after damping): the factor must be about as close to the float64 truth as
    the reference's float32 library chain is on a GPU, in norm and on the diagonal the block step
    divides by."""
    C = 2048
    g = torch.Generator().manual_seed(77)
    Z = torch.randn(3 * C, C, generator=g, dtype=torch.float64)
    Qm, _ = torch.linalg.qr(torch.randn(C, C, generator=g, dtype=torch.float64))
    X = (Z * torch.logspace(0, -2.5, C, dtype=torch.float64)) @ Qm.t()
    X[:, :4] *= 30
    H = ((X.t() @ X) * (2.0 / 64)).float()
    W = torch.randn(32, C, generator=g)
    U_cpu = O.hinv_upper_factor(H.clone(), W.clone(), 0.01)           # the oracle's float32 chain (LAPACK)
    # the same three library calls as the reference issues them on a GPU (bigptq.py:127-129)
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    Hg = H.to(DEV).clone()
    Hg += torch.eye(C, device=DEV) * (0.01 * torch.mean(torch.diag(Hg)))
    U_gpu = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(Hg)), upper=True).cpu()
    torch.backends.cuda.matmul.allow_tf32 = tf32
    Hd = H.double() + 0.01 * torch.diag(H.double()).mean() * torch.eye(C, dtype=torch.float64)
    U_true = torch.linalg.cholesky(torch.linalg.inv(Hd), upper=True)
    U = ops.hinv_upper_factor(H.to(DEV).clone(), W.to(DEV).clone(), 0.01).cpu()
    dt = torch.diag(U_true)

    def errors(V):
        return (float((V.double() - U_true).norm() / U_true.norm()),
                float(((torch.diag(V).double() - dt).abs() / dt).mean()))

    (e_dev, d_dev), (e_cpu, d_cpu), (e_gpu, d_gpu) = errors(U), errors(U_cpu), errors(U_gpu)
    assert e_dev <= max(1.5 * e_gpu, 4 * e_cpu), (e_dev, e_gpu, e_cpu)
    # the diagonal keeps a small systematic part (12 truncating tensor-core adds per K = 32 chunk)
    assert d_dev <= max(4.0 * d_gpu, 1e-5), (d_dev, d_gpu, d_cpu)


def test_factor_retry_and_fallback(ops):
    """A Hessian that is not positive definite takes the retry path and still returns a factor."""
    C = 256
    g = torch.Generator().manual_seed(9)
    A = torch.randn(C, C, generator=g)
    H = A + A.t()                                    # indefinite
    H[torch.arange(C), torch.arange(C)] = 1e-3
    U = ops.hinv_upper_factor(H.to(DEV).clone(), None, 0.01).cpu()
    assert torch.isfinite(U).all()
    assert bool((torch.diag(U) > 0).all())


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16, torch.float32))
def test_hessian_matches_float64(ops, dtype):
    g = torch.Generator().manual_seed(5)
    for T, C in ((300, 128), (2048, 384), (4096 + 64, 512)):
        X = torch.randn(T, C, generator=g)
        X[:, :2] *= 20
        Xd = X.to(dtype)
        ref = Xd.double().t() @ Xd.double()
        S = torch.zeros(C, C, device=DEV)
        Xg = Xd.to(DEV)
        half = (T // 2 // 8) * 8
        ops.hessian_accumulate(S, Xg[:half])         # accumulation over two calls
        ops.hessian_accumulate(S, Xg[half:])
        ops.hessian_finalize(S, 1.0)
        assert ops.hessian_status(DEV) == 0
        got = S.cpu().double()
        # tensor-core accumulation truncates: about 3e-8 relative per 16-token MMA step on a
        # same-sign running sum, bounded by the 2048-token chunking (x3 for the split float32 path)
        tol = 2e-5 if dtype == torch.float32 else 1e-5
        rel = (got - ref).norm() / ref.norm()
        assert rel < tol, (dtype, T, C, float(rel))
        assert torch.equal(got, got.t())
        dmax = ((torch.diag(got) - torch.diag(ref)).abs() / torch.diag(ref)).max()
        assert dmax < 2 * tol, float(dmax)


def test_hessian_matches_reference_add_batch(ops, linear):
    X = torch.from_numpy(linear["X"])
    nseq = int(linear["nseq"])
    ref = torch.from_numpy(linear["H"])
    S = torch.zeros(X.shape[1], X.shape[1], device=DEV)
    step = X.shape[0] // nseq
    for j in range(nseq):
        ops.hessian_accumulate(S, X[j * step:(j + 1) * step].to(DEV))
    ops.hessian_finalize(S, 2.0 / nseq)
    rel = (S.cpu() - ref).norm() / ref.norm()
    assert rel < 1e-5, float(rel)


@pytest.mark.parametrize("tech", O.TECHNIQUES)
def test_linear_given_reference_factor(ops, linear, tech):
    """Block loop + trailing updates with the reference's own factor U: per-block decisions
    must follow the reference (or be ties) and the result must match to rounding."""
    W = torch.from_numpy(linear["W"])
    H = torch.from_numpy(linear["H"]).clone()
    Wc = W.clone()
    U = O.hinv_upper_factor(H, Wc, 0.01)
    Wd = Wc.to(DEV).clone()
    out = ops.quantize_linear(Wd, U.contiguous().to(DEV), tech, want_codes=True)
    err = float(out["losses"].sum())
    assert ops.read_status(out["workspace"]) == 0
    ref_W = torch.from_numpy(linear[f"{tech}_Wq"])
    nblk = W.shape[1] // 128
    agree = nblk                            # blocks decided exactly like the reference
    for bi in range(nblk):
        tf = Hh.trace_fields(out["trace"][bi])
        # raises unless the decision is the reference's or a tie inside the band
        if Hh.check_search_against_reference(tf, linear[f"{tech}_b{bi}_errs"], f"{tech} block {bi}") != "exact":
            agree = bi
            break
    if agree:
        assert torch.allclose(Wd.cpu()[:, :agree * 128], ref_W[:, :agree * 128], rtol=1e-4, atol=1e-6)
    if agree == nblk:
        assert abs(err - float(linear[f"{tech}_error"])) <= 1e-4 * err
    X = torch.from_numpy(linear["X"])
    e_dev, e_ref = O.output_error(W, Wd.cpu(), X), O.output_error(W, ref_W, X)
    assert abs(e_dev - e_ref) <= Hh.OUTPUT_ERR_RTOL * e_ref


@pytest.mark.parametrize("tech", O.TECHNIQUES)
def test_bragptq_end_to_end(linear, tech):
    """The drop-in classes: add_batch x 6, fasterquant, against the reference's results."""
    import torch.nn as nn
    from crb_b200 import BRAGPTQ, Binarization
    W = torch.from_numpy(linear["W"])
    X = torch.from_numpy(linear["X"])
    nseq = int(linear["nseq"])
    lin = nn.Linear(W.shape[1], W.shape[0], bias=False)
    lin.weight.data = W.clone()
    lin = lin.to(DEV)
    g = BRAGPTQ(lin, Binarization(lin.weight, method=tech, groupsize=128), salient_metric="hessian")
    step = X.shape[0] // nseq
    for j in range(nseq):
        g.add_batch(X[j * step:(j + 1) * step].unsqueeze(0).to(DEV), None)
    assert g.nsamples == nseq
    Hfull = g.H.cpu()
    assert (Hfull - torch.from_numpy(linear["H"])).norm() / Hfull.norm() < 1e-5
    info = g.fasterquant(blocksize=128, percdamp=0.01)
    g.free()
    ref_W = torch.from_numpy(linear[f"{tech}_Wq"])
    Wq = lin.weight.data.cpu()
    e_dev, e_ref = O.output_error(W, Wq, X), O.output_error(W, ref_W, X)
    assert abs(e_dev - e_ref) <= Hh.OUTPUT_ERR_RTOL * e_ref, (e_dev, e_ref)
    assert abs(info["error"] - float(linear[f"{tech}_error"])) <= Hh.OUTPUT_ERR_RTOL * info["error"]
    # injected Hessian (the reference's diagnostics assign g.H / g.nsamples)
    lin2 = nn.Linear(W.shape[1], W.shape[0], bias=False)
    lin2.weight.data = W.clone()
    lin2 = lin2.to(DEV)
    g2 = BRAGPTQ(lin2, Binarization(lin2.weight, method=tech, groupsize=128), salient_metric="hessian")
    g2.H = torch.from_numpy(linear["H"]).to(DEV)
    g2.nsamples = nseq
    info2 = g2.fasterquant(blocksize=128)
    assert abs(info2["error"] - float(linear[f"{tech}_error"])) <= Hh.OUTPUT_ERR_RTOL * info2["error"]


@pytest.mark.parametrize("bi", (0, 9))
def test_config1_blocks(ops, config1, bi):
    """Two blocks of the 2048x2048 single-linear configuration (inputs captured from the reference run)."""
    W = torch.from_numpy(config1[f"b{bi}_Win"])
    d = torch.from_numpy(config1[f"b{bi}_d"])
    Wq, out = run_block(ops, W, d, "crb")
    tf = Hh.trace_fields(out["trace"])
    outcome = Hh.check_search_against_reference(tf, config1[f"b{bi}_errs"], f"config1 block {bi}")
    m1, m2, m3 = Hh.masks_from_codes(out["codes"])
    if outcome == "exact":
        assert np.array_equal(m3[0].nonzero().flatten().numpy(), config1[f"b{bi}_m3cols"])
        assert torch.equal(m1, Hh.unpack(config1[f"b{bi}_m1"], W.shape))
        ref_Q = torch.from_numpy(config1[f"b{bi}_Qout"])
        assert torch.allclose(Wq, ref_Q, rtol=2e-5, atol=1e-7)


def test_block_step_is_deterministic_and_row_count_agnostic(ops):
    """Full-size properties: two runs are bit-identical; ragged row counts work."""
    g = torch.Generator().manual_seed(77)
    for R in (1, 7, 4096, 16384 + 40, 36864):            # 36864: the tallest linear of the largest configuration
        W = torch.randn(R, 256, generator=g) * 0.02
        d = 0.5 + torch.rand(256, generator=g)
        U = torch.diag(d).to(DEV)
        outs = []
        for _ in range(2):
            Wd = W.to(DEV).clone()
            o = ops.block_step(Wd, U, 1, "crb")
            outs.append((Wd.cpu(), o["Err"].cpu(), o["codes"].cpu(), o["trace"].cpu()))
        assert all(torch.equal(a, b) for a, b in zip(outs[0], outs[1]))
        Wq, Err, codes, trace = outs[0]
        assert torch.equal(Wq[:, :128], W[:, :128])                 # other blocks untouched
        m1, m2, m3 = Hh.masks_from_codes(codes)
        assert bool(((m1.int() + m2.int() + m3.int()) == 1).all())
        tf = Hh.trace_fields(trace)
        assert 1 <= tf["n_salient"] <= 49 and 0 <= tf["split_index"] <= 80
        assert int(m3[0].sum()) == tf["n_salient"]
        # every row-group holds at most 2 (order 1) or 4 (order 2) distinct values
        for r in range(min(R, 5)):
            for grp, lim in ((m1, 2), (m2, 2), (m3, 4)):
                assert len(torch.unique(Wq[r, 128:][grp[r]])) <= lim


def test_split_quantiles_match_numpy(ops):
    """The device radix selection reproduces numpy.quantile on the metric (salient zeros included)."""
    g = torch.Generator().manual_seed(123)
    for R in (64, 3000):
        W = torch.randn(R, 128, generator=g) * 0.02
        W[::5, 7] = 0.0
        d = 0.5 + torch.rand(128, generator=g)
        Wq, out = run_block(ops, W, d, "braq")
        tf = Hh.trace_fields(out["trace"])
        ref = O.block_step(W, d, "braq")
        if tf["n_salient"] != ref.trace.n_salient:
            continue
        ws = out["workspace"]
        assert ws is not None
        assert tf["split_index"] == ref.trace.split_index or min(tf["split_gap"], ref.trace.split_gap) < Hh.TIE_GAP
        if tf["split_index"] == ref.trace.split_index:
            assert np.float32(tf["split_value"]) == np.float32(ref.trace.split_values[ref.trace.split_index])


def test_fused_selection_gives_the_same_bits(ops):
    """The cooperative one-kernel quantile selection and the three stream-ordered kernels are two
    schedules of the same phases: split values, decisions and outputs agree bit for bit, also on
    inputs with many equal values (whole bins of ties) and with exact zeros."""
    g = torch.Generator().manual_seed(5)
    for R, kind in ((33, "gauss"), (4096, "gauss"), (4096, "ties"), (16384 + 40, "gauss"), (2048, "zeros")):
        W = torch.randn(R, 256, generator=g) * 0.02
        if kind == "ties":
            W = torch.round(W * 200) / 200                          # a few dozen distinct values
        if kind == "zeros":
            W[:, 128 + 3::4] = 0.0
        d = 0.5 + torch.rand(256, generator=g)
        U = torch.diag(d).to(DEV)
        outs = []
        for fused in (False, True):
            old = ops.set_fused_selection(fused)
            try:
                Wd = W.to(DEV).clone()
                o = ops.block_step(Wd, U, 1, "crb")
                torch.cuda.synchronize()
            finally:
                ops.set_fused_selection(old)
            assert ops.read_status(o["workspace"]) == 0
            outs.append((Wd.cpu(), o["Err"].cpu(), o["codes"].cpu(), o["trace"].cpu()))
        for a, b in zip(outs[0], outs[1]):
            assert torch.equal(a, b), (R, kind)


@pytest.fixture(scope="module")
def variants(golden_dir):
    return np.load(os.path.join(golden_dir, "variants.npz"))


@pytest.mark.parametrize("tech", ("crb_norefine", "crb_symdamp", "crb_symdamp_norefine"))
@pytest.mark.parametrize("ci", (0, 3))
def test_crb_flag_variants_match_reference(ops, blocks, variants, ci, tech):
    """skip_refinement / symmetric_damp of the v7 binarizer (binary.py:2885-2890) on the device."""
    W = torch.from_numpy(blocks[f"c{ci}_W"])
    masks = [Hh.unpack(blocks[f"c{ci}_{n}"], W.shape) for n in ("m1", "m2", "m3")]
    for g, m in enumerate(masks):
        for order in (1, 2):
            q = ops.binarize_group(W.to(DEV), m.to(DEV), order, tech).cpu()
            ref = torch.from_numpy(variants[f"c{ci}_{tech}_g{g}_o{order}"])
            assert torch.allclose(q, ref, rtol=5e-5, atol=1e-7), (tech, g, order, (q - ref).abs().max())
    ragged = masks[0].clone()
    ragged[::7] = False
    q = ops.binarize_group(W.to(DEV), ragged.to(DEV), 2, tech).cpu()
    assert torch.allclose(q, torch.from_numpy(variants[f"c{ci}_{tech}_ragged_o2"]), rtol=5e-5, atol=1e-7)


@pytest.mark.parametrize("tech,orders", [("braq", (2, 2, 2)), ("crb", (2, 2, 2)), ("crb", (2, 1, 1)),
                                         ("crb_symdamp_norefine", (1, 1, 2))])
def test_bragptq_other_orders_and_variants(linear, variants, tech, orders):
    """fasterquant(orders=...) hands orders[i] to the quantizer of group i (bigptq.py:246-247)."""
    import torch.nn as nn
    from crb_b200 import BRAGPTQ, Binarization
    tag = f"{tech}_{''.join(map(str, orders))}"
    W = torch.from_numpy(linear["W"])
    lin = nn.Linear(W.shape[1], W.shape[0], bias=False)
    lin.weight.data = W.clone()
    lin = lin.to(DEV)
    g = BRAGPTQ(lin, Binarization(lin.weight, method=tech, groupsize=128), salient_metric="hessian")
    g.verbose = False
    g.H = torch.from_numpy(linear["H"]).to(DEV)
    g.nsamples = int(linear["nseq"])
    info = g.fasterquant(blocksize=128, percdamp=0.01, orders=orders)
    Wq = lin.weight.data.cpu()
    ref_W = torch.from_numpy(variants[f"{tag}_Wq"])
    nblk = W.shape[1] // 128
    agree = nblk
    for bi in range(nblk):
        tf = Hh.trace_fields(g.last_trace[bi])
        if Hh.check_search_against_reference(tf, variants[f"{tag}_b{bi}_errs"], f"{tag} block {bi}", rtol=1e-4) != "exact":
            agree = bi
            break
    if agree:
        close = torch.isclose(Wq[:, :agree * 128], ref_W[:, :agree * 128], rtol=1e-3, atol=1e-6).float().mean().item()
        assert close >= Hh.SIGN_AGREEMENT, (tag, close)
    X = torch.from_numpy(linear["X"])
    e_dev, e_ref = O.output_error(W, Wq, X), O.output_error(W, ref_W, X)
    assert abs(e_dev - e_ref) <= Hh.OUTPUT_ERR_RTOL * e_ref, (tag, e_dev, e_ref)
    assert abs(info["error"] - float(variants[f"{tag}_error"])) <= Hh.OUTPUT_ERR_RTOL * info["error"]


@pytest.mark.parametrize("ci", (0, 1, 3))
def test_magnitude_metric_block_matches_reference(ops, blocks, variants, ci):
    """salient_metric="magnitude" (utils/structure.py:11-12): signed metric values through the sort,
    the hole-based salient search and the two-tailed mid group of the split search."""
    W = torch.from_numpy(blocks[f"c{ci}_W"])
    d = torch.from_numpy(blocks[f"c{ci}_d"])
    Wd = W.to(DEV).clone()
    out = ops.block_step(Wd, torch.diag(d).to(DEV), 0, "crb", metric="magnitude")
    torch.cuda.synchronize()
    tf = Hh.trace_fields(out["trace"])
    outcome = Hh.check_search_against_reference(tf, variants[f"mag_c{ci}_errs"], f"magnitude case {ci}")
    g1, g2, g3 = Hh.masks_from_codes(out["codes"].cpu())
    assert bool(((g1.int() + g2.int() + g3.int()) == 1).all())
    if outcome == "exact":
        for got, name in ((g1, "m1"), (g2, "m2"), (g3, "m3")):
            assert torch.equal(got, Hh.unpack(variants[f"mag_c{ci}_{name}"], W.shape)), name
        ref_Q = torch.from_numpy(variants[f"mag_c{ci}_crb_Q"])
        assert torch.allclose(Wd.cpu(), ref_Q, rtol=2e-5, atol=1e-7), (Wd.cpu() - ref_Q).abs().max()


@pytest.mark.parametrize("tech", ("braq", "crb"))
def test_magnitude_metric_linear_matches_reference(linear, variants, tech):
    import torch.nn as nn
    from crb_b200 import BRAGPTQ, Binarization
    W = torch.from_numpy(linear["W"])
    lin = nn.Linear(W.shape[1], W.shape[0], bias=False)
    lin.weight.data = W.clone()
    lin = lin.to(DEV)
    g = BRAGPTQ(lin, Binarization(lin.weight, method=tech, groupsize=128), salient_metric="magnitude")
    g.verbose = False
    g.H = torch.from_numpy(linear["H"]).to(DEV)
    g.nsamples = int(linear["nseq"])
    info = g.fasterquant(blocksize=128, percdamp=0.01)
    Wq = lin.weight.data.cpu()
    ref_W = torch.from_numpy(variants[f"mag_{tech}_Wq"])
    nblk = W.shape[1] // 128
    agree = nblk
    for bi in range(nblk):
        tf = Hh.trace_fields(g.last_trace[bi])
        if Hh.check_search_against_reference(tf, variants[f"mag_{tech}_b{bi}_errs"], f"magnitude {tech} block {bi}",
                                             rtol=1e-4) != "exact":
            agree = bi
            break
    if agree:
        close = torch.isclose(Wq[:, :agree * 128], ref_W[:, :agree * 128], rtol=1e-3, atol=1e-6).float().mean().item()
        assert close >= Hh.SIGN_AGREEMENT, (tech, close)
    X = torch.from_numpy(linear["X"])
    e_dev, e_ref = O.output_error(W, Wq, X), O.output_error(W, ref_W, X)
    assert abs(e_dev - e_ref) <= Hh.OUTPUT_ERR_RTOL * e_ref, (tech, e_dev, e_ref)
    assert abs(info["error"] - float(variants[f"mag_{tech}_error"])) <= Hh.OUTPUT_ERR_RTOL * info["error"]


@pytest.mark.parametrize("C", (128, 384, 1024))
def test_hessian_pack_round_trip(ops, C):
    """The packed form holds exactly the tiles the accumulation maintains; summing packed partial
    sums and unpacking equals summing the matrices."""
    g = torch.Generator().manual_seed(C)
    parts = [torch.randn(C, C, generator=g).to(DEV) for _ in range(3)]
    n = ops.hessian_packed_floats(C)
    bands = torch.arange(C) // 256 * 256
    keep = (torch.arange(C)[None, :] >= bands[:, None]).to(DEV)             # row r keeps columns from its band on
    assert n == int(keep.sum())
    total = torch.zeros(n, device=DEV)
    for p in parts:
        buf = torch.empty(n, device=DEV)
        ops.hessian_pack(p, buf)
        assert torch.equal(buf, p[keep])
        total += buf
    out = torch.full((C, C), -7.0, device=DEV)
    ops.hessian_unpack(total, out)
    expect = torch.where(keep, parts[0] + parts[1] + parts[2], torch.full_like(out, -7.0))
    assert torch.equal(out, expect)
