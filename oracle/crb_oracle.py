"""CPU restatement of the CRB / BiLLM calibration-time binarization path.

TEST INFRASTRUCTURE ONLY: this module is the checker for the CUDA path and the
timed CPU baseline ("port").  The shipped package never imports it.

Parity status: PINNED.  `tests/golden/make_golden.py` imports the unmodified
reference, runs it on seeded inputs and stores its outputs; the tests in
`tests/test_oracle_golden.py` require this restatement to reproduce those
outputs (bit-exact masks / weights for braq and crb, 1e-6 for crbog).

Everything is float32 torch-on-CPU arithmetic in the same operation order as
the reference so that the argmin decisions of the two searches agree.  Each
function cites the reference lines it restates (paths inside the reference
project).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

TECHNIQUES = ("braq", "crbog", "crb")
# the same v7 function with skip_refinement / symmetric_damp set (binary.py:2885-2890)
CRB_VARIANTS = {"crb": (False, False), "crb_norefine": (True, False), "crb_symdamp": (False, True),
                "crb_symdamp_norefine": (True, True)}
SALIENT_LIMIT = 50          # utils/structure.py:16 passes up_lim=50 (bigptq.py:142)
N_SPLITS = 81               # utils/autosearch.py:65


# --------------------------------------------------------------------------------------
# Hessian accumulation                                              (bigptq.py:37-54)
# --------------------------------------------------------------------------------------
def hessian_add_batch(H: torch.Tensor, nsamples: int, inp: torch.Tensor) -> int:
    """Running Hessian update of BRAGPTQ.add_batch (bigptq.py:41-53), in place.

    `inp` is [tokens, C] or [batch, tokens, C]; the batch count is what the
    reference adds to `nsamples`.  Returns the new sample count.
    """
    if inp.dim() == 2:
        inp = inp.unsqueeze(0)
    b = inp.shape[0]
    x_t = inp.reshape(-1, inp.shape[-1]).t()          # C x tokens
    H *= nsamples / (nsamples + b)
    nsamples += b
    x_t = math.sqrt(2 / nsamples) * x_t.float()
    H += x_t.matmul(x_t.t())
    return nsamples


def hessian_from_tokens(x: torch.Tensor, n_sequences: int) -> torch.Tensor:
    """H built by `n_sequences` successive add_batch calls on equal slices of x [T, C]."""
    T, C = x.shape
    H = torch.zeros(C, C)
    n = 0
    step = T // n_sequences
    for j in range(n_sequences):
        n = hessian_add_batch(H, n, x[j * step:(j + 1) * step])
    return H


# --------------------------------------------------------------------------------------
# Damping + factorisation                                          (bigptq.py:101-129)
# --------------------------------------------------------------------------------------
def hinv_upper_factor(H: torch.Tensor, W: torch.Tensor, percdamp: float) -> torch.Tensor:
    """Dead-column fix, damping and U = chol(inv(H), upper)  (bigptq.py:103-129).

    Mutates H and W exactly like the reference (dead columns: H[d,d]=1, W[:,d]=0).
    """
    C = H.shape[0]
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W[:, dead] = 0
    idx = torch.arange(C)
    H[idx, idx] += percdamp * torch.mean(torch.diag(H))
    L = None
    for _ in range(10):                                   # bigptq.py:115-123
        try:
            L = torch.linalg.cholesky(H)
            break
        except torch._C._LinAlgError:
            extra = 1e-3 * torch.mean(torch.diag(H))
            if extra == 0:
                extra = 1e-6
            H[idx, idx] += extra
    if L is None:                                         # bigptq.py:124-126
        L = torch.diag(torch.sqrt(torch.diag(H).clamp(min=1e-8)))
    Hinv = torch.cholesky_inverse(L)
    return torch.linalg.cholesky(Hinv, upper=True)


# --------------------------------------------------------------------------------------
# Binarizers
# --------------------------------------------------------------------------------------
def _masked_mean(v: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Row mean over mask with the reference's nanmean-then-zero rule (binary.py:28-29)."""
    cnt = mask.sum(dim=1)
    s = torch.where(mask, v, torch.zeros((), dtype=v.dtype)).sum(dim=1)
    m = s / cnt
    return torch.where(cnt == 0, torch.zeros_like(m), m)


def braq_residual(x: torch.Tensor, mask: torch.Tensor, order: int,
                  parts: Optional[list] = None) -> torch.Tensor:
    """Residual binary expansion `high_order_residual` (binary.py:18-39).

    Each pass: mu = masked row mean of the residual, alpha = masked mean |r-mu|,
    add (mu + alpha*sign(r-mu)) on the mask.  `parts` (optional) receives
    (mu, alpha, sign) per pass.
    """
    total = torch.zeros_like(x)
    base = x * mask
    for _ in range(order):
        r = base - total
        mu = _masked_mean(r, mask)
        dev = r - mu[:, None]
        alpha = _masked_mean(dev.abs(), mask)
        s = torch.where(mask, torch.sign(dev), torch.zeros((), dtype=x.dtype))
        piece = s * alpha[:, None]
        piece += mu[:, None]
        total = total + piece * mask
        if parts is not None:
            parts.append((mu, alpha, s))
    return total


def _crb_solve(B1, B2, c1w, c2w, d, maskf, lam, corr_damp, symmetric_damp=False):
    """Damped, Tikhonov-regularised 2x2 solve of CRB v7 (binary.py:1582-1596)."""
    c12 = (B1 * B2 * maskf).sum(dim=1)
    if symmetric_damp:                                    # binary.py:1584-1585
        c12 = c12 * (1.0 - corr_damp)
    else:
        c12 = torch.where(c12 > 0, c12 * (1.0 - corr_damp), c12)
    A = d + lam
    den = A * A - c12 * c12
    ok = den.abs() > 1e-12
    den_s = torch.where(ok, den, torch.ones_like(den))
    a1 = torch.clamp((A * c1w - c12 * c2w) / den_s, min=0.0)
    a2 = torch.clamp((A * c2w - c12 * c1w) / den_s, min=0.0)
    zero = torch.zeros_like(a1)
    return torch.where(ok, a1, zero), torch.where(ok, a2, zero)


def crb_binarize(x: torch.Tensor, mask: torch.Tensor, order: int, lam: float = 1e-5,
                 corr_damp: float = 0.1, parts: Optional[list] = None, skip_refinement: bool = False,
                 symmetric_damp: bool = False) -> torch.Tensor:
    """`coupled_residual_binarization_stable_v7` (binary.py:1544-1638).

    order 1: mean + alpha*sign (binary.py:1570-1576); order 2: two coupled
    expansions, joint scale solve, two sign refinements, residual-mean
    correction (binary.py:1598-1636).
    """
    mf = mask.float()
    base = x.clone() * mask
    d = mf.sum(dim=1)
    dsafe = torch.clamp(d, min=1.0)
    mu = (base * mf).sum(dim=1) / dsafe
    c = (base - mu[:, None]) * mf
    B1 = torch.sign(c) * mf
    a_init = (c.abs() * mf).sum(dim=1) / dsafe
    if order == 1:
        if parts is not None:
            parts.append((mu, a_init, B1))
        return (mu[:, None] + a_init[:, None] * B1) * mf

    def centred_sign(t):
        tm = (t * mf).sum(dim=1) / dsafe
        return torch.sign((t - tm[:, None]) * mf) * mf

    B2 = centred_sign((c - a_init[:, None] * B1) * mf)
    c1w = (c * B1).sum(dim=1)
    c2w = (c * B2).sum(dim=1)
    a1, a2 = _crb_solve(B1, B2, c1w, c2w, d, mf, lam, corr_damp, symmetric_damp)
    if not skip_refinement:                                            # binary.py:1617
        B2 = centred_sign((c - a1[:, None] * B1) * mf)                 # step 5
        c2w = (c * B2).sum(dim=1)
        a1, a2 = _crb_solve(B1, B2, c1w, c2w, d, mf, lam, corr_damp, symmetric_damp)
        B1 = centred_sign((c - a2[:, None] * B2) * mf)                 # step 6
        c1w = (c * B1).sum(dim=1)
        a1, a2 = _crb_solve(B1, B2, c1w, c2w, d, mf, lam, corr_damp, symmetric_damp)
    approx = (a1[:, None] * B1 + a2[:, None] * B2) * mf            # step 7
    resid = (c - approx) * mf
    mu_fix = (resid * mf).sum(dim=1) / dsafe
    if parts is not None:
        parts.append((mu, mu_fix, a1, a2, B1, B2))
    return (mu[:, None] + mu_fix[:, None] + a1[:, None] * B1 + a2[:, None] * B2) * mf


def crbog_binarize(x: torch.Tensor, mask: torch.Tensor, order: int,
                   parts: Optional[list] = None) -> torch.Tensor:
    """`coupled_residual_binarization` (binary.py:577-687).

    order 1 is the braq single pass (binary.py:595-630).  order 2 is the
    reference's per-row loop (binary.py:644-685) evaluated for all rows at
    once: float32 sums, the 2x2 solve in float64, alphas rounded to float32
    before they scale the sign planes.
    """
    if order == 1:
        return braq_residual(x, mask, 1, parts)
    R = x.shape[0]
    same_cols = bool((mask == mask[0:1]).all())
    if same_cols:
        cols = mask[0].nonzero().flatten()
        v = x[:, cols].contiguous()
        m = torch.ones_like(v, dtype=torch.bool)
    else:
        cols = None
        v, m = x * mask, mask
    n = m.sum(dim=1)
    has = n > 0
    nf = n.float()
    zero = torch.zeros((), dtype=x.dtype)
    mu = torch.where(m, v, zero).sum(dim=1) / nf
    c = torch.where(m, v - mu[:, None], zero)
    B1 = torch.sign(c)
    a1 = c.abs().sum(dim=1) / nf
    r = torch.where(m, c - a1[:, None] * B1, zero)
    B2 = torch.sign(r)
    a2 = r.abs().sum(dim=1) / nf
    dd = nf.double()
    c12 = (B1 * B2).sum(dim=1).double()
    c1w = (c * B1).sum(dim=1).double()
    c2w = (c * B2).sum(dim=1).double()
    det = dd * dd - c12 * c12
    ok = det.abs() > 1e-12
    det_s = torch.where(ok, det, torch.ones_like(det))
    n1 = torch.clamp((c1w * dd - c2w * c12) / det_s, min=0.0).float()
    n2 = torch.clamp((c2w * dd - c1w * c12) / det_s, min=0.0).float()
    a1 = torch.where(ok, n1, a1)
    a2 = torch.where(ok, n2, a2)
    q = mu[:, None] + a1[:, None] * B1 + a2[:, None] * B2
    q = torch.where(m & has[:, None], q, zero)
    if parts is not None:
        parts.append((mu, a1, a2, B1, B2, cols))
    if cols is None:
        return q
    out = torch.zeros_like(x)
    out[:, cols] = q
    return out


def binarize(technique: str, x, mask, order, lam=1e-5, corr_damp=0.1, parts=None):
    """Dispatch of `Binarization.quantize` for the three techniques (binary.py:2875-2884)."""
    if technique == "braq":
        return braq_residual(x, mask, order, parts)
    if technique == "crbog":
        return crbog_binarize(x, mask, order, parts)
    if technique in CRB_VARIANTS:
        skip, sym = CRB_VARIANTS[technique]
        return crb_binarize(x, mask, order, lam, corr_damp, parts, skip, sym)
    raise NotImplementedError(technique)


# --------------------------------------------------------------------------------------
# Structural partition search                  (utils/structure.py, autosearch.py, mask.py)
# --------------------------------------------------------------------------------------
def quantile_linear_f32(flat: np.ndarray, probs: np.ndarray) -> np.ndarray:
    """numpy.quantile(method='linear') for float32 data and float32 probabilities.

    Restates numpy 2.x (lib/_function_base_impl.py `_quantile`, `_lerp`) as it is
    reached from utils/autosearch.py:66-68: the virtual index (N-1)*p is formed
    in float32, so is the fractional weight, and the interpolation is
    a + (b-a)*t for t < 0.5, b - (b-a)*(1-t) otherwise, all float32.
    """
    flat = np.asarray(flat, dtype=np.float32)
    probs = np.asarray(probs, dtype=np.float32)
    n = flat.size
    vidx = np.float32(n - 1) * probs
    lo = np.floor(vidx)
    t = (vidx - lo).astype(np.float32)
    lo = lo.astype(np.int64)
    hi = np.minimum(lo + 1, n - 1)
    need = np.unique(np.concatenate([lo, hi]))
    part = np.partition(flat, need)
    a, b = part[lo], part[hi]
    diff = b - a
    out = a + diff * t
    alt = b - diff * (np.float32(1) - t)
    return np.where(t >= np.float32(0.5), alt, out).astype(np.float32)


def split_masks(M: torch.Tensor, mask3: torch.Tensor, border) -> Tuple[torch.Tensor, torch.Tensor]:
    """`generate_structural_mask` (utils/mask.py:7-18): low (< border) / mid (>= border)."""
    rest = ~mask3
    g = torch.abs(M * rest)
    return (g < border) * rest, (g >= border) * rest


@dataclass
class SearchTrace:
    """Everything the two searches decide for one block."""
    top_cols: torch.Tensor            # the 50 highest-score columns, best first
    salient_err: List[float]          # 49 float32 means, candidate i = index + 1
    n_salient: int
    split_values: np.ndarray          # 81 float32 split candidates
    split_err: List[float]            # 81 float32 means
    split_index: int
    split_value: float

    @staticmethod
    def _gap(errs: Sequence[float], best: int) -> float:
        e = np.asarray(errs, dtype=np.float64)
        others = np.delete(e, best)
        return float((others.min() - e[best]) / max(abs(e[best]), 1e-300))

    @property
    def salient_gap(self) -> float:
        """Relative distance from the winning salient count to the runner-up."""
        return self._gap(self.salient_err, self.n_salient - 1)

    @property
    def split_gap(self) -> float:
        return self._gap(self.split_err, self.split_index)


def _mse(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.mean((a - b) ** 2)                       # utils/autosearch.py:8-10


def search_partition(M: torch.Tensor, up_lim: int = SALIENT_LIMIT):
    """`structural_searching` (utils/autosearch.py:28-83).

    Stage 1 (autosearch.py:37-55): column score = sum_r |M|; the top `up_lim`
    columns, best first; for i = 1..up_lim-1 the error of order-2 braq on the
    top-i columns plus order-2 braq on the rest; first strict minimum wins.
    Stage 2 (autosearch.py:57-81): 81 quantiles (0.10..0.90) of |M * ~mask3|
    (zeros at salient columns included); for each the error of order-1 braq on
    the two sides plus the salient group; first strict minimum wins.
    Returns (split value as 0-dim float32 tensor, mask3, trace).
    """
    R, B = M.shape
    score = M.abs().sum(dim=0)
    _, top = torch.topk(score, up_lim)
    best_i, best_e = max(1, up_lim // 3), float("inf")
    sal_err = []
    for i in range(1, up_lim):
        m3 = torch.zeros(R, B, dtype=torch.bool)
        m3[:, top[:i]] = True
        e = _mse(M, braq_residual(M, ~m3, 2) + braq_residual(M, m3, 2))
        sal_err.append(e.item())
        if e < best_e:
            best_e, best_i = e, i
    _, top_best = torch.topk(score, best_i)
    mask3 = torch.zeros(R, B, dtype=torch.bool)
    mask3[:, top_best] = True
    g3 = braq_residual(M, mask3, 2)

    flat = torch.abs(M * (~mask3)).view(-1)
    probs = torch.linspace(0.10, 0.90, N_SPLITS)
    pvals = torch.tensor(np.quantile(flat.numpy(), q=probs.numpy()))
    best_p, best_e2, best_k = pvals[len(pvals) // 2], float("inf"), -1
    split_err = []
    for k, p in enumerate(pvals):
        m1, m2 = split_masks(M, mask3, p)
        e = _mse(M, braq_residual(M, m1, 1) + braq_residual(M, m2, 1) + g3)
        split_err.append(e.item())
        if e < best_e2:
            best_e2, best_p, best_k = e, p, k
    trace = SearchTrace(top.clone(), sal_err, best_i, pvals.numpy().copy(), split_err,
                        best_k, float(best_p))
    return best_p, mask3, trace


def hessian_metric(W_blk: torch.Tensor, u_diag: torch.Tensor) -> torch.Tensor:
    """Salience metric w^2 / diag(U)^2 (utils/structure.py:10)."""
    return W_blk ** 2 / (u_diag.reshape(1, -1)) ** 2


def partition_block(W_blk: torch.Tensor, u_diag: torch.Tensor, metric: str = "hessian"):
    """`structural_guassian_distribution` (utils/structure.py:8-20) -> (m1, m2, m3, trace)."""
    if metric == "hessian":
        M = hessian_metric(W_blk, u_diag)
    elif metric == "magnitude":
        M = W_blk
    else:
        raise NotImplementedError(metric)
    p, mask3, trace = search_partition(M, SALIENT_LIMIT)
    m1, m2 = split_masks(M, mask3, p)
    return m1, m2, mask3, trace


# --------------------------------------------------------------------------------------
# Block step and the whole per-linear loop                 (bigptq.py:131-148, 235-291)
# --------------------------------------------------------------------------------------
@dataclass
class BlockResult:
    Q: torch.Tensor                   # R x B quantised block
    Err: torch.Tensor                 # R x B  (w - q) / d
    loss_rows: torch.Tensor           # R      sum_j (w - q)^2 / d^2  (not yet halved)
    masks: Tuple[torch.Tensor, torch.Tensor, torch.Tensor]
    trace: SearchTrace
    codes: torch.Tensor               # R x B uint8: bits0-1 B1+1, bits2-3 B2+1, bits4-5 group
    scales: torch.Tensor              # R x 8 float32, see `block_step`


def block_step(W_blk: torch.Tensor, u_diag: torch.Tensor, technique: str = "crb",
               lam: float = 1e-5, corr_damp: float = 0.1, metric: str = "hessian",
               orders: Sequence[int] = (1, 1, 2)) -> BlockResult:
    """One 128-column block of the legacy partition=3 path (bigptq.py:142-263).

    scales columns: 0 mu_low, 1 alpha_low, 2 mu_mid, 3 alpha_mid, then for the
    salient group braq: 4 mu1, 5 alpha1, 6 mu2, 7 alpha2;  crb: 4 mu+mu_fix,
    5 alpha1, 6 alpha2, 7 0;  crbog: 4 mu, 5 alpha1, 6 alpha2, 7 0.
    """
    W1 = W_blk.clone()
    m1, m2, m3, trace = partition_block(W1, u_diag, metric)
    R, B = W1.shape
    Q = torch.zeros_like(W1)
    codes = torch.zeros(R, B, dtype=torch.uint8)
    scales = torch.zeros(R, 8)
    for g, (mask, order) in enumerate(zip((m1, m2, m3), orders)):
        parts: list = []
        qg = binarize(technique, W1, mask, order, lam, corr_damp, parts)
        Q += qg * mask
        s1 = torch.zeros(R, B)
        s2 = torch.zeros(R, B)
        if order == 1:
            mu, al, s = parts[0]
            scales[:, 2 * g], scales[:, 2 * g + 1] = mu, al
            s1 = s
        elif g < 2:
            # two expansions on the low / mid group (orders other than (1, 1, 2)): sign planes
            # only, the 8 scale slots are laid out for the default orders
            if technique == "braq":
                s1, s2 = parts[0][2], parts[1][2]
            elif technique in CRB_VARIANTS:
                s1, s2 = parts[0][4], parts[0][5]
            else:
                b1_, b2_, cols_ = parts[0][3], parts[0][4], parts[0][5]
                if cols_ is None:
                    s1, s2 = b1_, b2_
                else:
                    s1[:, cols_], s2[:, cols_] = b1_, b2_
        elif technique == "braq":
            (mu1, al1, sa), (mu2, al2, sb) = parts
            scales[:, 4], scales[:, 5], scales[:, 6], scales[:, 7] = mu1, al1, mu2, al2
            s1, s2 = sa, sb
        elif technique in CRB_VARIANTS:
            mu, mu_fix, a1, a2, b1, b2 = parts[0]
            scales[:, 4], scales[:, 5], scales[:, 6] = mu + mu_fix, a1, a2
            s1, s2 = b1, b2
        else:
            mu, a1, a2, b1, b2, cols = parts[0]
            scales[:, 4], scales[:, 5], scales[:, 6] = mu, a1, a2
            if cols is None:
                s1, s2 = b1, b2
            else:
                s1[:, cols], s2[:, cols] = b1, b2
        code = ((s1 + 1).to(torch.uint8) | ((s2 + 1).to(torch.uint8) << 2) | (g << 4))
        codes = torch.where(mask, code.to(torch.uint8), codes)
    d = u_diag.reshape(1, -1)
    Err = (W1 - Q) / d
    loss = ((W1 - Q) ** 2 / d ** 2).sum(dim=1)
    return BlockResult(Q, Err, loss, (m1, m2, m3), trace, codes, scales)


@dataclass
class LinearResult:
    W: torch.Tensor                   # R x C float32 after the loop (all quantised)
    error: float                      # sum(Losses), the value fasterquant returns
    U: torch.Tensor
    blocks: List[BlockResult] = field(default_factory=list)


def quantize_linear(W: torch.Tensor, H: torch.Tensor, technique: str = "crb",
                    blocksize: int = 128, percdamp: float = 0.01, lam: float = 1e-5,
                    corr_damp: float = 0.1, metric: str = "hessian",
                    keep_blocks: bool = True, U: Optional[torch.Tensor] = None,
                    orders: Sequence[int] = (1, 1, 2)) -> LinearResult:
    """`BRAGPTQ.fasterquant` for crb/crbog/braq with partition=3 (bigptq.py:56-291).

    W [R, C] float32 (cloned), H [C, C] float32 (consumed).  If `U` is given the
    factorisation is skipped (used to drive the CUDA path and the oracle from
    the same factor).
    """
    W = W.clone().float()
    R, C = W.shape
    if U is None:
        U = hinv_upper_factor(H, W, percdamp)
    losses = torch.zeros(R)
    res = LinearResult(W, 0.0, U)
    for st in range(0, C, blocksize):
        ed = min(st + blocksize, C)
        blk = block_step(W[:, st:ed], torch.diag(U[st:ed, st:ed]), technique, lam,
                         corr_damp, metric, orders)
        W[:, st:ed] = blk.Q
        losses += blk.loss_rows / 2
        W[:, ed:] -= blk.Err.matmul(U[st:ed, ed:])
        if keep_blocks:
            res.blocks.append(blk)
    res.error = torch.sum(losses).item()
    return res


def output_error(W_ref: torch.Tensor, Wq: torch.Tensor, X: torch.Tensor) -> float:
    """||(W - Q) X||_F over calibration tokens X [T, C], accumulated in float64."""
    D = (W_ref.double() - Wq.double())
    return float(torch.linalg.norm(X.double() @ D.t()))
