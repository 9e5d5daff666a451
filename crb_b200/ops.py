"""Tensor-level wrappers around the C ABI (device tensors in, device tensors out).

Every function here runs hand-written sm_100a kernels from libcrb_b200.so on the
current CUDA stream.  There is no CPU or PyTorch fallback: a non-CUDA tensor or a
missing library raises.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import _lib
from ._lib import BLOCK, TRACE_DOUBLES, CrbError, check, lib, ptr, stream_ptr

_workspaces: Dict[tuple, torch.Tensor] = {}


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise CrbError("crb_b200 runs on CUDA tensors only (no CPU fallback)")


def _workspace(kind: str, nbytes: int, device) -> torch.Tensor:
    """Zero-initialised, cached scratch buffer per (kind, device, current stream); grows on demand.

    Keying by stream lets several linears be processed concurrently on different streams
    without sharing scratch memory."""
    key = (kind, torch.device(device).index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def release_workspaces():
    _workspaces.clear()


def _dtype_code(t: torch.Tensor) -> int:
    name = str(t.dtype).replace("torch.", "")
    if name not in _lib.DTYPES:
        raise CrbError(f"unsupported activation dtype {t.dtype}")
    return _lib.DTYPES[name]


# ------------------------------------------------------------------------------------------
def hessian_accumulate(S: torch.Tensor, X: torch.Tensor) -> torch.Tensor:
    """S += X^T X.  S [C, C] float32 (upper-triangle tiles are maintained), X [T, C].

    Returns the workspace of the call; its first word collects the kernel's status flags
    (CRB_FLAG_WAIT_LIMIT if a bounded wait ran out), see `read_status`."""
    _need_cuda(S, X)
    if X.dim() != 2 or S.shape != (X.shape[1], X.shape[1]) or S.dtype != torch.float32:
        raise CrbError("hessian_accumulate: X must be [T, C] and S [C, C] float32")
    if X.stride(1) != 1:
        X = X.contiguous()
    if not S.is_contiguous():
        raise CrbError("S must be contiguous")
    T, Cc = X.shape
    code = _dtype_code(X)
    L = lib()
    nbytes = L.crb_hessian_workspace_bytes(Cc, T, code)
    ws = _workspace("hessian", nbytes, S.device)
    check(L.crb_hessian_accumulate(ptr(X), code, T, Cc, X.stride(0), ptr(S), ptr(ws), ws.numel(),
                                   stream_ptr()), "crb_hessian_accumulate")
    return ws


def hessian_finalize(S: torch.Tensor, scale: float) -> None:
    """In place: H = scale * S, lower triangle mirrored from the upper one."""
    _need_cuda(S)
    check(lib().crb_hessian_finalize(ptr(S), S.shape[0], float(scale), stream_ptr()), "crb_hessian_finalize")


def hessian_packed_floats(C: int) -> int:
    return int(lib().crb_hessian_packed_floats(int(C)))


def hessian_pack(S: torch.Tensor, packed: torch.Tensor) -> None:
    """The maintained (upper-triangle tile) part of S [C, C] -> packed [hessian_packed_floats(C)]."""
    _need_cuda(S, packed)
    check(lib().crb_hessian_pack(ptr(S), S.shape[0], ptr(packed), stream_ptr()), "crb_hessian_pack")


def hessian_unpack(packed: torch.Tensor, S: torch.Tensor) -> None:
    _need_cuda(S, packed)
    check(lib().crb_hessian_unpack(ptr(packed), S.shape[0], ptr(S), stream_ptr()), "crb_hessian_unpack")


def hessian_status(device) -> int:
    ws = _workspaces.get(("hessian", torch.device(device).index, torch.cuda.current_stream(device).cuda_stream))
    return 0 if ws is None else lib().crb_read_status(ptr(ws), stream_ptr())


def factor_enqueue(H: torch.Tensor, W: Optional[torch.Tensor], percdamp: float, extra_damp_steps: int,
                   status: torch.Tensor) -> None:
    """Enqueues one factorisation attempt (no host synchronisation): H is overwritten by U and
    `status[0]` receives CRB_FLAG_BAD_PIVOT if a pivot was not positive."""
    _need_cuda(H, W, status)
    Cc = H.shape[0]
    if H.dtype != torch.float32 or not H.is_contiguous() or H.shape != (Cc, Cc):
        raise CrbError("H must be a contiguous [C, C] float32 tensor")
    if W is not None and (W.dtype != torch.float32 or W.stride(1) != 1):
        raise CrbError("W must be float32 with unit column stride")
    L = lib()
    ws = _workspace("factor", L.crb_factor_workspace_bytes(Cc), H.device)
    check(L.crb_hinv_upper_factor(ptr(H), Cc, ptr(W), 0 if W is None else W.shape[0],
                                  0 if W is None else W.stride(0), float(percdamp), int(extra_damp_steps),
                                  ptr(ws), ws.numel(), ptr(status), stream_ptr()), "crb_hinv_upper_factor")


def diagonal_fallback(H: torch.Tensor, diag0: torch.Tensor, percdamp: float, max_retries: int = 10) -> torch.Tensor:
    """Last resort of bigptq.py:124-126 after every damping retry failed: U = diag(1/sqrt(diag H))."""
    diag = diag0.clone()
    diag[diag == 0] = 1
    mean = diag.mean()
    damp = percdamp * mean
    mean = mean + damp
    for _ in range(max_retries):
        extra = 1e-3 * mean
        damp = damp + extra
        mean = mean + extra
    H.zero_()
    torch.diagonal(H).copy_(torch.rsqrt(torch.clamp(diag + damp, min=1e-8)))
    return H


def hinv_upper_factor(H: torch.Tensor, W: Optional[torch.Tensor], percdamp: float,
                      max_retries: int = 10, restore=None) -> torch.Tensor:
    """Dead-column fix, damping and U = chol(inv(H), upper), written over H (returned).

    Mirrors bigptq.py:101-129 including the retry with extra damping: the device
    factorisation reports a failed pivot through a status word, and the host then
    rebuilds from the saved H with one more damping step, up to 10 times; after that
    the diagonal fallback of bigptq.py:124-126 is used.  `restore(H)` refills H with the
    undamped Hessian for a retry; without it a copy of H is kept for that purpose.
    """
    status = torch.zeros(4, dtype=torch.int32, device=H.device)
    saved = H.clone() if restore is None else None
    diag0 = torch.diagonal(H).clone()
    for attempt in range(max_retries):          # extra damping steps 0 .. 9, like bigptq.py:115-123
        if attempt > 0:
            if restore is None:
                H.copy_(saved)
            else:
                restore(H)
            status.zero_()
        factor_enqueue(H, W, percdamp, attempt, status)
        flags = int(status[0].item())
        if flags & _lib.FLAG_WAIT_LIMIT:
            raise CrbError("factorisation: a bounded wait inside a kernel ran out (CRB_FLAG_WAIT_LIMIT)")
        if not (flags & _lib.FLAG_BAD_PIVOT):
            return H
    return diagonal_fallback(H, diag0, percdamp, max_retries)


def block_step(W: torch.Tensor, U: torch.Tensor, block: int, technique: str = "crb",
               lam: float = 1e-5, corr_damp: float = 0.1, metric: str = "hessian",
               losses: Optional[torch.Tensor] = None, want_codes: bool = True,
               orders=(1, 1, 2), reuse: Optional[dict] = None) -> dict:
    """One 128-column block in place on W; returns Err, losses, codes, scales, trace.

    `scales` are produced for the default orders (1, 1, 2) only (None otherwise).  `reuse` takes the
    dict an earlier call on the same shape returned: its buffers are written again instead of
    allocating new ones (losses keep accumulating)."""
    _need_cuda(W, U)
    R = W.shape[0]
    L = lib()
    ws = _workspace("block", L.crb_block_workspace_bytes(R), W.device)
    dev = W.device
    ocode = _lib.orders_code(orders)
    if reuse is not None:
        Err, losses, codes, scales, trace = (reuse[k] for k in ("Err", "losses", "codes", "scales", "trace"))
    else:
        Err = torch.empty(R, BLOCK, dtype=torch.float32, device=dev)
        if losses is None:
            losses = torch.zeros(R, dtype=torch.float32, device=dev)
        codes = torch.zeros(R, BLOCK, dtype=torch.uint8, device=dev) if want_codes else None
        scales = torch.zeros(R, 8, dtype=torch.float32, device=dev) \
            if want_codes and ocode == _lib.ORDERS_DEFAULT else None
        trace = torch.zeros(TRACE_DOUBLES, dtype=torch.float64, device=dev)
    check(L.crb_block_step(ptr(W), R, W.stride(0), ptr(U), U.stride(0), block,
                           _lib.TECHNIQUES[technique], ocode, lam, corr_damp, _lib.METRICS[metric],
                           ptr(Err), ptr(losses), ptr(codes), ptr(scales), ptr(trace), ptr(ws),
                           ws.numel(), stream_ptr()), "crb_block_step")
    return dict(Err=Err, losses=losses, codes=codes, scales=scales, trace=trace, workspace=ws)


def block_step_static(W: torch.Tensor, U: torch.Tensor, block: int, technique: str = "crb",
                      lam: float = 1e-5, corr_damp: float = 0.1, metric: str = "hessian", *,
                      Err: torch.Tensor, losses: torch.Tensor, codes: Optional[torch.Tensor] = None,
                      scales: Optional[torch.Tensor] = None, trace: Optional[torch.Tensor] = None,
                      flags: Optional[torch.Tensor] = None, orders=(1, 1, 2)) -> None:
    """`block_step` for callers that may not allocate: every buffer, outputs included, is passed
    in, and the scratch memory is the library's built-in array (at most
    `crb_block_step_static_max_rows()` rows; calls on one device must not overlap)."""
    _need_cuda(W, U, Err, losses)
    R = W.shape[0]
    L = lib()
    limit = L.crb_block_step_static_max_rows()
    if R > limit:
        raise CrbError(f"block_step_static serves at most {limit} rows per call, got {R}")
    check(L.crb_block_step_static(ptr(W), R, W.stride(0), ptr(U), U.stride(0), block,
                                  _lib.TECHNIQUES[technique], _lib.orders_code(orders), lam, corr_damp,
                                  _lib.METRICS[metric],
                                  ptr(Err), ptr(losses), ptr(codes), ptr(scales), ptr(trace), ptr(flags),
                                  stream_ptr()), "crb_block_step_static")


def binarize_group(w: torch.Tensor, mask: torch.Tensor, order: int, technique: str,
                   lam: float = 1e-5, corr_damp: float = 0.1) -> torch.Tensor:
    """Binarization.quantize on a [R, 128] block with an arbitrary boolean mask."""
    _need_cuda(w, mask)
    if w.dim() != 2 or w.shape[1] != BLOCK or mask.shape != w.shape:
        raise CrbError(f"binarize_group works on [R, {BLOCK}] blocks")
    wf = w.float().contiguous()
    m8 = mask.to(torch.uint8).contiguous()
    q = torch.empty_like(wf)
    check(lib().crb_binarize_group(ptr(wf), wf.shape[0], wf.stride(0), ptr(m8), m8.stride(0), int(order),
                                   _lib.TECHNIQUES[technique], lam, corr_damp, ptr(q), q.stride(0),
                                   stream_ptr()), "crb_binarize_group")
    return q.to(w.dtype)


def trailing_update(W: torch.Tensor, Err: torch.Tensor, U: torch.Tensor, block: int) -> None:
    """W[:, (block+1)*128:] -= Err @ U[block*128:(block+1)*128, (block+1)*128:]  (bigptq.py:264)."""
    _need_cuda(W, Err, U)
    check(lib().crb_trailing_update(ptr(W), W.shape[0], W.shape[1], W.stride(0), ptr(Err), ptr(U),
                                    U.stride(0), block, stream_ptr()), "crb_trailing_update")


def gemm_f32(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, alpha: float = 1.0, beta: float = 0.0,
             b_is_nk: bool = False, lower_only: bool = False, b_lower: bool = False,
             a_lower: bool = False) -> torch.Tensor:
    """C = alpha * A @ (B.T if b_is_nk else B) + beta * C on the tensor cores (hi/lo TF32 split).

    `b_lower` / `a_lower` promise a lower-triangular B [K, N] / A [M, K] whose zero part is skipped."""
    _need_cuda(A, B, C)
    M, K = A.shape
    N = B.shape[0] if b_is_nk else B.shape[1]
    status = torch.zeros(1, dtype=torch.int32, device=A.device)
    shape = int(lower_only) | 2 * int(b_lower) | 4 * int(a_lower)
    check(lib().crb_gemm_f32(int(b_is_nk), shape, M, N, K, alpha, ptr(A), A.stride(0), ptr(B),
                             B.stride(0), beta, ptr(C), C.stride(0), ptr(status), stream_ptr()), "crb_gemm_f32")
    return C


def quantize_linear(W: torch.Tensor, U: torch.Tensor, technique: str = "crb", lam: float = 1e-5,
                    corr_damp: float = 0.1, metric: str = "hessian", want_codes: bool = False,
                    want_trace: bool = True, orders=(1, 1, 2)) -> dict:
    """The whole block loop of fasterquant on W [R, C] float32 in place, given U."""
    _need_cuda(W, U)
    R, Cc = W.shape
    if W.dtype != torch.float32 or W.stride(1) != 1 or U.dtype != torch.float32:
        raise CrbError("W must be float32 with unit column stride and U float32")
    if U.stride(1) != 1:
        U = U.contiguous()
    if Cc % BLOCK:
        raise CrbError(f"in_features must be a multiple of {BLOCK}")
    L = lib()
    dev = W.device
    ws = _workspace("linear", L.crb_linear_workspace_bytes(R), dev)
    nblk = Cc // BLOCK
    losses = torch.zeros(R, dtype=torch.float32, device=dev)
    ocode = _lib.orders_code(orders)
    if want_codes and ocode != _lib.ORDERS_DEFAULT:
        raise NotImplementedError("codes / scales (the packed form) exist for orders (1, 1, 2) only")
    codes = torch.zeros(R, Cc, dtype=torch.uint8, device=dev) if want_codes else None
    scales = torch.zeros(nblk, R, 8, dtype=torch.float32, device=dev) if want_codes else None
    trace = torch.zeros(nblk, TRACE_DOUBLES, dtype=torch.float64, device=dev) if want_trace else None
    check(L.crb_quantize_linear(ptr(W), R, Cc, W.stride(0), ptr(U), U.stride(0),
                                _lib.TECHNIQUES[technique], ocode, lam, corr_damp, _lib.METRICS[metric],
                                ptr(losses), ptr(codes), ptr(scales), ptr(trace), ptr(ws), ws.numel(),
                                stream_ptr()), "crb_quantize_linear")
    return dict(losses=losses, codes=codes, scales=scales, trace=trace, workspace=ws)


def read_status(workspace: torch.Tensor) -> int:
    rc = lib().crb_read_status(ptr(workspace), stream_ptr())
    if rc < 0:
        check(rc, "crb_read_status")
    return rc


def selftest_wait_limit(device, limit_us: int = 1000) -> int:
    """Makes a bounded wait of the tensor-core GEMM run out on purpose (its producer withholds the
    loads) and returns the status flags the kernel left: CRB_FLAG_WAIT_LIMIT must be among them."""
    scratch = torch.empty(256 * 1024, dtype=torch.uint8, device=device)
    status = torch.zeros(4, dtype=torch.int32, device=device)
    check(lib().crb_selftest_wait_limit(ptr(scratch), scratch.numel(), int(limit_us), ptr(status), stream_ptr()),
          "crb_selftest_wait_limit")
    return int(status[0].item())


def set_factor_lookahead(enable: bool) -> bool:
    """Look-ahead over the rank-1024 updates of the factorisation on or off; returns the old setting."""
    return bool(lib().crb_set_factor_lookahead(int(bool(enable))))


def set_trailing_lookahead(mode: int) -> int:
    """Look-ahead over the grouped trailing updates of `quantize_linear`: 0 off, 1 by shape (default),
    2 whenever there are more than two groups of blocks; returns the old mode.  Same bits either way."""
    return int(lib().crb_set_trailing_lookahead(int(mode)))


def set_fused_selection(enable: bool) -> bool:
    """Quantile selection of the block step as one cooperative kernel (True) or three kernels (False,
    the default); returns the old setting."""
    return bool(lib().crb_set_fused_selection(int(bool(enable))))


def set_dependent_launch(enable: bool) -> bool:
    """Switches programmatic dependent launch of the kernel chains on or off; returns the old setting."""
    return bool(lib().crb_set_dependent_launch(int(bool(enable))))


def launch_count() -> int:
    return int(lib().crb_launch_count())
