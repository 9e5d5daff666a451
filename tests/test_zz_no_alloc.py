"""crb_block_step_static (the block step that brings its own scratch memory) against
crb_block_step on the same inputs, twice in a row.

The entry point exists for callers that are not allowed to allocate device memory when they
need a block step; here every buffer is created up front and the two static calls in the
middle run without any allocation by the library.  This file is collected last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _inputs(R, seed):
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn(R, 256, generator=g) * 0.02).to(DEV)
    d = 0.5 + torch.rand(256, generator=g)
    U = torch.diag(d).to(DEV)
    return W, U


def _static_call(ops, W, U, block, tech):
    from crb_b200 import _lib
    R = W.shape[0]
    out = dict(Err=torch.empty(R, 128, device=DEV), losses=torch.zeros(R, device=DEV),
               codes=torch.zeros(R, 128, dtype=torch.uint8, device=DEV),
               scales=torch.zeros(R, 8, device=DEV),
               trace=torch.zeros(_lib.TRACE_DOUBLES, dtype=torch.float64, device=DEV),
               flags=torch.full((1,), 77, dtype=torch.int32, device=DEV))
    ops.block_step_static(W, U, block, tech, **out)
    return out


@pytest.mark.parametrize("tech", ("crb", "braq"))
def test_static_block_step_matches_workspace_variant_twice(tech):
    from crb_b200 import ops
    # two different problems back to back: the second call must not see leftovers of the first
    cases = [(4096, 1, 5), (300, 0, 6)]
    expected = []
    for R, block, seed in cases:
        W, U = _inputs(R, seed)
        ref = ops.block_step(W, U, block, tech)
        expected.append((W.clone(), {k: ref[k].clone() for k in ("Err", "losses", "codes", "scales", "trace")}))
    torch.cuda.synchronize()
    for (R, block, seed), (W_ref, ref) in zip(cases, expected):
        W, U = _inputs(R, seed)
        got = _static_call(ops, W, U, block, tech)
        torch.cuda.synchronize()
        assert int(got["flags"][0]) == 0
        assert torch.equal(W, W_ref)
        for k in ("Err", "losses", "codes", "scales", "trace"):
            assert torch.equal(got[k], ref[k]), k


def test_static_block_step_refuses_too_many_rows():
    from crb_b200 import _lib, ops
    L = _lib.lib()
    limit = L.crb_block_step_static_max_rows()
    assert limit == 16384
    R = limit + 1
    W, U = _inputs(R, 9)
    W0 = W.clone()
    Err = torch.empty(R, 128, device=DEV)
    losses = torch.zeros(R, device=DEV)
    with pytest.raises(_lib.CrbError):
        ops.block_step_static(W, U, 0, "crb", Err=Err, losses=losses)
    rc = L.crb_block_step_static(ctypes.c_void_p(W.data_ptr()), R, W.stride(0), ctypes.c_void_p(U.data_ptr()),
                                 U.stride(0), 0, 2, 112, 1e-5, 0.1, 0, ctypes.c_void_p(Err.data_ptr()),
                                 ctypes.c_void_p(losses.data_ptr()), None, None, None, None,
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -5
    assert b"built-in scratch" in L.crb_status_string(rc)
    torch.cuda.synchronize()
    assert torch.equal(W, W0)
