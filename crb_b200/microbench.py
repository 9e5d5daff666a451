"""Times one entry point of the library on synthetic inputs of a chosen size.

    python -m crb_b200.microbench hessian  --T 16384 --C 4096 [--dtype float16]
    python -m crb_b200.microbench factor   --C 4096
    python -m crb_b200.microbench block    --R 4096 --technique crb
    python -m crb_b200.microbench trailing --R 4096 --C 4096
    python -m crb_b200.microbench linear   --R 4096 --C 4096 --technique crb
    python -m crb_b200.microbench dequant  --R 4096 --C 4096 --technique crb
    python -m crb_b200.microbench gemm     --R 4096 --C 4096 --T 1024     (C[R,C] -= A[R,T] B[C,T]^T)

Each run does `--warmup` untimed and `--iters` timed calls bracketed by CUDA events on the
launching stream and prints one JSON line with the time per call and the algorithmic
throughput (bytes or flop per call as documented per subcommand).  Small sizes make these
commands suitable for profiler captures.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops


def _time(fn, warmup, iters, setup=None):
    for _ in range(warmup):
        if setup:
            setup()
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if setup:
            setup()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def _synthetic_factor(C, dev, seed=0):
    """An upper factor with the structure the block loop sees: positive diagonal, small off-diagonal."""
    g = torch.Generator(device=dev).manual_seed(seed)
    U = torch.randn(C, C, generator=g, device=dev) * (0.02 / C ** 0.5)
    U = torch.triu(U, 1)
    U += torch.diag(0.5 + torch.rand(C, generator=g, device=dev))
    return U.contiguous()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["hessian", "factor", "block", "trailing", "linear", "dequant", "gemm"])
    ap.add_argument("--R", type=int, default=4096)
    ap.add_argument("--C", type=int, default=4096)
    ap.add_argument("--T", type=int, default=16384)
    ap.add_argument("--dtype", default="float16", choices=["float16", "bfloat16", "float32"])
    ap.add_argument("--technique", default="crb", choices=["crb", "crbog", "braq"])
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--no_dependent_launch", action="store_true",
                    help="plain stream-ordered launches instead of programmatic dependent launch")
    ap.add_argument("--fused_selection", action="store_true",
                    help="quantile selection of the block step as one cooperative kernel")
    ap.add_argument("--lookahead", type=int, default=None, choices=(0, 1, 2),
                    help="trailing-update look-ahead of the linear loop: 0 off, 1 by shape (default), 2 always")
    ap.add_argument("--no_factor_lookahead", action="store_true",
                    help="factorisation: the whole rank-1024 update on the caller's stream")
    a = ap.parse_args(argv)
    if a.no_factor_lookahead:
        ops.set_factor_lookahead(False)
    if a.lookahead is not None:
        ops.set_trailing_lookahead(a.lookahead)
    if a.fused_selection:
        ops.set_fused_selection(True)
    if a.no_dependent_launch:
        ops.set_dependent_launch(False)
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(1)
    out = {"what": a.what, "R": a.R, "C": a.C, "T": a.T, "dependent_launch": not a.no_dependent_launch,
           "fused_selection": a.fused_selection, "lookahead": a.lookahead}
    launches0 = ops.launch_count()

    if a.what == "hessian":
        X = torch.randn(a.T, a.C, generator=g, device=dev).to(getattr(torch, a.dtype))
        S = torch.zeros(a.C, a.C, device=dev)
        ms = _time(lambda: ops.hessian_accumulate(S, X), a.warmup, a.iters)
        nt = (a.C + 255) // 256
        tiles = nt * (nt + 1) // 2
        passes = 3 if a.dtype == "float32" else 1
        issued = tiles * 256 * 256 * 2.0 * a.T * passes
        out.update(ms=ms, dtype=a.dtype, tflops_issued=issued / ms / 1e9,
                   tflops_full_product=2.0 * a.T * a.C * a.C / ms / 1e9,
                   note="flop issued on upper-triangle 256x256 tiles; full product = 2*T*C^2")
    elif a.what == "factor":
        X = torch.randn(2 * a.C, a.C, generator=g, device=dev)
        H0 = (X.t() @ X) / a.C
        H = H0.clone()
        ms = _time(lambda: ops.hinv_upper_factor(H, None, 0.01, restore=lambda h: h.copy_(H0)), a.warmup, a.iters,
                   setup=lambda: H.copy_(H0))
        out.update(ms=ms, gflops=(2.0 / 3.0) * a.C ** 3 / ms / 1e6,
                   note="2*C^3/3 flop (one factorisation + one triangular inverse), includes the status read")
    elif a.what == "block":
        W = torch.randn(a.R, 256, generator=g, device=dev) * 0.02
        U = _synthetic_factor(256, dev)
        W0 = W.clone()
        ms = _time(lambda: ops.block_step(W, U, 0, a.technique, want_codes=False), a.warmup, a.iters,
                   setup=lambda: W.copy_(W0))
        bytes_alg = 1536.0 * a.R + 65536
        out.update(ms=ms, gbs=bytes_alg / ms / 1e6, technique=a.technique,
                   note="algorithmic bytes per block = 1536*R + 64 KiB (read W block, write Q and Err, U block, losses)")
    elif a.what == "trailing":
        W = torch.randn(a.R, a.C, generator=g, device=dev)
        Err = torch.randn(a.R, 128, generator=g, device=dev)
        U = _synthetic_factor(a.C, dev)
        ms = _time(lambda: ops.trailing_update(W, Err, U, 0), a.warmup, a.iters)
        n = a.C - 128
        out.update(ms=ms, tflops=2.0 * a.R * 128 * n / ms / 1e9, gbs=(8.0 * a.R * n + 4 * a.R * 128 + 4 * 128 * n) / ms / 1e6,
                   note="first block of the loop: flop 2*R*128*(C-128); bytes read+write W[:,128:] + Err + U rows")
    elif a.what == "gemm":
        # the shape of the factorisation's rank-K updates: both operands row-major with K contiguous
        A = torch.randn(a.R, a.T, generator=g, device=dev)
        B = torch.randn(a.C, a.T, generator=g, device=dev)
        Cm = torch.zeros(a.R, a.C, device=dev)
        ms = _time(lambda: ops.gemm_f32(A, B, Cm, alpha=-1.0, beta=1.0, b_is_nk=True), a.warmup, a.iters)
        out.update(ms=ms, tflops_fp32_equivalent=2.0 * a.R * a.C * a.T / ms / 1e9,
                   tflops_tf32_issued=6.0 * a.R * a.C * a.T / ms / 1e9,
                   note="M=R, N=C, K=T; three TF32 MMAs per float32 product term")
    elif a.what == "dequant":
        from . import packed
        W = torch.randn(a.R, a.C, generator=g, device=dev) * 0.02
        U = _synthetic_factor(a.C, dev)
        o = ops.quantize_linear(W, U, a.technique, want_codes=True, want_trace=False)
        p = packed.pack_linear(o["codes"], o["scales"], W, a.technique)
        Wout = torch.empty_like(W)
        ms = _time(lambda: packed.dequantize(p, Wout), a.warmup, a.iters)
        assert torch.equal(Wout, W)
        out.update(ms=ms, technique=a.technique, bits_per_weight=p.bits_per_weight(),
                   gbs=(4.0 * a.R * a.C + p.nbytes()) / ms / 1e6,
                   note="bytes: float32 weights written + packed planes and scales read")
    else:
        W = torch.randn(a.R, a.C, generator=g, device=dev) * 0.02
        U = _synthetic_factor(a.C, dev)
        W0 = W.clone()
        ms = _time(lambda: ops.quantize_linear(W, U, a.technique, want_trace=False), a.warmup, a.iters,
                   setup=lambda: W.copy_(W0))
        nblk = a.C // 128
        out.update(ms=ms, ms_per_block=ms / nblk, technique=a.technique,
                   block_gbs=(1536.0 * a.R + 65536) * nblk / ms / 1e6,
                   note="whole block loop incl. trailing updates; block_gbs counts the block-step bytes only")
    out["launches_per_call"] = (ops.launch_count() - launches0) / (a.warmup + a.iters)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
