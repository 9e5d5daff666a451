"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference <checkout of the reference> [--config1]

The reference is imported as it lies (nothing is copied); two modules it
imports but never uses (`exceptiongroup`, `pyparsing`) are stubbed, and
`torch.cuda.synchronize` is made a no-op on a CUDA-less host.  Captures are
taken by wrapping functions from the outside:
  * bigptq.structural_guassian_distribution -> per block (W_blk, diag U_blk, masks)
  * utils.autosearch.error_computing        -> the 49 + 81 candidate errors per block
All inputs come from seeded CPU generators defined in this file, so the
fixtures can be regenerated bit-for-bit.

Outputs (numpy .npz, float32 unless noted):
  blocks.npz    single-block cases: metric search + the three binarizers
  linear.npz    a 96x256 linear: Hessian from 6 add_batch calls, fasterquant x 3 techniques
  config1.npz   (only with --config1) the 2048x2048 / 262144-token case, compact outputs
  layers.npz    the reference's own layer loop (run.py quant_sequential) on a 2-layer random-init
                OPT-shaped model: per-linear errors, quantized weights, final hidden states
  variants.npz  group outputs of the crb_norefine / crb_symdamp / crb_symdamp_norefine quantizers
                and of a linear run with orders other than (1, 1, 2)
"""
from __future__ import annotations

import argparse
import contextlib
import io
import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(path):
    for name, attr in (("exceptiongroup", "catch"), ("pyparsing", "line")):
        if name not in sys.modules:
            mod = types.ModuleType(name)
            setattr(mod, attr, None)
            sys.modules[name] = mod
    if not torch.cuda.is_available():
        torch.cuda.synchronize = lambda *a, **k: None
    if path not in sys.path:
        sys.path.insert(0, path)
    import bigptq
    import binary
    import utils.autosearch as autosearch
    return bigptq, binary, autosearch


# ---------------------------------------------------------------- seeded inputs
def make_block(R, seed, scale=0.02, hot_cols=3):
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(R, 128, generator=g) * scale
    d = 0.5 + torch.rand(128, generator=g)
    hot = torch.randperm(128, generator=g)[:hot_cols]
    d[hot] *= 0.2                      # small diag(U) -> large metric -> salient columns
    return W, d


def make_linear(R, C, T, seed, outlier_frac=0.01):
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(R, C, generator=g) * 0.02
    X = torch.randn(T, C, generator=g)
    n_out = max(1, int(round(C * outlier_frac)))
    ch = torch.randperm(C, generator=g)[:n_out]
    X[:, ch] *= 20
    return W, X


class Capture:
    """Records per-block inputs, masks and candidate errors of one fasterquant run."""

    def __init__(self, bigptq, autosearch):
        self.bigptq, self.autosearch = bigptq, autosearch
        self.blocks = []
        self._errs = []

    def __enter__(self):
        self._sgd = self.bigptq.structural_guassian_distribution
        self._ec = self.autosearch.error_computing

        def ec(a, b):
            e = self._ec(a, b)
            self._errs.append(float(e))
            return e

        def sgd(tmp, H=None, metric="magnitude", up_lim=30, orders=(1, 1, 2)):
            self._errs = []
            with contextlib.redirect_stdout(io.StringIO()):
                m1, m2, m3 = self._sgd(tmp, H, metric, up_lim, orders=orders)
            self.blocks.append(dict(W=tmp.clone(), d=torch.diag(H).clone(), m1=m1.clone(),
                                    m2=m2.clone(), m3=m3.clone(), errs=list(self._errs)))
            return m1, m2, m3

        self.autosearch.error_computing = ec
        self.bigptq.structural_guassian_distribution = sgd
        return self

    def __exit__(self, *exc):
        self.autosearch.error_computing = self._ec
        self.bigptq.structural_guassian_distribution = self._sgd


def pack(mask):
    return np.packbits(mask.numpy().astype(np.uint8), axis=None)


def gen_blocks(bigptq, binary, autosearch, out):
    cases = [(64, 11, 0.02, 3), (256, 12, 0.02, 5), (200, 13, 0.05, 0), (33, 14, 0.02, 20)]
    data = {"n_cases": np.int64(len(cases))}
    for ci, (R, seed, scale, hot) in enumerate(cases):
        W, d = make_block(R, seed, scale, hot)
        Hblk = torch.diag(d)
        with Capture(bigptq, autosearch) as cap:
            m1, m2, m3 = bigptq.structural_guassian_distribution(W, Hblk, "hessian", 50)
        blk = cap.blocks[0]
        data[f"c{ci}_W"] = W.numpy()
        data[f"c{ci}_d"] = d.numpy()
        data[f"c{ci}_errs"] = np.asarray(blk["errs"], dtype=np.float64)
        for name, m in (("m1", m1), ("m2", m2), ("m3", m3)):
            data[f"c{ci}_{name}"] = pack(m)
        for tech in ("braq", "crbog", "crb"):
            qz = binary.Binarization(W, method=tech, groupsize=128, corr_damp=0.1, lam=1e-5)
            Q = torch.zeros_like(W)
            for g, (m, order) in enumerate(zip((m1, m2, m3), (1, 1, 2))):
                qg = qz.quantize(W, m, order=order)
                data[f"c{ci}_{tech}_q{g}"] = qg.numpy()
                Q += qg * m
            data[f"c{ci}_{tech}_Q"] = Q.numpy()
    np.savez_compressed(out, **data)
    print("wrote", out)


def run_reference_linear(bigptq, binary, autosearch, W, H, nsamples, tech):
    R, C = W.shape
    lin = nn.Linear(C, R, bias=False)
    lin.weight.data = W.clone()
    qz = binary.Binarization(lin.weight, method=tech, groupsize=128, corr_damp=0.1, lam=1e-5)
    g = bigptq.BRAGPTQ(lin, qz, salient_metric="hessian")
    g.H = H.clone()
    g.nsamples = nsamples
    with Capture(bigptq, autosearch) as cap, contextlib.redirect_stdout(io.StringIO()):
        info = g.fasterquant(blocksize=128, percdamp=0.01, partition=3)
    return lin.weight.data.clone(), info["error"], cap.blocks


def gen_linear(bigptq, binary, autosearch, out):
    R, C, T, nseq = 96, 256, 768, 6
    W, X = make_linear(R, C, T, seed=21, outlier_frac=0.02)
    lin = nn.Linear(C, R, bias=False)
    lin.weight.data = W.clone()
    g = bigptq.BRAGPTQ(lin, binary.Binarization(lin.weight, method="braq", groupsize=128), "hessian")
    for j in range(nseq):
        g.add_batch(X[j * (T // nseq):(j + 1) * (T // nseq)].unsqueeze(0), None)
    H = g.H.clone()
    data = dict(W=W.numpy(), X=X.numpy(), H=H.numpy(), nseq=np.int64(nseq))
    for tech in ("braq", "crbog", "crb"):
        Wq, err, blocks = run_reference_linear(bigptq, binary, autosearch, W, H, nseq, tech)
        data[f"{tech}_Wq"] = Wq.numpy()
        data[f"{tech}_error"] = np.float64(err)
        for bi, blk in enumerate(blocks):
            data[f"{tech}_b{bi}_Win"] = blk["W"].numpy()
            data[f"{tech}_b{bi}_d"] = blk["d"].numpy()
            data[f"{tech}_b{bi}_errs"] = np.asarray(blk["errs"], dtype=np.float64)
            for name in ("m1", "m2", "m3"):
                data[f"{tech}_b{bi}_{name}"] = pack(blk[name])
    np.savez_compressed(out, **data)
    print("wrote", out)


def gen_config1(bigptq, binary, autosearch, out, keep_blocks=(0, 9)):
    """The single-linear workload: W 2048x2048 N(0,0.02^2); X 128x2048x2048 N(0,1), 1% channels x20; crb."""
    R = C = 2048
    nseq, seqlen = 128, 2048
    g = torch.Generator().manual_seed(1)
    W = torch.randn(R, C, generator=g) * 0.02
    ch = torch.randperm(C, generator=g)[: C // 100]
    lin = nn.Linear(C, R, bias=False)
    lin.weight.data = W.clone()
    gp = bigptq.BRAGPTQ(lin, binary.Binarization(lin.weight, method="crb", groupsize=128), "hessian")
    G = torch.zeros(C, C, dtype=torch.float64)
    for j in range(nseq):
        gx = torch.Generator().manual_seed(1000 + j)
        x = torch.randn(seqlen, C, generator=gx)
        x[:, ch] *= 20
        gp.add_batch(x.unsqueeze(0), None)
        G += (x.t() @ x).double()
    H = gp.H.clone()
    Wq, err, blocks = run_reference_linear(bigptq, binary, autosearch, W, H, nseq, "crb")
    D = (W - Wq).double()
    out_err = float(torch.sqrt(torch.clamp((D @ G * D).sum(), min=0)))
    data = dict(error=np.float64(err), out_err=np.float64(out_err),
                Wq_rows=Wq[:32].numpy(), channels=ch.numpy(),
                H_diag=torch.diag(H).numpy(), H_row0=H[0].numpy(),
                Wq_colnorm=torch.linalg.norm(Wq.double(), dim=0).numpy())
    for bi, blk in enumerate(blocks):
        data[f"b{bi}_errs"] = np.asarray(blk["errs"], dtype=np.float64)
        data[f"b{bi}_m3cols"] = blk["m3"][0].nonzero().flatten().numpy()
        data[f"b{bi}_frac"] = np.asarray([blk[n].float().mean().item() for n in ("m1", "m2", "m3")])
        if bi in keep_blocks:
            data[f"b{bi}_Win"] = blk["W"].numpy()
            data[f"b{bi}_d"] = blk["d"].numpy()
            data[f"b{bi}_m1"] = pack(blk["m1"])
            data[f"b{bi}_Qout"] = Wq[:, bi * 128:(bi + 1) * 128].numpy()
    np.savez_compressed(out, **data)
    print("wrote", out, "error", err, "out_err", out_err)


# ---------------------------------------------------------------- variants of the same kernels
VARIANTS = ("crb_norefine", "crb_symdamp", "crb_symdamp_norefine")       # binary.py:2885-2890


def run_reference_linear_orders(bigptq, binary, autosearch, W, H, nsamples, tech, orders):
    R, C = W.shape
    lin = nn.Linear(C, R, bias=False)
    lin.weight.data = W.clone()
    qz = binary.Binarization(lin.weight, method=tech, groupsize=128, corr_damp=0.1, lam=1e-5)
    g = bigptq.BRAGPTQ(lin, qz, salient_metric="hessian")
    g.H = H.clone()
    g.nsamples = nsamples
    with Capture(bigptq, autosearch) as cap, contextlib.redirect_stdout(io.StringIO()):
        info = g.fasterquant(blocksize=128, percdamp=0.01, partition=3, orders=orders)
    return lin.weight.data.clone(), info["error"], cap.blocks


def gen_variants(bigptq, binary, autosearch, out):
    """(a) the three flag variants of the v7 binarizer on the masks of two block cases, order 1 and 2,
    plus an element-structured mask with empty rows; (b) whole-linear runs with `orders` other than
    (1, 1, 2) (bigptq.py:246-247 passes orders[i] to the quantizer) and with a flag variant."""
    data = {}
    blocks = np.load(os.path.join(HERE, "blocks.npz"))
    for ci in (0, 3):
        W = torch.from_numpy(blocks[f"c{ci}_W"])
        n = W.numel()
        masks = [torch.from_numpy(np.unpackbits(blocks[f"c{ci}_{k}"])[:n].reshape(W.shape).astype(bool))
                 for k in ("m1", "m2", "m3")]
        ragged = masks[0].clone()
        ragged[::7] = False
        for tech in VARIANTS:
            qz = binary.Binarization(W, method=tech, groupsize=128, corr_damp=0.1, lam=1e-5)
            for g, m in enumerate(masks):
                for order in (1, 2):
                    data[f"c{ci}_{tech}_g{g}_o{order}"] = qz.quantize(W, m, order=order).numpy()
            data[f"c{ci}_{tech}_ragged_o2"] = qz.quantize(W, ragged, order=2).numpy()
    lin = np.load(os.path.join(HERE, "linear.npz"))
    W, H, nseq = torch.from_numpy(lin["W"]), torch.from_numpy(lin["H"]), int(lin["nseq"])
    W_lin, H_lin = W, H
    for tech, orders in (("braq", (2, 2, 2)), ("crb", (2, 2, 2)), ("crb", (2, 1, 1)), ("crb_symdamp_norefine", (1, 1, 2))):
        tag = f"{tech}_{''.join(map(str, orders))}"
        Wq, err, blks = run_reference_linear_orders(bigptq, binary, autosearch, W, H, nseq, tech, orders)
        data[f"{tag}_Wq"] = Wq.numpy()
        data[f"{tag}_error"] = np.float64(err)
        for bi, blk in enumerate(blks):
            data[f"{tag}_b{bi}_errs"] = np.asarray(blk["errs"], dtype=np.float64)
    # (c) the magnitude salience metric (utils/structure.py:11-12): the searches run on the signed
    # weights themselves; single blocks and a whole linear
    for ci in (0, 1, 3):
        W = torch.from_numpy(blocks[f"c{ci}_W"])
        d = torch.from_numpy(blocks[f"c{ci}_d"])
        with Capture(bigptq, autosearch) as cap:
            m1, m2, m3 = bigptq.structural_guassian_distribution(W, torch.diag(d), "magnitude", 50)
        data[f"mag_c{ci}_errs"] = np.asarray(cap.blocks[0]["errs"], dtype=np.float64)
        for name, m in (("m1", m1), ("m2", m2), ("m3", m3)):
            data[f"mag_c{ci}_{name}"] = pack(m)
        qz = binary.Binarization(W, method="crb", groupsize=128, corr_damp=0.1, lam=1e-5)
        Q = torch.zeros_like(W)
        for m, order in zip((m1, m2, m3), (1, 1, 2)):
            Q += qz.quantize(W, m, order=order) * m
        data[f"mag_c{ci}_crb_Q"] = Q.numpy()
    for tech in ("braq", "crb"):
        R, C = W_lin.shape
        layer = nn.Linear(C, R, bias=False)
        layer.weight.data = W_lin.clone()
        qz = binary.Binarization(layer.weight, method=tech, groupsize=128, corr_damp=0.1, lam=1e-5)
        g = bigptq.BRAGPTQ(layer, qz, salient_metric="magnitude")
        g.H = H_lin.clone()
        g.nsamples = nseq
        with Capture(bigptq, autosearch) as cap, contextlib.redirect_stdout(io.StringIO()):
            info = g.fasterquant(blocksize=128, percdamp=0.01, partition=3)
        data[f"mag_{tech}_Wq"] = layer.weight.data.clone().numpy()
        data[f"mag_{tech}_error"] = np.float64(info["error"])
        for bi, blk in enumerate(cap.blocks):
            data[f"mag_{tech}_b{bi}_errs"] = np.asarray(blk["errs"], dtype=np.float64)
            data[f"mag_{tech}_b{bi}_m1"] = pack(blk["m1"])
            data[f"mag_{tech}_b{bi}_m3"] = pack(blk["m3"])
    np.savez_compressed(out, **data)
    print("wrote", out)


# ---------------------------------------------------------------- the reference's layer loop
LAYER_CASES = {
    # name: (synthetic shape, technique, float32 model?, nsamples, seqlen, percdamp)
    "opt_f32_crb": ("opt-tiny", "crb", True, 16, 256, 0.01),
    "opt_f16_braq": ("opt-tiny", "braq", False, 16, 256, 0.01),
}


def layer_case_inputs(case):
    """Model and calibration batches of a LAYER_CASES entry (seeded, CPU generators)."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from crb_b200.synth import build_synthetic_model, synthetic_calibration
    shape, tech, f32, nsamples, seqlen, percdamp = LAYER_CASES[case]
    model = build_synthetic_model(shape, n_layers=2, seed=3, attn="eager")
    if f32:
        model = model.float()
    model.seqlen = seqlen
    loader = synthetic_calibration(model.config.vocab_size, nsamples=nsamples, seqlen=seqlen, seed=1)
    return model, loader


def gen_layers(reference_path, out):
    """run.quant_sequential (run.py:122-387) as the reference runs it, on CPU, with the module
    globals `args` / `groupsize` it reads set from outside.  Per-linear errors are recorded by
    a subclass of BRAGPTQ bound to run.BRAGPTQ, the final hidden states by a forward hook on the
    last decoder layer (the last `nsamples` calls are the re-propagation pass)."""
    import run as refrun
    from argparse import Namespace
    data = {}
    for case, (shape, tech, f32, nsamples, seqlen, percdamp) in LAYER_CASES.items():
        model, loader = layer_case_inputs(case)
        refrun.args = Namespace(model="facebook/" + shape, nsamples=nsamples, low_quant_method=tech, minlayer=-1,
                                maxlayer=1000, quant_only="", invert=False, corr_damp=0.1, lam=1e-5, coupling=0.5,
                                salient_metric="hessian", disable_gptq=False, percdamp=percdamp, blocksize=128,
                                partition=3, global_scale=False)
        refrun.groupsize = 128
        errors, block_errs = [], []
        base = refrun.BRAGPTQ
        import bigptq as ref_bigptq
        import utils.autosearch as ref_autosearch

        class Recorder(base):
            def fasterquant(self, *a, **k):
                with Capture(ref_bigptq, ref_autosearch) as cap:
                    info = base.fasterquant(self, *a, **k)
                errors.append(float(info["error"]))
                block_errs.append([np.asarray(b["errs"], dtype=np.float64) for b in cap.blocks])
                return info

        hidden = []
        last = model.model.decoder.layers[-1]
        handle = last.register_forward_hook(
            lambda mod, inp, outp: hidden.append((outp[0] if isinstance(outp, (tuple, list)) else outp).detach().clone()))
        refrun.BRAGPTQ = Recorder
        try:
            with contextlib.redirect_stdout(io.StringIO()):
                refrun.quant_sequential(model, loader, "cpu")
        finally:
            refrun.BRAGPTQ = base
            handle.remove()
        final = torch.stack([h.reshape(seqlen, -1) for h in hidden[-nsamples:]])
        data[f"{case}_errors"] = np.asarray(errors, dtype=np.float64)
        data[f"{case}_hidden"] = final.float().numpy().astype(np.float32 if f32 else np.float16)
        names = []
        for li, layer in enumerate(model.model.decoder.layers):
            for name, mod in refrun.find_layers(layer).items():
                names.append(f"{li}.{name}")
                data[f"{case}_w_{li}.{name}"] = mod.weight.data.float().numpy().astype(np.float32 if f32 else np.float16)
        data[f"{case}_names"] = np.asarray(names)
        for name, per_block in zip(names, block_errs):       # the 130 candidate errors of every block
            data[f"{case}_errs_{name}"] = np.stack(per_block)
        print(case, "errors", errors)
    np.savez_compressed(out, **data)
    print("wrote", out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of an unmodified checkout of the reference project")
    ap.add_argument("--config1", action="store_true")
    ap.add_argument("--only", default="", help="comma list of fixtures to (re)generate: blocks,linear,layers,variants")
    args = ap.parse_args()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    mods = load_reference(args.reference)
    only = set(filter(None, args.only.split(",")))
    if not only or "blocks" in only:
        gen_blocks(*mods, os.path.join(HERE, "blocks.npz"))
    if not only or "linear" in only:
        gen_linear(*mods, os.path.join(HERE, "linear.npz"))
    if not only or "layers" in only:
        gen_layers(args.reference, os.path.join(HERE, "layers.npz"))
    if not only or "variants" in only:
        gen_variants(*mods, os.path.join(HERE, "variants.npz"))
    if args.config1:
        gen_config1(*mods, os.path.join(HERE, "config1.npz"))


if __name__ == "__main__":
    main()
