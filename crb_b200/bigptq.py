"""`BRAGPTQ`: drop-in for the reference class of the same name (bigptq.py:18-298).

Same constructor, attributes and methods; the arithmetic runs in the sm_100a
kernels of libcrb_b200.so:

    add_batch    -> tcgen05 Hessian accumulation      (bigptq.py:37-54)
    fasterquant  -> device factorisation + block loop  (bigptq.py:56-291)

Only the path of the techniques braq / crbog / crb (and the crb_norefine / crb_symdamp /
crb_symdamp_norefine variants of crb) is implemented: partition=3, orders with one or two
expansions per group, blocksize 128, salience metric hessian or magnitude; anything else raises
NotImplementedError instead of silently taking another route.
"""
from __future__ import annotations

import time

import torch
import torch.nn as nn

from . import ops
from ._lib import BLOCK, TECHNIQUES, orders_code, FLAG_BAD_PIVOT, FLAG_NONFINITE, FLAG_WAIT_LIMIT, CrbError

try:  # transformers.Conv1D weights are stored transposed (bigptq.py:28-29)
    import transformers
    _Conv1D = transformers.Conv1D
except Exception:  # pragma: no cover
    _Conv1D = ()


class BRAGPTQ:
    def __init__(self, layer, braq_quantizer, salient_metric, disable_gptq=False):
        self.layer = layer
        self.dev = self.layer.weight.device
        if self.dev.type != "cuda":
            raise CrbError("BRAGPTQ needs the layer on a CUDA device (no CPU fallback)")
        shape = layer.weight.shape
        if isinstance(layer, nn.Conv2d):
            self.rows, self.columns = shape[0], int(shape[1:].numel())
        elif _Conv1D and isinstance(layer, _Conv1D):
            self.rows, self.columns = shape[1], shape[0]
        else:
            self.rows, self.columns = shape[0], shape[1]
        self.nsamples = 0
        self.braq_quantizer = braq_quantizer
        self.salient_metric = salient_metric
        self.disable_gptq = disable_gptq
        # Unscaled running sum  S = sum_j X_j^T X_j  (upper-triangle tiles); H = 2/nsamples * S.
        self._S = torch.zeros((self.columns, self.columns), device=self.dev, dtype=torch.float32)
        self._H_set = None          # a Hessian assigned from outside (diagnostics inject g.H)
        self._H_keep = None
        self._hess_ws = None        # workspace of the Hessian kernel: its first word holds the status flags
        self.last_flags = 0
        self.last_trace = None
        self.last_timing = {}
        self.verbose = True         # the reference prints time and error per linear (bigptq.py:273-274)
        self.pack = False           # set to keep the packed form of the result in `self.packed`
        self.packed = None

    # ---- the Hessian as the reference exposes it ------------------------------------------
    @property
    def H(self):
        """The scaled Hessian 2/n * sum X^T X as a full symmetric matrix (bigptq.py:50-53)."""
        if self._H_set is not None:
            return self._H_set
        if self._S is None:
            return None
        H = self._S.clone()
        ops.hessian_finalize(H, 2.0 / max(self.nsamples, 1))
        return H

    @H.setter
    def H(self, value):
        if value is None:
            self._H_set, self._S = None, None
            return
        if value.device != self.dev:
            value = value.to(self.dev)
        self._H_set = value.float().contiguous()

    @H.deleter
    def H(self):
        self._H_set, self._S = None, None

    def add_batch(self, inp, out=None, blocksize=1024):
        """Accumulates the layer input into the Hessian (bigptq.py:37-54)."""
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        batch = inp.shape[0]
        if not isinstance(self.layer, nn.Linear) and not (_Conv1D and isinstance(self.layer, _Conv1D)):
            raise NotImplementedError("add_batch: only nn.Linear / Conv1D layers are supported")
        x = inp.reshape(-1, inp.shape[-1])
        if self._H_set is not None:
            # continue from an injected Hessian: S = H * n / 2
            self._S = self._H_set * (self.nsamples / 2.0)
            self._H_set = None
        self._hess_ws = ops.hessian_accumulate(self._S, x)
        self.nsamples += batch

    def _restore_hessian(self, H):
        if self._H_keep is not None:
            H.copy_(self._H_keep)
        else:
            H.copy_(self._S)
            ops.hessian_finalize(H, 2.0 / max(self.nsamples, 1))

    def fasterquant(self, blocksize=128, percdamp=0.01, partition=3, orders=(1, 1, 2),
                    global_scale=False):
        """Binarizes the layer's weight in place and returns {"error": float} (bigptq.py:56-291)."""
        state = self.fasterquant_begin(blocksize, percdamp, partition, orders, global_scale)
        return self.fasterquant_end(state)

    # The three steps below let a caller overlap several linears, each on its own stream:
    #   begin  - enqueues the factorisation (attempt 0); no host synchronisation
    #   blocks - reads the factorisation status (waits for that stream only), handles the rare
    #            damping retry and enqueues the whole block loop; returns without waiting for it
    #   commit - (optional) enqueues the write-back of the binarized weight INTO the layer's
    #            existing weight storage on the linear's stream and returns the event that marks
    #            it; a caller can then enqueue work that reads the weight (behind that event)
    #            before anything has waited for the block loop on the host
    #   end    - waits for the block loop, reads the error and writes the weight back
    # A caller with several linears runs every `begin`, then every `blocks`, then every `end`.
    # `factor_from` names the state of another linear with the very same Hessian (q/k/v of one
    # attention block): its factor U is read instead of computing an identical one.
    def fasterquant_begin(self, blocksize=128, percdamp=0.01, partition=3, orders=(1, 1, 2),
                          global_scale=False, factor_from=None):
        technique = getattr(self.braq_quantizer, "method", None)
        if technique not in TECHNIQUES:
            raise NotImplementedError(f"technique {technique!r}: implemented are {sorted(TECHNIQUES)}")
        if partition != 3:
            raise NotImplementedError("only partition=3 is implemented")
        orders_code(orders)                                         # raises for anything but 1 / 2 per group
        if blocksize != BLOCK:
            raise NotImplementedError(f"only blocksize {BLOCK} is implemented")
        if self.disable_gptq:
            raise NotImplementedError("disable_gptq (RTN) is not implemented")
        if self.salient_metric not in ("hessian", "magnitude"):          # utils/structure.py:9-14
            raise NotImplementedError(f"salient_metric {self.salient_metric!r}: hessian and magnitude are implemented")
        assert self.braq_quantizer.groupsize % blocksize == 0       # bigptq.py:147
        if self.columns % BLOCK:
            raise NotImplementedError(f"in_features must be a multiple of {BLOCK}")

        st = {"tick": time.time(), "percdamp": percdamp, "technique": technique,
              "stream": torch.cuda.current_stream(self.dev), "leader": factor_from, "orders": tuple(orders),
              "ev": [torch.cuda.Event(enable_timing=True) for _ in range(3)]}
        W = self.layer.weight.data.clone()
        if isinstance(self.layer, nn.Conv2d):
            W = W.flatten(1)
        if _Conv1D and isinstance(self.layer, _Conv1D):
            W = W.t()
        st["W"] = W.float().contiguous()
        st["ev"][0].record()
        if factor_from is not None:
            if factor_from["percdamp"] != percdamp or factor_from["H"].shape[0] != self.columns:
                raise CrbError("factor_from: the other linear does not have the same Hessian and damping")
            # dead input channels zero the weight column (bigptq.py:103-105); the factor is the leader's
            st["W"].masked_fill_((factor_from["diag0"] == 0).unsqueeze(0), 0.0)
            self._H_set, self._S, self._H_keep = None, None, None
            return st
        # the reference consumes H here (bigptq.py:101-102)
        if self._H_set is not None:
            H, self._H_keep = self._H_set.clone(), self._H_set
        else:
            H, self._H_keep = self._S.clone(), None
            ops.hessian_finalize(H, 2.0 / max(self.nsamples, 1))
        st["H"] = H
        st["diag0"] = torch.diagonal(H).clone()
        # status[0]: flags of the factorisation; status[1]: flags the Hessian kernel left (read together
        # with the factorisation's, so checking them costs no extra synchronisation)
        st["status"] = torch.zeros(4, dtype=torch.int32, device=self.dev)
        if self._hess_ws is not None:
            st["status"][1:2].copy_(self._hess_ws[:4].view(torch.int32))
        ops.factor_enqueue(H, st["W"], percdamp, 0, st["status"])
        return st

    def fasterquant_blocks(self, st):
        if "out" in st:
            return st
        with torch.cuda.stream(st["stream"]):
            W = st["W"]
            if st["leader"] is not None:
                lead = st["leader"]
                if "factor_done" not in lead:
                    raise CrbError("factor_from: run fasterquant_blocks of the other linear first")
                st["stream"].wait_event(lead["factor_done"])
                U = lead["H"]
            else:
                H = st["H"]
                attempt = 0
                while True:
                    f_factor, f_hessian = st["status"][:2].tolist()
                    if (f_factor | f_hessian) & FLAG_WAIT_LIMIT:
                        raise CrbError("a bounded wait inside the %s kernels ran out (CRB_FLAG_WAIT_LIMIT): "
                                       "the result would be incomplete"
                                       % ("Hessian" if f_hessian & FLAG_WAIT_LIMIT else "factorisation"))
                    if not (f_factor & FLAG_BAD_PIVOT):
                        break
                    attempt += 1                                          # bigptq.py:115-123: extras 0 .. 9
                    if attempt >= 10:
                        ops.diagonal_fallback(H, st["diag0"], st["percdamp"])   # bigptq.py:124-126
                        break
                    self._restore_hessian(H)
                    st["status"][0] = 0
                    ops.factor_enqueue(H, W, st["percdamp"], attempt, st["status"])
                U = H
                st["factor_done"] = torch.cuda.Event()
                st["factor_done"].record()
                self._H_set, self._S, self._H_keep = None, None, None
            st["ev"][1].record()
            lam = float(getattr(self.braq_quantizer, "lam", 1e-5))
            corr_damp = float(getattr(self.braq_quantizer, "corr_damp", 0.1))
            st["out"] = ops.quantize_linear(W, U, st["technique"], lam, corr_damp, self.salient_metric,
                                            want_codes=bool(self.pack), want_trace=True, orders=st["orders"])
            st["ev"][2].record()
        return st

    def fasterquant_commit(self, st):
        """Enqueues `layer.weight.data.copy_(binarized W)` behind the block loop; returns its event.

        The status flags of the block loop are only read by `fasterquant_end`: if that raises, the
        layer's weight has already been overwritten with the incomplete result."""
        self.fasterquant_blocks(st)
        if "committed" not in st:
            with torch.cuda.stream(st["stream"]):
                W = st["W"]
                if _Conv1D and isinstance(self.layer, _Conv1D):
                    W = W.t()
                self.layer.weight.data.copy_(W.reshape(self.layer.weight.shape))
                st["committed"] = torch.cuda.Event()
                st["committed"].record()
        return st["committed"]

    def fasterquant_end(self, st):
        self.fasterquant_blocks(st)
        with torch.cuda.stream(st["stream"]):
            out, W = st["out"], st["W"]
            error = torch.sum(out["losses"]).item()                     # synchronises this stream
            flags = ops.read_status(out["workspace"])
            if flags & ~FLAG_NONFINITE:
                raise CrbError(f"block loop reported device status flags {flags:#x}")
            self.last_trace = out["trace"]
            self.last_flags = flags
            ev = st["ev"]
            self.last_timing = {"factor_ms": ev[0].elapsed_time(ev[1]), "blocks_ms": ev[1].elapsed_time(ev[2])}
            if self.pack:
                from .packed import pack_linear
                self.packed = pack_linear(out["codes"], out["scales"], W, st["technique"])
            if self.verbose:
                print("time %.2f" % (time.time() - st["tick"]))
                print("error", error)
            if "committed" not in st:                                   # bigptq.py:278-280
                if _Conv1D and isinstance(self.layer, _Conv1D):
                    W = W.t()
                self.layer.weight.data = W.reshape(self.layer.weight.shape).to(self.layer.weight.data.dtype)
        return {"error": error}

    def free(self):
        """Drops the Hessian (bigptq.py:293-298).  The cached allocator is left alone."""
        self._H_set, self._S = None, None
