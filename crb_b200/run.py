"""Layer-by-layer calibration and binarization: the caller side of the hot path.

Mirrors the reference's `run.py` for the techniques braq / crbog / crb:

    python -m crb_b200.run MODEL DATASET {crb,crbog,braq} --blocksize 128 --salient_metric hessian

* `quant_sequential(model, dataloader, dev, args)` follows run.py:122-387: capture the
  inputs of layer 0, then per decoder layer hook every linear, run the calibration
  sequences, quantize each linear with `BRAGPTQ.fasterquant`, re-propagate with the
  quantized weights and hand the outputs to the next layer.
* Differences that do not change results: the sequences are pushed through a layer in
  batches (`--forward_batch`) instead of one by one; linears that receive the same input
  tensor (q/k/v, gate/up) share one Hessian accumulator instead of computing it three times;
  under torch.distributed (one process per GPU) every rank runs its share of the sequences,
  the partial Hessians are summed with one all-reduce, each linear is quantized by one owner
  rank and the quantized weights are broadcast.

Checkpoints and datasets are not reachable offline: model names resolve to seeded
random-init models of the same shape (`crb_b200.synth`) unless a local checkpoint directory
is given, and the calibration set is uniform random token ids unless a cached loader file
of the reference's format exists under $BILLM_DOWNLOADS_DIR.
"""
from __future__ import annotations

import argparse
import os
import time
from types import SimpleNamespace
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from . import parallel
from .bigptq import BRAGPTQ
from .binary import Binarization
from .synth import build_synthetic_model, resolve_shape, synthetic_calibration

TECHNIQUES = ("braq", "crbog", "crb", "crb_norefine", "crb_symdamp", "crb_symdamp_norefine")


def find_layers(module, layers=(nn.Conv2d, nn.Linear), name=""):
    """All quantizable sub-modules of `module` by dotted name (modelutils.py:8-16)."""
    if type(module) in layers:
        return {name: module}
    res = {}
    for child_name, child in module.named_children():
        res.update(find_layers(child, layers, name + "." + child_name if name else child_name))
    return res


def default_args(**overrides) -> SimpleNamespace:
    """The reference's argparse defaults for this path (run.py:764-944)."""
    a = SimpleNamespace(model="synthetic:opt-tiny", dataset="wikitext2", low_quant_method="crb",
                        nsamples=128, seed=0, percdamp=0.01, blocksize=128, salient_metric="hessian",
                        partition=3, global_scale=False, disable_gptq=False, minlayer=-1, maxlayer=1000,
                        quant_only="", invert=False, corr_damp=0.1, lam=1e-5, coupling=0.5,
                        device="cuda:0", seqlen=None, forward_batch=8, act_offload_gib=64.0, act_stage_gib=16.0,
                        reprop_lanes=16, reprop_overlap=None, shard_skew=True, replicate_result=False, verbose=True, save_packed=None)
    for k, v in overrides.items():
        setattr(a, k, v)
    return a


def get_model(model_name: str, fill_device: Optional[str] = None, n_layers: Optional[int] = None,
              attn: str = "sdpa"):
    """A local checkpoint directory is loaded as is; any other name gives the seeded random-init
    model of that shape (run.py:19-71 downloads instead, which is impossible offline)."""
    if os.path.isdir(model_name):
        from transformers import AutoModelForCausalLM
        model = AutoModelForCausalLM.from_pretrained(model_name, dtype="auto", local_files_only=True,
                                                     attn_implementation=attn)
        model.seqlen = min(model.config.max_position_embeddings, 2048)
        model.eval()
        return model
    if resolve_shape(model_name) is None:
        raise ValueError(f"{model_name!r} is neither a local checkpoint nor a known synthetic shape")
    return build_synthetic_model(model_name, n_layers=n_layers, fill_device=fill_device, attn=attn)


def get_loaders(name: str, nsamples: int, seed: int, seqlen: int, model, model_name: str = ""):
    """The reference's cached calibration loader if one exists locally, else uniform token ids."""
    downloads = os.environ.get("BILLM_DOWNLOADS_DIR", "./downloads")
    cache = f"{downloads}/DOWNLOAD_{name}_{nsamples}_{seed}_{seqlen}_{model_name}.pt"
    if os.path.exists(cache):
        return torch.load(cache)
    return synthetic_calibration(model.config.vocab_size, nsamples, seqlen, seed), None


# ---------------------------------------------------------------------------------------------
def _decoder_parts(model):
    """(layers, modules that must sit on the device while layer-0 inputs are captured)."""
    inner = model.model
    if hasattr(inner, "decoder"):                                   # OPT (run.py:132-147)
        dec = inner.decoder
        pre = [dec.embed_tokens, dec.embed_positions]
        for opt_name in ("project_in", "project_out"):
            if getattr(dec, opt_name, None) is not None:
                pre.append(getattr(dec, opt_name))
        return dec.layers, pre
    pre = [inner.embed_tokens, inner.norm]                          # Llama family (run.py:148-153)
    if hasattr(inner, "rotary_emb"):
        pre.append(inner.rotary_emb)
    return inner.layers, pre


_STREAMS: Dict[object, list] = {}


def _copy_streams(dev):
    """(activations host->device, device->host, weight broadcast, weights host->device) side streams
    of a device, created once.  Layer weights have a stream of their own on the way in: the next
    layer's 0.4 GB are requested when a layer starts, and on the activations' stream they would sit
    in front of that layer's first calibration batch."""
    key = ("copy", torch.device(dev).index or 0)
    if key not in _STREAMS:
        _STREAMS[key] = [torch.cuda.Stream(device=dev) for _ in range(4)]
    return _STREAMS[key]


def _lane_streams(dev, n):
    """Streams of the re-propagation pass (lowest priority), created once per device."""
    lanes = _STREAMS.setdefault(("lanes", torch.device(dev).index or 0), [])
    while len(lanes) < n:
        lanes.append(torch.cuda.Stream(device=dev, priority=0))
    return lanes[:n]


class _Resident:
    """Moves a module's parameters to the device and back without losing the pinned host copies.

    `prefetch()` starts the host->device copies on a side stream (so that they overlap the work of
    the layer before); `__enter__` then only makes the current stream wait for them.
    `__exit__(defer=True)` starts the copies back on a side stream and returns at once; `finish()`
    waits for them.  The plain `with` form does both synchronously.

    With several ranks every process holds the same model in host memory, and N copies of a layer
    over PCIe cost the host N times the traffic.  `loader` names the one rank that reads its host
    copy; the others receive the layer over NVLink (a broadcast on `parallel.weights_group()`).
    `keeper` names the one rank whose host copy receives the (quantized) parameters at the end; on
    the other ranks the module simply points at its untouched host tensors again.  Both default to
    None: every rank copies in and out for itself.
    """

    def __init__(self, module: nn.Module, dev, loader: Optional[int] = None, keeper: Optional[int] = None):
        self.module, self.dev, self.host = module, dev, {}
        self._ready = None
        self._back = None
        self._keep = []
        rank, ws = parallel.world()
        shared = ws > 1 and torch.device(dev).type == "cuda"
        self.loader = loader if shared else None
        self.keeper = keeper if shared else None
        self.rank = rank

    def _tensors(self):
        return list(self.module.named_parameters()) + list(self.module.named_buffers())

    def _bring_in(self):
        """Host -> device for every parameter still on the host, on the current stream."""
        group = parallel.weights_group() if self.loader is not None else None
        for name, p in self._tensors():
            if p.device.type == "cuda":
                continue
            self.host[name] = p.data
            shared = self.loader is not None and p.data.is_contiguous()     # same on every rank
            if not shared or self.rank == self.loader:
                p.data = p.data.to(self.dev, non_blocking=True)
            else:
                p.data = torch.empty(p.data.shape, dtype=p.data.dtype, device=self.dev)
            if shared:
                parallel.broadcast_(p.data, self.loader, group)

    def prefetch(self):
        if torch.device(self.dev).type != "cuda" or self._ready is not None:
            return self
        h2d = _copy_streams(self.dev)[3]
        with torch.cuda.stream(h2d):
            self._bring_in()
            self._ready = torch.cuda.Event()
            self._ready.record(h2d)
        return self

    def __enter__(self):
        if torch.device(self.dev).type != "cuda":
            return self.module
        if self._ready is not None:
            torch.cuda.current_stream(self.dev).wait_event(self._ready)
            return self.module
        self._bring_in()
        return self.module

    def __exit__(self, *exc, defer=False):
        if not self.host:
            return
        tensors = dict(self._tensors())
        main = torch.cuda.current_stream(self.dev)
        stream = _copy_streams(self.dev)[1] if defer else main
        if defer:
            stream.wait_stream(main)
        keep = self.keeper is None or self.rank == self.keeper
        with torch.cuda.stream(stream):
            for name, host in self.host.items():
                p = tensors[name]
                if keep:
                    host.copy_(p.data, non_blocking=True)
                self._keep.append(p.data)            # the device copy lives until the copy back is done
                p.data = host
            self._back = torch.cuda.Event()
            self._back.record(stream)
        self.host.clear()
        if not defer:
            self.finish()

    def finish(self):
        if self._back is not None:
            self._back.synchronize()
            self._back = None
        self._keep.clear()
        self._ready = None


class _Feeder:
    """Hands the layer its calibration batches.  Device-resident activations are sliced; activations
    kept in pinned host memory (the reference offloads them above 8 GiB, run.py:166-172) are
    copied one batch ahead on a side stream, so that the copy of batch j + 1 overlaps the layer
    forward of batch j.  When this rank's shard fits `keep_gib`, the copies land in a device buffer
    that holds the whole shard and the re-propagation pass (`second_pass`) reads that buffer
    instead of copying everything in again; larger shards go through two batch-sized buffers."""

    _buffers: Dict[tuple, list] = {}        # per shape: [device buffers, events "slot no longer read"]

    def __init__(self, inps: torch.Tensor, fb: int, dev, keep_gib: float = 0.0, _resident=None):
        self.inps, self.fb, self.dev = inps, fb, torch.device(dev)
        self.n = inps.shape[0]
        self.staged = inps.device.type == "cpu" and self.dev.type == "cuda"
        self.whole = False
        if _resident is not None:           # second pass over a shard that pass 1 left on the device
            self.staged, self.whole = False, True
            self.buf, self.free = _resident
            self.main = torch.cuda.current_stream(self.dev)
            return
        if not self.staged:
            return
        nb = len(self)
        nbytes = inps.numel() * inps.element_size()
        self.whole = nbytes <= keep_gib * (1024 ** 3)
        slots = nb if self.whole else 2
        rows = self.n if self.whole else 2 * fb
        key = (self.dev.index or 0, fb, rows, tuple(inps.shape[1:]), inps.dtype)
        if key not in _Feeder._buffers:
            buf = torch.empty((rows,) + tuple(inps.shape[1:]), dtype=inps.dtype, device=self.dev)
            first = torch.cuda.Event()
            first.record(torch.cuda.current_stream(self.dev))       # the buffers exist from here on
            _Feeder._buffers[key] = [buf, [first] * slots]
        self.buf, self.free = _Feeder._buffers[key]    # `free` is shared: the next feeder continues it
        self.h2d = _copy_streams(self.dev)[0]
        self.main = torch.cuda.current_stream(self.dev)
        self.ready = [None] * slots
        self._stage(0)

    def _slot(self, idx):
        return idx if self.whole else idx & 1

    def _rows(self, idx):
        j = idx * self.fb
        m = min(self.fb, self.n - j)
        first = j if self.whole else (idx & 1) * self.fb
        return j, m, self.buf[first:first + m]

    def _stage(self, idx):
        j, m, dst = self._rows(idx)
        if j >= self.n:
            return
        slot = self._slot(idx)
        self.h2d.wait_event(self.free[slot])           # the slot's previous batch has been consumed
        written = _WRITTEN.get((self.inps.data_ptr(), j))
        if written is not None:
            self.h2d.wait_event(written)               # these rows were an output on its way to the host
        with torch.cuda.stream(self.h2d):
            dst.copy_(self.inps[j:j + m], non_blocking=True)
            self.ready[slot] = torch.cuda.Event()
            self.ready[slot].record(self.h2d)

    def __len__(self):
        return (self.n + self.fb - 1) // self.fb

    def batch(self, idx, stream=None):
        """Batch `idx` on the device; call in increasing order, `done(idx)` after its last use.
        `stream` is the stream that reads the batch (default: the one current at construction)."""
        if not self.staged and not self.whole:
            j = idx * self.fb
            return self.inps[j:j + min(self.fb, self.n - j)].to(self.dev, non_blocking=True)
        view = self._rows(idx)[2]
        if self.staged:
            self._stage(idx + 1)
            (stream or self.main).wait_event(self.ready[self._slot(idx)])
        return view

    def done(self, idx, stream=None):
        if self.staged or self.whole:
            ev = torch.cuda.Event()
            ev.record(stream or self.main)
            self.free[self._slot(idx)] = ev

    def second_pass(self):
        """The feeder of the re-propagation pass over the same rows."""
        if self.staged and self.whole:
            return _Feeder(self.inps, self.fb, self.dev, _resident=(self.buf, self.free))
        return _Feeder(self.inps, self.fb, self.dev)


# (host buffer address, first row) -> event "these rows have arrived in host memory"; a feeder that
# later reads the rows back waits for exactly that copy instead of for the whole copy stream
_WRITTEN: Dict[tuple, object] = {}


def _store_outputs(outs: torch.Tensor, j: int, y: torch.Tensor, dev):
    """outs[j : j + len(y)] = y; towards pinned host memory the copy runs on a side stream."""
    if outs.device.type == "cpu" and torch.device(dev).type == "cuda":
        d2h = _copy_streams(dev)[1]
        d2h.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(d2h):
            outs[j:j + y.shape[0]].copy_(y, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(d2h)
        _WRITTEN[(outs.data_ptr(), j)] = ev
        y.record_stream(d2h)
    else:
        outs[j:j + y.shape[0]].copy_(y, non_blocking=True)


class _Catcher(nn.Module):
    """Stands in for layer 0, records its input and keyword arguments, then aborts the forward
    (run.py:175-201)."""

    def __init__(self, module, sink):
        super().__init__()
        self.module, self.sink = module, sink

    def __getattr__(self, name):
        if name in ("module", "sink"):
            return super().__getattr__(name)
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)

    def forward(self, inp, **kwargs):
        self.sink["inps"].append(inp)
        self.sink["kwargs"] = kwargs
        raise ValueError


def _replay_kwargs(kwargs: dict, batch: int) -> dict:
    """Layer keyword arguments captured with batch 1, widened to `batch` sequences."""
    out = {}
    for k, v in kwargs.items():
        if k in ("past_key_values", "past_key_value", "use_cache"):
            continue
        if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == 1 and batch > 1:
            v = v.expand(batch, *v.shape[1:])
        elif isinstance(v, tuple) and all(torch.is_tensor(t) for t in v):
            v = tuple(t.expand(batch, *t.shape[1:]) if t.dim() >= 1 and t.shape[0] == 1 and batch > 1 else t
                      for t in v)
        out[k] = v
    out["use_cache"] = False
    return out


def _stream_pool(dev, n):
    """Side streams per device, created once: scratch buffers are cached per stream.

    Slot 0 serves the most expensive linear of a layer, whose serial chain of small kernels decides
    when the layer is done: it gets the highest priority, so that its kernels are placed first
    whenever an SM frees up among the wide kernels of the other linears; the other linears come
    next, ahead of the forwards of the re-propagation pass that run beside them."""
    pool = _STREAMS.setdefault(torch.device(dev).index or 0, [])
    while len(pool) < n:
        pool.append(torch.cuda.Stream(device=dev, priority=-2 if len(pool) == 0 else -1))
    return pool


class _TailReached(Exception):
    """Raised by the hook of a layer's last linear to end a calibration forward early."""


def _layer_out(res):
    return res[0] if isinstance(res, (tuple, list)) else res


class _Timer:
    """Per-phase device time (CUDA events on the current stream; host clock without CUDA)."""

    def __init__(self):
        self.ms: Dict[str, float] = {}
        self._pending = []
        self.cuda = torch.cuda.is_available()

    def span(self, name):
        timer = self

        class _Span:
            def __enter__(self):
                if timer.cuda:
                    self.a = torch.cuda.Event(enable_timing=True)
                    self.b = torch.cuda.Event(enable_timing=True)
                    self.a.record()
                else:
                    self.t0 = time.perf_counter()

            def __exit__(self, *exc):
                if timer.cuda:
                    self.b.record()
                    timer._pending.append((name, self.a, self.b))
                else:
                    timer.ms[name] = timer.ms.get(name, 0.0) + (time.perf_counter() - self.t0) * 1e3

        return _Span()

    def collect(self):
        if self.cuda:
            torch.cuda.synchronize()
        for name, a, b in self._pending:
            self.ms[name] = self.ms.get(name, 0.0) + a.elapsed_time(b)
        self._pending.clear()
        return self.ms


@torch.no_grad()
def quantize_layer(layer: nn.Module, index: int, inps: torch.Tensor, outs: torch.Tensor,
                   layer_kwargs: dict, args, dev, timer: Optional[_Timer] = None,
                   traces: Optional[dict] = None) -> Dict[str, float]:
    """One iteration of the layer loop (run.py:236-385) for a layer already on `dev`.

    `inps` / `outs` hold this rank's sequences [n_local, seqlen, hidden] (device or pinned host).
    Returns the per-linear `error` values (only the owner rank's are non-zero before the sum).
    `traces` (optional dict) receives the per-block search traces of the linears this rank owns.
    """
    timer = timer or _Timer()
    rank, ws = parallel.world()
    subset = find_layers(layer)
    gptq: Dict[str, BRAGPTQ] = {}
    for name in subset:
        if (not (args.minlayer <= index < args.maxlayer and args.quant_only in name)) == (not args.invert):
            continue
        quantizer = Binarization(subset[name].weight, method=args.low_quant_method, groupsize=args.blocksize,
                                 corr_damp=args.corr_damp, lam=args.lam, coupling=args.coupling)
        gptq[name] = BRAGPTQ(subset[name], quantizer, salient_metric=args.salient_metric,
                             disable_gptq=args.disable_gptq)
        gptq[name].verbose = bool(args.verbose)
        gptq[name].pack = bool(getattr(args, "save_packed", None))

    # ---- pass 1: Hessians.  Linears fed by the very same tensor share one accumulator. ----
    alias: Dict[str, str] = {}
    seen: Dict[tuple, tuple] = {}
    cur = {"batch": 1}

    # The hooks run BEFORE each linear: add_batch only needs the input (bigptq.py:37-54 never reads
    # `out`).  The first forward of the layer records the order in which the linears are called;
    # in the following ones the hook of the last linear stops the forward right after its Hessian
    # update, because nothing computed from there on is used: the outputs of this pass are
    # overwritten by the re-propagation with the quantized weights (run.py:376-377).
    call_order: List[str] = []

    def make_hook(name):
        def hook(_, inp):
            x = inp[0].data
            if x.dim() == 2 and cur["batch"] > 1:
                # some layers flatten [batch, tokens, C] before their linears (OPT fc1 / fc2); the
                # sample count of add_batch is the number of sequences (bigptq.py:41-49)
                x = x.reshape(cur["batch"], -1, x.shape[-1])
            if cur["last"] is None:
                call_order.append(name)
            key = (x.data_ptr(), tuple(x.shape), x.dtype)
            if name not in alias:
                if key in seen and seen[key][0] != name:
                    alias[name] = seen[key][0]
                else:
                    seen[key] = (name, x)      # keeps x alive so that its address stays unique
                    gptq[name].add_batch(x, None)
            if name == cur["last"]:
                raise _TailReached()
        return hook

    cur["last"] = None
    handles = [subset[name].register_forward_pre_hook(make_hook(name)) for name in gptq]
    n_local = inps.shape[0]
    fb = max(1, int(args.forward_batch))
    if n_local > fb:
        # same number of forwards, evenly filled (18 sequences: 6 + 6 + 6 instead of 8 + 8 + 2)
        n_batches = (n_local + fb - 1) // fb
        fb = (n_local + n_batches - 1) // n_batches
    with timer.span("forward_hessian"):
        feed = _Feeder(inps, fb, dev, keep_gib=float(getattr(args, "act_stage_gib", 16.0)))
        for b in range(len(feed)):
            x = feed.batch(b)
            seen.clear()
            cur["batch"] = x.shape[0]
            try:
                layer(x, **_replay_kwargs(layer_kwargs, x.shape[0]))
            except _TailReached:
                pass
            feed.done(b)
            if b == 0 and getattr(args, "skip_dead_tail", True) and call_order \
                    and call_order.count(call_order[-1]) == 1:
                cur["last"] = call_order[-1]
        seen.clear()
    for h in handles:
        h.remove()
    # pass 2 re-reads the shard pass 1 left on the device; a shard too large for that starts
    # travelling again now, while the linears are quantized
    feed2 = feed.second_pass()
    leaders = [n for n in gptq if n not in alias]
    with timer.span("hessian_allreduce"):
        if ws > 1:
            parallel.allreduce_hessians_([gptq[n]._S for n in leaders])
            total = int(parallel.sum_over_ranks(float(n_local), dev))
            for n in leaders:
                gptq[n].nsamples = total
    for name, lead in alias.items():
        gptq[name]._S = gptq[lead]._S
        gptq[name].nsamples = gptq[lead].nsamples

    # ---- quantization: each linear on its owner rank, result broadcast ----
    shapes = {n: (gptq[n].rows, gptq[n].columns) for n in gptq}
    owners = parallel.assign_owners(shapes, ws)
    errors: Dict[str, float] = {n: 0.0 for n in gptq}        # same key order on every rank
    mine = [n for n in gptq if owners[n] == rank]
    order = sorted(gptq, key=lambda n: -parallel.linear_cost(*shapes[n]))     # same on every rank
    main = torch.cuda.current_stream(dev) if dev.type == "cuda" else None
    concurrent = main is not None and getattr(args, "concurrent_linears", True)
    states = {}

    def finish(name, info):
        errors[name] = info["error"]
        if traces is not None and gptq[name].last_trace is not None:
            traces[name] = gptq[name].last_trace.cpu()
        if getattr(gptq[name], "packed", None) is not None:
            from . import packed as _packed
            os.makedirs(args.save_packed, exist_ok=True)
            _packed.save(os.path.join(args.save_packed, f"layer{index}.{name}.npz"), gptq[name].packed)
            gptq[name].packed = None
        for k, v in gptq[name].last_timing.items():
            timer.ms[k] = timer.ms.get(k, 0.0) + v

    if not concurrent:
        with timer.span("fasterquant"):
            for name in mine:
                if args.verbose:
                    print(index, name)
                    print("Quantizing ...")
                finish(name, gptq[name].fasterquant(percdamp=args.percdamp, blocksize=args.blocksize,
                                                    partition=args.partition, global_scale=args.global_scale))
            for name in gptq:
                gptq[name].free()
        with timer.span("weight_broadcast"):
            if ws > 1:
                for name in gptq:
                    parallel.broadcast_(subset[name].weight.data, owners[name])
        # ---- pass 2: re-propagate with the quantized weights (run.py:376-377) ----
        with timer.span("forward_repropagate"):
            feed = feed2
            for b in range(len(feed)):
                x = feed.batch(b)
                y = _layer_out(layer(x, **_replay_kwargs(layer_kwargs, x.shape[0])))
                feed.done(b)
                _store_outputs(outs, b * fb, y.reshape(x.shape), dev)
        del gptq
        return errors

    # Device path.  Every linear of this rank gets its own stream, so that the serial parts of one
    # (128-wide diagonal factorisations, small block kernels) overlap the wide kernels of another.
    # Each binarized weight is written into the layer's weight storage on the linear's stream (then
    # broadcast when there are several ranks) and an event marks it; the host does not wait for a
    # block loop before everything, the second pass included, has been enqueued.
    # `reprop_overlap` lets the forwards of the second pass start before the last linear is done:
    # its batches run on side streams and wait, in front of every linear, for that linear's event,
    # so a forward runs up to the first linear that is still being quantized.  On ONE B200 this moved
    # no time (the block loops and the forwards' GEMMs both need whole SMs - shared memory - so they
    # take turns on the SMs instead of sharing them): it is off there.  With three ranks or more it is
    # on (for device-resident activations): the ranks that do not own the layer's most expensive
    # linear would otherwise sit idle while its owner works (see parallel.plan_shards for the other
    # half of that arrangement).
    with timer.span("fasterquant"):
        start = torch.cuda.Event()
        start.record(main)
        mine_order = [n for n in order if owners[n] == rank]
        pool = _stream_pool(dev, len(mine_order))
        slot_of = {name: slot for slot, name in enumerate(mine_order)}
        # linears that share a Hessian on this rank share its factor: leaders first
        lead_of = {n: alias[n] for n in mine_order if n in alias and alias[n] in slot_of}
        begin_order = [n for n in mine_order if n not in lead_of] + [n for n in mine_order if n in lead_of]
        for name in begin_order:
            s = pool[slot_of[name]]
            s.wait_event(start)
            with torch.cuda.stream(s):
                states[name] = gptq[name].fasterquant_begin(
                    percdamp=args.percdamp, blocksize=args.blocksize, partition=args.partition,
                    global_scale=args.global_scale,
                    factor_from=states[lead_of[name]] if name in lead_of else None)
        # cheapest factorisations finish first: enqueue their block loops as soon as they are checked
        committed = {}
        for name in reversed(begin_order[:len(mine_order) - len(lead_of)]):
            committed[name] = gptq[name].fasterquant_commit(states[name])
            for other in (n for n in lead_of if lead_of[n] == name):
                committed[other] = gptq[other].fasterquant_commit(states[other])
        # the event behind which a linear's weight may be read on this rank; with several ranks the
        # weights travel in the order in which they get ready (cheapest first), on a stream of their own
        ready = dict(committed)
        if ws > 1:
            bc = _copy_streams(dev)[2]
            bc.wait_event(start)
            with torch.cuda.stream(bc):
                for name in reversed(order):
                    if name in committed:
                        bc.wait_event(committed[name])
                    parallel.broadcast_(subset[name].weight.data, owners[name])
                    ready[name] = torch.cuda.Event()
                    ready[name].record(bc)

        overlap = getattr(args, "reprop_overlap", None)
        if overlap is None:
            # host-resident activations: started early, the forwards would all end together and leave
            # the copies of their outputs nothing to hide behind
            overlap = ws >= 3 and inps.device.type == "cuda"
        feed = feed2
        lanes = []
        if overlap:
            # ---- pass 2 (run.py:376-377) started early, gated per linear ----
            def gate(name):
                def hook(_, inp):
                    torch.cuda.current_stream(dev).wait_event(ready[name])
                return hook

            handles = [subset[name].register_forward_pre_hook(gate(name)) for name in gptq]
            lanes = _lane_streams(dev, min(len(feed), max(1, int(getattr(args, "reprop_lanes", 16)))))
            try:
                for b in range(len(feed)):
                    lane = lanes[b % len(lanes)]
                    lane.wait_event(start)
                    with torch.cuda.stream(lane):
                        x = feed.batch(b, lane)
                        y = _layer_out(layer(x, **_replay_kwargs(layer_kwargs, x.shape[0])))
                        feed.done(b, lane)
                        _store_outputs(outs, b * fb, y.reshape(x.shape), dev)
            finally:
                for h in handles:
                    h.remove()
        # the phase ends on the caller's stream when the last weight is in place
        for name in gptq:
            main.wait_event(ready[name])
    with timer.span("forward_repropagate"):
        if overlap:
            # what the side streams still have to do is the exposed part of pass 2
            for lane in lanes:
                main.wait_stream(lane)
        else:
            # ---- pass 2: re-propagate with the quantized weights (run.py:376-377) ----
            for b in range(len(feed)):
                x = feed.batch(b)
                y = _layer_out(layer(x, **_replay_kwargs(layer_kwargs, x.shape[0])))
                feed.done(b)
                _store_outputs(outs, b * fb, y.reshape(x.shape), dev)
    for name in reversed(mine_order):
        if args.verbose:
            print(index, name)
            print("Quantizing ...")
        finish(name, gptq[name].fasterquant_end(states[name]))
    states.clear()
    for name in gptq:
        gptq[name].free()
    del gptq
    return errors


@torch.no_grad()
def quant_sequential(model, dataloader, dev, args=None) -> dict:
    """Calibrate and binarize every decoder layer in turn (run.py:122-387)."""
    args = args or default_args()
    args.low_quant_method = str(args.low_quant_method).lower()
    if args.low_quant_method not in TECHNIQUES:
        raise NotImplementedError(f"technique {args.low_quant_method!r}: implemented are {TECHNIQUES}")
    dev = torch.device(dev)
    rank, ws = parallel.world()
    if args.verbose:
        print("Starting ...")
    use_cache = model.config.use_cache
    model.config.use_cache = False
    layers, pre = _decoder_parts(model)
    dtype = next(iter(model.parameters())).dtype
    hidden = model.config.hidden_size
    batches = list(dataloader)[: args.nsamples]
    # (uneven shards pay only while the activations stay on the device: the copies of host-resident
    # shards need the whole layer to hide behind, see quantize_layer)
    stays_on_device = (len(batches) / ws) * model.seqlen * hidden * 2 <= args.act_offload_gib * (1024 ** 3)
    shard_sizes = getattr(args, "shard_sizes", None) or parallel.plan_shards(
        len(batches), ws, {n: tuple(m.weight.shape) for n, m in find_layers(layers[0]).items()},
        skew=dev.type == "cuda" and stays_on_device and bool(getattr(args, "shard_skew", True)))
    mine = parallel.shard_range(len(batches), rank, ws, shard_sizes)

    # ---- capture the inputs of layer 0 for this rank's sequences (run.py:175-201) ----
    sink = {"inps": [], "kwargs": {}}
    residents = [_Resident(m, dev) for m in pre] + [_Resident(layers[0], dev)]
    for r in residents:
        r.__enter__()
    layers[0] = _Catcher(layers[0], sink)
    for j in mine:
        try:
            model(batches[j][0].to(dev))
        except ValueError:
            pass
    layers[0] = layers[0].module
    for r in reversed(residents):
        r.__exit__()
    n_local = len(sink["inps"])
    act_bytes = n_local * model.seqlen * hidden * 2
    on_host = act_bytes > args.act_offload_gib * (1024 ** 3)         # run.py:166-172 uses 8 GiB
    pin = on_host and torch.cuda.is_available()
    kw = dict(dtype=dtype, device="cpu", pin_memory=pin) if on_host else dict(dtype=dtype, device=dev)
    inps = torch.zeros((n_local, model.seqlen, hidden), **kw)
    for j, x in enumerate(sink["inps"]):
        inps[j].copy_(x.reshape(model.seqlen, hidden))
    outs = torch.zeros((n_local, model.seqlen, hidden), **kw)
    layer_kwargs = sink["kwargs"]
    sink["inps"].clear()
    if args.verbose:
        print("Ready.")

    timer = _Timer()
    all_errors: List[Dict[str, float]] = []
    all_traces: List[Optional[dict]] = []
    t0 = time.time()
    # weights stream through the device: layer i + 1 is copied in and layer i - 1 copied out while
    # layer i is being quantized
    # (with several ranks one of them, a different one per layer, reads the layer from host memory and
    # the others get it over NVLink; the result goes back to rank 0's host copy only, unless
    # `replicate_result` asks for every rank's)
    keeper = None if getattr(args, "replicate_result", False) else 0

    def resident(i):
        return _Resident(layers[i], dev, loader=i % ws, keeper=keeper)

    nxt = resident(0).prefetch() if len(layers) else None
    leaving = None
    for i in range(len(layers)):
        res, nxt = nxt, None
        layer = res.__enter__()
        if i + 1 < len(layers):
            nxt = resident(i + 1).prefetch()
        layer_traces = {} if getattr(args, "keep_traces", False) else None
        errs = quantize_layer(layer, i, inps, outs, layer_kwargs, args, dev, timer, layer_traces)
        all_traces.append(layer_traces)
        if leaving is not None:
            leaving.finish()
        res.__exit__(defer=True)
        leaving = res
        all_errors.append(errs)
        inps, outs = outs, inps
    if leaving is not None:
        leaving.finish()
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)          # outputs on their way to the host have arrived
    timing = timer.collect()
    timing["wall_s"] = time.time() - t0
    model.config.use_cache = use_cache
    total = sum(sum(e.values()) for e in all_errors)
    total = parallel.sum_over_ranks(total, dev)
    return {"errors": all_errors, "error_sum": total, "timing_ms": timing, "final_hidden": inps,
            "traces": all_traces}


# ---------------------------------------------------------------------------------------------
def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="CRB / BiLLM calibration-time binarization on B200")
    p.add_argument("model", type=str, help="local checkpoint directory or a model name whose shape is known")
    p.add_argument("dataset", type=str, choices=["wikitext2", "ptb", "c4"])
    p.add_argument("low_quant_method", type=str.lower, choices=list(TECHNIQUES))
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--nsamples", type=int, default=128)
    p.add_argument("--seqlen", type=int, default=None)
    p.add_argument("--percdamp", type=float, default=0.01)
    p.add_argument("--blocksize", type=int, default=128)
    p.add_argument("--salient_metric", type=str, default="magnitude", choices=["magnitude", "hessian"])
    p.add_argument("--partition", type=int, default=3)
    p.add_argument("--global_scale", action="store_true")
    p.add_argument("--device", type=str, default="cuda:0")
    p.add_argument("--disable_gptq", action="store_true")
    p.add_argument("--minlayer", type=int, default=-1)
    p.add_argument("--maxlayer", type=int, default=1000)
    p.add_argument("--quant_only", type=str, default="")
    p.add_argument("--invert", action="store_true")
    p.add_argument("--corr_damp", type=float, default=0.1)
    p.add_argument("--lam", type=float, default=1e-5)
    p.add_argument("--coupling", type=float, default=0.5)
    p.add_argument("--layers", type=int, default=None, help="synthetic models only: number of decoder layers")
    p.add_argument("--forward_batch", type=int, default=8, help="sequences per layer forward")
    p.add_argument("--act_offload_gib", type=float, default=64.0,
                   help="activations of all sequences stay in pinned host memory above this size (run.py:166-172 uses 8)")
    p.add_argument("--act_stage_gib", type=float, default=16.0,
                   help="host-resident activations: a shard up to this size is copied in once per layer and kept "
                        "on the device for both passes")
    p.add_argument("--reprop_lanes", type=int, default=16,
                   help="with --reprop_overlap: batches that may be in flight (each on its own stream); each holds "
                        "one batch of intermediate activations")
    p.add_argument("--reprop_overlap", type=int, default=None, choices=(0, 1),
                   help="1: start the forwards of the re-propagation pass (on side streams, gated per linear) while "
                        "the layer's last linear is still being quantized; default: on with three ranks or more")
    p.add_argument("--replicate_result", action="store_true",
                   help="several ranks: write the binarized weights back into every rank's host copy of the model "
                        "(default: rank 0's only)")
    p.add_argument("--no_shard_skew", dest="shard_skew", action="store_false",
                   help="always split the calibration sequences evenly over the ranks")
    p.add_argument("--save_packed", type=str, default=None,
                   help="directory that receives the packed form (bit planes + scales) of every binarized linear")
    p.add_argument("--quiet", action="store_true")
    return p


def main(argv=None):
    args = build_parser().parse_args(argv)
    args.verbose = not args.quiet
    if "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        args.device = f"cuda:{local}"
    rank, ws = parallel.world()
    args.verbose = args.verbose and rank == 0
    model = get_model(args.model, fill_device=args.device, n_layers=args.layers)
    if args.seqlen:
        model.seqlen = args.seqlen
    loader, _ = get_loaders(args.dataset, args.nsamples, args.seed, model.seqlen, model, args.model)
    tick = time.time()
    out = quant_sequential(model, loader, args.device, args)
    if rank == 0:
        print("quantization time:", time.time() - tick, "s")
        print("sum of block errors:", out["error_sum"])
        print({k: round(v, 1) for k, v in out["timing_ms"].items()})
    return out


if __name__ == "__main__":
    main()
