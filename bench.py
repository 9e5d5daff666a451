"""Benchmark of the calibration-time binarization path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Metric: wall seconds to CRB-binarize the OPT-6.7b-shaped model (32 decoder layers,
128 x 2048 calibration tokens), lower is better.  A step is ONE decoder layer through the
whole path (hooked calibration forwards -> Hessians -> factorisation -> block loop with
trailing updates -> re-propagation); all 32 layers have the same shape and cost, so
`value` = seconds per step x 32.  Weights are random-init and the calibration ids are
uniform random (no checkpoints or datasets offline).

`value` times the step with the layer weights and the layer inputs resident in HBM;
`e2e` times the same step when the layer weights and the calibration activations start
in pinned host memory and the quantized weights and layer outputs are copied back.

--impl reference times the reference's own CPU code of the path (oracle/_ref when it was
built, else the CPU restatement in oracle/) on the host cores on one fixed bounded sample
and extrapolates it to the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = "opt-6.7b"
MODEL_LAYERS = 32
NSAMPLES, SEQLEN = 128, 2048


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons = [], [], set()
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
CPU_SAMPLE_ROWS, CPU_SAMPLE_COLS, CPU_SAMPLE_SEQS = 4096, 4096, 8


def cpu_reference_sample(technique="crb"):
    """Times the reference's path on the host cores on ONE fixed, bounded sample and extrapolates.

    Sample (the same wherever this is called): one whole q_proj-shaped linear, 4096 x 4096 --
    Hessian from 8 sequences of 2048 tokens through add_batch, then fasterquant (damping,
    factorisation chain, all 32 block steps with their trailing updates).  The code timed is the
    reference's own (`oracle/_ref`, its modules byte-compiled where they lie) when that was built,
    else the CPU restatement in `oracle/`.  Every host thread is used whatever OMP_NUM_THREADS the
    launcher exported.
    Extrapolation to one OPT-6.7b decoder layer: add_batch time scales with tokens x C^2 and runs
    once per linear in the reference (q, k, v recompute the same Hessian: run.py:341-353); the
    factorisation scales with C^3; the block loop with rows x cols (whole linear measured, so the
    per-block fixed costs are in the figure).  Layer forwards are NOT included (hot path only).
    """
    import contextlib
    import io
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    rows, cols, nseq = CPU_SAMPLE_ROWS, CPU_SAMPLE_COLS, CPU_SAMPLE_SEQS
    g = torch.Generator().manual_seed(0)
    W = torch.randn(rows, cols, generator=g) * 0.02
    xs = [torch.randn(1, SEQLEN, cols, generator=g).half() for _ in range(nseq)]
    from oracle import build_ref
    kind = "reference" if build_ref.available() else "port"
    if kind == "reference":
        bigptq, binary, _ = build_ref.load()
        lin = torch.nn.Linear(cols, rows, bias=False)
        lin.weight.data = W.clone()
        gq = bigptq.BRAGPTQ(lin, binary.Binarization(lin.weight, method=technique, groupsize=128), "hessian")
        t0 = time.time()
        for x in xs:
            gq.add_batch(x, None)
        t_hess = time.time() - t0
        # few tokens: lift the diagonal so that the factorisation needs no retry
        gq.H += torch.eye(cols) * gq.H.diagonal().mean() * 0.1
        chol = torch.linalg.cholesky
        t_fac = [0.0]

        def timed_chol(*a, **k):
            t = time.time()
            out = chol(*a, **k)
            t_fac[0] += time.time() - t
            return out

        inv = torch.cholesky_inverse

        def timed_inv(*a, **k):
            t = time.time()
            out = inv(*a, **k)
            t_fac[0] += time.time() - t
            return out

        torch.linalg.cholesky, torch.cholesky_inverse = timed_chol, timed_inv
        try:
            t0 = time.time()
            with contextlib.redirect_stdout(io.StringIO()):
                gq.fasterquant(blocksize=128, percdamp=0.01, partition=3)
            t_quant = time.time() - t0
        finally:
            torch.linalg.cholesky, torch.cholesky_inverse = chol, inv
        t_factor, t_blocks = t_fac[0], t_quant - t_fac[0]
    else:
        from oracle import crb_oracle as O
        H = torch.zeros(cols, cols)
        t0 = time.time()
        n = 0
        for x in xs:
            n = O.hessian_add_batch(H, n, x)
        t_hess = time.time() - t0
        H += torch.eye(cols) * H.diagonal().mean() * 0.1
        t0 = time.time()
        Wc = W.clone()
        U = O.hinv_upper_factor(H, Wc, 0.01)
        t_factor = time.time() - t0
        t0 = time.time()
        O.quantize_linear(Wc, None, technique, U=U, keep_blocks=False)
        t_blocks = time.time() - t0
    d, f = 4096, 16384
    hess_unit = t_hess / (nseq * SEQLEN * cols * cols)             # s per token * C^2
    # the reference accumulates one Hessian per linear: q, k, v, out, fc1 on 4096 inputs, fc2 on 16384
    layer_hess = hess_unit * NSAMPLES * SEQLEN * (5 * d * d + f * f)
    layer_factor = t_factor / cols ** 3 * (5 * d ** 3 + f ** 3)
    layer_blocks = t_blocks / (rows * cols) * (4 * d * d + 2 * d * f)
    layer_s = layer_hess + layer_factor + layer_blocks
    return dict(layer_s=layer_s, sample_s=t_hess + t_factor + t_blocks, kind=kind,
                phases=dict(hessian_s=layer_hess, factor_s=layer_factor, blocks_s=layer_blocks),
                sample_phases=dict(hessian_s=t_hess, factor_s=t_factor, blocks_s=t_blocks),
                cores=torch.get_num_threads(),
                sample=(("the reference's own code (oracle/_ref)" if kind == "reference" else "CPU port of the reference path")
                        + f": one whole {rows}x{cols} linear (q_proj shape), add_batch on {nseq}x{SEQLEN} tokens, "
                          f"fasterquant with its factorisation chain and all 32 block steps; extrapolated per phase to one "
                          f"{MODEL} layer (forwards excluded)"))


CPU_ARM_BUDGET_S = 200.0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # every step is the same fixed sample; when W + K of them would not fit the budget, fewer
    # repeats are run (at least one timed), never a smaller sample
    times, info, spent, done_warm = [], None, 0.0, 0
    for i in range(args.warmup + args.steps):
        warm = i < args.warmup
        if info is not None and spent + info["sample_s"] * 1.3 > CPU_ARM_BUDGET_S and (warm or times):
            continue
        if warm and done_warm >= 1 and spent + 2 * info["sample_s"] * 1.3 > CPU_ARM_BUDGET_S:
            continue                          # keep room for one timed repeat
        t0 = time.time()
        info = cpu_reference_sample(args.technique)
        spent += time.time() - t0
        if warm:
            done_warm += 1
        else:
            times.append(info["layer_s"])
    layer_s = sum(times) / len(times)
    value = layer_s * MODEL_LAYERS
    line = {"impl": "reference", "metric": "wall_s_to_binarize_opt_6.7b_crb", "value": value, "unit": "s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": layer_s * 1e3,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(args),
            "cpu_baseline": {"value": value, "unit": "s", "cores": info["cores"], "kind": info["kind"],
                             "sample": info["sample"], "sample_s": info["sample_s"],
                             "repeats_timed": len(times), "repeats_warmup": done_warm},
            "e2e": {"value": value, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "phases_s_per_layer": info["phases"]}
    print(json.dumps(line))


def workload_config(args):
    return {"workload": f"{MODEL} shape (d_model 4096, ffn 16384, 32 heads, fp16), {MODEL_LAYERS} layers, "
                        f"{NSAMPLES}x{SEQLEN} uniform-token calibration, technique {args.technique}, blocksize 128, "
                        f"salient_metric hessian; one step = one decoder layer, value = 32 x step",
            "technique": args.technique, "layers_timed": args.steps, "layers_model": MODEL_LAYERS,
            "nsamples": NSAMPLES, "seqlen": SEQLEN, "parallelism": f"token-sharded Hessians + per-linear owners x{args.gpus}",
            "l2": "inputs larger than L2 (per-layer activations 2 GiB, weights 0.4 GiB)"}


# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    from crb_b200 import ops, parallel
    from crb_b200 import run as crun
    from crb_b200.synth import synthetic_calibration

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    per_arm = args.warmup + args.steps
    n_layers = 2 * per_arm                      # layers [0, per_arm): resident arm; the rest: host arm
    model = crun.get_model(args.model, fill_device=str(dev), n_layers=n_layers)
    model.seqlen = args.seqlen
    qargs = crun.default_args(model=args.model, low_quant_method=args.technique, nsamples=args.nsamples,
                              device=str(dev), forward_batch=args.forward_batch, verbose=False,
                              reprop_overlap=None if args.reprop_overlap is None else bool(args.reprop_overlap))
    loader = synthetic_calibration(model.config.vocab_size, args.nsamples, args.seqlen, seed=0)

    # ---- layer-0 inputs of this rank's sequences, kept in pinned host memory.  The two arms shard the
    # sequences differently from three ranks on: with device-resident activations the owner of the
    # layer's dominant last linear gets fewer sequences (parallel.plan_shards); with host buffers the
    # split stays even, because there the copies of a shard need the whole layer to hide behind ----
    layers, pre = crun._decoder_parts(model)
    shapes0 = {n: tuple(m.weight.shape) for n, m in crun.find_layers(layers[0]).items()}
    shard_sizes = parallel.plan_shards(len(loader), world, shapes0, skew=not args.no_shard_skew)
    shard_sizes_host = parallel.plan_shards(len(loader), world, shapes0, skew=False)
    hidden = model.config.hidden_size
    dtype = next(iter(model.parameters())).dtype
    sink = {"inps": [], "kwargs": {}}

    def capture(sizes):
        mine = parallel.shard_range(len(loader), rank, world, sizes)
        sink["inps"].clear()
        with torch.no_grad():
            res = [crun._Resident(m, dev) for m in pre] + [crun._Resident(layers[0], dev)]
            for r in res:
                r.__enter__()
            layers[0] = crun._Catcher(layers[0], sink)
            for j in mine:
                try:
                    model(loader[j][0].to(dev))
                except ValueError:
                    pass
            layers[0] = layers[0].module
            for r in reversed(res):
                r.__exit__()
        buf = torch.empty((len(sink["inps"]), args.seqlen, hidden), dtype=dtype, pin_memory=True)
        for j, x in enumerate(sink["inps"]):
            buf[j].copy_(x.reshape(args.seqlen, hidden))
        return buf

    first = capture(shard_sizes)
    dev_in = torch.empty(tuple(first.shape), dtype=dtype, device=dev)
    dev_out = torch.empty_like(dev_in)
    dev_in.copy_(first)
    host_in = first if shard_sizes_host == shard_sizes else capture(shard_sizes_host)
    del first
    host_out = torch.empty_like(host_in, pin_memory=True)
    layer_kwargs = sink["kwargs"]
    sink["inps"].clear()
    layer_bytes = sum(p.numel() * p.element_size() for p in layers[0].parameters())
    act_bytes = host_in.numel() * host_in.element_size()

    # ---- roofline of the dominant kernel: the tcgen05 Hessian accumulation, timed alone before the
    # long loops (the peak it is compared with is the burst figure of a kernel timed alone) ----
    peaks = read_peaks()
    d, f = hidden, model.config.ffn_dim if hasattr(model.config, "ffn_dim") else model.config.intermediate_size
    roof = hessian_roofline(dev, d, f, args, peaks)
    roof_extra = extra_rooflines(dev, d, f, args.technique, peaks) if rank == 0 else None

    timer = crun._Timer()
    sampler = ClockSampler(local)
    step_events = []
    errors = []

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- arm 1 (`value`): weights and activations resident in HBM when a step starts ----
    def resident_step(i, timed):
        nonlocal dev_in, dev_out
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        with crun._Resident(layers[i], dev) as layer:
            # this arm times a step whose weights and activations are resident: all ranks start it
            # together, so that one rank's slower weight copy between two steps (untimed) does not
            # show up as waiting time inside the next step's collectives on the other ranks
            barrier()
            ev[0].record()
            with torch.no_grad():
                errs = crun.quantize_layer(layer, i, dev_in, dev_out, layer_kwargs, qargs, dev,
                                           timer if timed else None)
            ev[1].record()
        dev_in, dev_out = dev_out, dev_in                  # next layer calibrates on these outputs
        if timed:
            step_events.append(ev)
            errors.append(sum(errs.values()))

    for i in range(args.warmup):
        resident_step(i, False)
    barrier()
    launches0 = ops.launch_count()
    sampler.start()
    t0 = time.time()
    for i in range(args.warmup, per_arm):
        resident_step(i, True)
    barrier()
    wall = time.time() - t0
    clocks = sampler.stop()
    launches = ops.launch_count() - launches0
    phases = timer.collect()
    dev_ms = sum(e[0].elapsed_time(e[1]) for e in step_events)

    # ---- arm 2 (`e2e`): the same call on HOST buffers.  Weights and activations start every step in
    # pinned host memory and end there; quantize_layer streams the activations through the device
    # batch by batch (once in, once out) and the weights of the next / previous layer move while a
    # layer is being quantized.  Timed as a whole: first copy in to last copy out. ----
    torch.cuda.synchronize()
    qargs_host = crun.default_args(**{**vars(qargs), "reprop_overlap": bool(args.reprop_overlap)})

    def host_steps(first, count):
        nonlocal host_in, host_out
        if count <= 0:
            return
        # one rank (a different one per layer) reads the layer from host memory, the others receive it
        # over NVLink; the quantized layer goes back to rank 0's host copy
        def resident(i):
            return crun._Resident(layers[i], dev, loader=i % world, keeper=0)

        nxt = resident(first).prefetch()
        leaving = None
        for i in range(first, first + count):
            res, nxt = nxt, None
            layer = res.__enter__()
            if i + 1 < first + count:
                nxt = resident(i + 1).prefetch()
            with torch.no_grad():
                crun.quantize_layer(layer, i, host_in, host_out, layer_kwargs, qargs_host, dev, None)
            if leaving is not None:
                leaving.finish()
            res.__exit__(defer=True)
            leaving = res
            host_in, host_out = host_out, host_in
        leaving.finish()
        torch.cuda.current_stream().wait_stream(crun._copy_streams(dev)[1])

    host_steps(per_arm, args.warmup)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    host_steps(per_arm + args.warmup, args.steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    # per-rank step time and phases (device time on each rank's own stream), to see which rank and
    # which phase the maximum comes from
    keys = ["forward_hessian", "hessian_allreduce", "fasterquant", "weight_broadcast", "forward_repropagate"]
    mine_vec = torch.tensor([dev_ms] + [phases.get(k, 0.0) for k in keys], dtype=torch.float64, device=dev)
    if world > 1:
        gathered = [torch.zeros_like(mine_vec) for _ in range(world)]
        dist.all_gather(gathered, mine_vec)
    else:
        gathered = [mine_vec]
    per_rank = [{"step": round(float(v[0]) / args.steps, 2),
                 **{k: round(float(v[1 + j]) / args.steps, 2) for j, k in enumerate(keys)}} for v in gathered]
    dev_ms = parallel.max_over_ranks(dev_ms, dev)
    e2e_ms = parallel.max_over_ranks(e2e_ms, dev)
    launches = int(parallel.sum_over_ranks(float(launches), dev))
    err_sum = parallel.sum_over_ranks(float(sum(errors)), dev)
    act_bytes = int(parallel.sum_over_ranks(float(act_bytes), dev))          # all ranks' shards
    # the layer itself crosses PCIe once each way whatever the number of ranks
    ms_per_step = dev_ms / args.steps
    value = ms_per_step * MODEL_LAYERS / 1e3
    e2e_value = e2e_ms / args.steps * MODEL_LAYERS / 1e3


    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            ref_gpu = reference_eager_on_gpu(dev, args.technique)
        except Exception as exc:            # a baseline, not the product: report and go on
            ref_gpu = {"unavailable": f"{type(exc).__name__}: {exc}"}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        info = cpu_reference_sample(args.technique)
        cpu = {"value": info["layer_s"] * MODEL_LAYERS, "unit": "s", "cores": info["cores"], "kind": info["kind"],
               "sample": info["sample"], "sample_s": info["sample_s"], "phases_s_per_layer": info["phases"]}

    if rank == 0:
        line = {"metric": "wall_s_to_binarize_opt_6.7b_crb", "value": value, "unit": "s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32 (fp16 operands on the Hessian tensor cores)",
                "data": "synthetic", "config": workload_config(args),
                "e2e": {"value": e2e_value, "unit": "s", "h2d_bytes_per_step": layer_bytes + act_bytes,
                        "d2h_bytes_per_step": layer_bytes + act_bytes + 8 * 6,
                        "note": "same call on pinned host buffers, bytes summed over ranks; per step the layer's weights "
                                "(read from host memory by one rank, passed on over NVLink) "
                                "and each rank's activation shard are copied in once (the shard stays on the device for the "
                                "re-propagation pass) and the quantized weights and the layer outputs are copied "
                                "out; copies overlap compute"},
                "gpu_launches": launches, "clocks": clocks, "roofline": roof, "roofline_extra": roof_extra,
                "cpu_baseline": cpu, "reference_eager_gpu": ref_gpu,
                "phases_ms_per_step": {k: v / args.steps for k, v in phases.items()},
                "per_rank_ms_per_step": per_rank, "sequences_per_rank": shard_sizes,
                "sequences_per_rank_e2e": shard_sizes_host,
                "block_error_sum_per_layer": err_sum / args.steps, "wall_clock_s_timed_region": wall,
                "peaks": peaks["source"]}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of k_hessian_umma_pair on fp16
# X [T, C], from an ncu capture of exactly that launch (profiles/k_hessian_umma_pair_fp16.txt);
# the algorithmic bytes of the launch are T*C*2 + 2 * 4 * C*(C+256)/2 = 1.63e9.
HESSIAN_DRAM_BYTES = {(16384, 16384): 10915788544 + 560216064}


def hessian_roofline(dev, d, f, args, peaks):
    """Times the Hessian kernel alone on this workload's largest input (fc2: tokens x ffn) with
    CUDA events on the launching stream and relates the MMA flops it issues to the measured peak."""
    from crb_b200 import ops
    T = args.forward_batch * args.seqlen
    X = torch.randn(T, f, device=dev, dtype=torch.float16)
    S = torch.zeros(f, f, device=dev)
    for _ in range(2):
        ops.hessian_accumulate(S, X)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    a.record()
    for _ in range(reps):
        ops.hessian_accumulate(S, X)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / reps
    nt = (f + 255) // 256
    tiles = nt * (nt + 1) // 2                      # upper-triangle 256 x 256 tiles, one per CTA pair
    issued = tiles * 256 * 256 * 2.0 * T
    algorithmic = 2.0 * T * f * f
    achieved = issued / (ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"]
    del X, S
    return {"kernel": "k_hessian_umma_pair", "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "traffic": HESSIAN_DRAM_BYTES.get((T, f)), "launch_ms": ms,
            "work": f"T={T} tokens x C={f}: {issued:.3e} flop issued on upper-triangle tiles "
                    f"({algorithmic:.3e} for the full product the reference computes)",
            "peak_source": f"{peaks['source']} cuBLAS bf16 burst"}


def reference_eager_on_gpu(dev, technique):
    """The reference's own eager-PyTorch path on this GPU, as the stronger baseline for the block
    loop: `BRAGPTQ.fasterquant` of the reference (oracle/_ref) on one 4096 x 4096 linear with an
    injected Hessian, next to this library on the very same inputs.  Rank 0, one GPU, bounded (the
    reference launches several thousand small kernels and synchronises some hundred times per block).
    """
    from oracle import build_ref
    if not build_ref.available():
        return None
    import contextlib
    import io
    from crb_b200 import BRAGPTQ, Binarization
    bigptq, binary, _ = build_ref.load()
    rows = cols = 4096
    g = torch.Generator(device=dev).manual_seed(5)
    W = torch.randn(rows, cols, generator=g, device=dev) * 0.02
    X = torch.randn(4 * SEQLEN, cols, generator=g, device=dev)
    H = (X.t() @ X) * (2.0 / 4)
    out = {"linear": f"{rows}x{cols}", "technique": technique}
    for name in ("ours", "reference"):
        lin = torch.nn.Linear(cols, rows, bias=False, device=dev, dtype=torch.float16)
        lin.weight.data = W.half()
        if name == "ours":
            q = BRAGPTQ(lin, Binarization(lin.weight, method=technique, groupsize=128), salient_metric="hessian")
            q.verbose = False
        else:
            q = bigptq.BRAGPTQ(lin, binary.Binarization(lin.weight, method=technique, groupsize=128), "hessian")
        reps = 3 if name == "ours" else 1
        best = None
        for _ in range(reps):
            lin.weight.data = W.half()
            q.H = H.clone()
            q.nsamples = 4
            torch.cuda.synchronize()
            t0 = time.time()
            with contextlib.redirect_stdout(io.StringIO()):
                info = q.fasterquant(blocksize=128, percdamp=0.01)
            torch.cuda.synchronize()
            dt = time.time() - t0
            best = dt if best is None else min(best, dt)
        out[f"{name}_fasterquant_s"] = best
        out[f"{name}_error"] = float(info["error"])
    out["speedup"] = out["reference_fasterquant_s"] / out["ours_fasterquant_s"]
    return out


def _time_ms(fn, reps, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def extra_rooflines(dev, d, f, technique, peaks):
    """The other two kernels the metric names, each timed alone with CUDA events on the launching
    stream at the workload's shapes: the trailing-update GEMM (K = 128, fc2-shaped: 4096 rows,
    16384 columns, first block) and the block step (fc1-shaped: 16384 rows; q_proj-shaped: 4096)."""
    from crb_b200 import ops
    out = []
    # ---- trailing update W[:, 128:] -= Err @ U[0:128, 128:]  (bigptq.py:264) ----
    R, C = d, f
    W = torch.randn(R, C, device=dev) * 0.02
    Err = torch.randn(R, 128, device=dev) * 0.01
    U = torch.triu(torch.randn(C, C, device=dev) * 0.01)
    ms = _time_ms(lambda: ops.trailing_update(W, Err, U, 0), reps=20)
    flops = 2.0 * R * 128 * (C - 128)
    nbytes = 8.0 * R * (C - 128) + 4.0 * R * 128 + 4.0 * 128 * (C - 128)
    out.append({"kernel": "k_gemm_tf32x3 (trailing update, K=128)", "bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "launch_ms": ms, "tflops_fp32_equivalent": flops / (ms * 1e-3) / 1e12,
                "tensor_frac_of_bf16_peak": 3.0 * flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                "work": f"R={R}, N={C - 128}, K=128: {flops:.3e} flop (three TF32 MMAs per term), "
                        f"{nbytes:.3e} B (W read + written, Err, U rows); 32 flop/B: HBM bound",
                "peak_source": f"{peaks['source']} copy bandwidth"})
    del W, Err, U
    # ---- block step: 8 dependent kernels per 128-column block ----
    for R in (f, d):
        W = torch.randn(R, 256, device=dev) * 0.02
        U = torch.diag(0.5 + torch.rand(256, device=dev))
        bufs = ops.block_step(W, U, 0, technique, want_codes=False)
        W0 = W.clone()

        def one_block():
            W[:, :128].copy_(W0[:, :128])         # the step overwrites its block with Q: start from weights again
            ops.block_step(W, U, 0, technique, reuse=bufs)

        ms_copy = _time_ms(lambda: W[:, :128].copy_(W0[:, :128]), reps=50, warm=10)
        ms = _time_ms(one_block, reps=50, warm=10) - ms_copy
        nbytes = 1536.0 * R + 65536.0
        out.append({"kernel": "block step (8 kernels)", "bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9,
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                    "launch_ms": ms,
                    "work": f"R={R}: {nbytes:.3e} algorithmic B per block (W block read, Q and Err written, U block, "
                            f"losses); the searches cost about 1e3 flop per element, so the step is latency / issue bound",
                    "peak_source": f"{peaks['source']} copy bandwidth"})
        del W, U
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--technique", default="crb", choices=["crb", "crbog", "braq"])
    ap.add_argument("--nsamples", type=int, default=NSAMPLES)
    ap.add_argument("--seqlen", type=int, default=SEQLEN)
    ap.add_argument("--forward_batch", type=int, default=8)
    ap.add_argument("--no_cpu_baseline", action="store_true")
    ap.add_argument("--reprop_overlap", type=int, default=None, choices=(0, 1),
                    help="forwards of the re-propagation pass on side streams, gated per linear "
                         "(default: on with three ranks or more; no gain on one GPU)")
    ap.add_argument("--no_shard_skew", action="store_true",
                    help="split the calibration sequences evenly even when one rank owns the critical linear")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
        run_ours(args)


if __name__ == "__main__":
    main()
