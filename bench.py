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

--impl reference times the CPU port of the reference's path (the oracle) on the host
cores on a bounded sample and extrapolates it to the same workload.
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
def cpu_port_sample(threads=None, rows=2048, cols=4096, nseq=2, technique="crb"):
    """Times the CPU port of the reference's path on a bounded sample and extrapolates.

    Sample: a `rows` x 4096 slice of a q_proj-shaped linear; Hessian from `nseq` sequences of
    2048 tokens; factorisation of the 4096 x 4096 Hessian; the full block loop on the slice.
    Extrapolation to one OPT-6.7b decoder layer: Hessian time scales with tokens x C^2 per
    distinct input, factorisation with C^3 per linear, block loop with rows x cols per linear.
    Layer forwards are NOT included (hot path only).
    """
    from oracle import crb_oracle as O
    if threads:
        torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    W = torch.randn(rows, cols, generator=g) * 0.02
    H = torch.zeros(cols, cols)
    t0 = time.time()
    n = 0
    for j in range(nseq):
        x = torch.randn(SEQLEN, cols, generator=g).half()
        n = O.hessian_add_batch(H, n, x.unsqueeze(0))
    t_hess = time.time() - t0
    # the sample Hessian comes from few tokens: lift the diagonal so that it stays well conditioned
    H += torch.eye(cols) * H.diagonal().mean() * 0.1
    t0 = time.time()
    Wc = W.clone()
    U = O.hinv_upper_factor(H, Wc, 0.01)
    t_factor = time.time() - t0
    t0 = time.time()
    O.quantize_linear(Wc, None, technique, U=U, keep_blocks=False)
    t_blocks = time.time() - t0
    d, f = 4096, 16384
    hess_unit = t_hess / (nseq * SEQLEN * cols * cols)             # s per token*C^2
    layer_hess = hess_unit * NSAMPLES * SEQLEN * (5 * d * d + f * f)   # q,k,v,out,fc1 inputs + fc2 input
    fac_unit = t_factor / cols ** 3
    layer_factor = fac_unit * (5 * d ** 3 + f ** 3)
    blk_unit = t_blocks / (rows * cols)
    layer_blocks = blk_unit * (4 * d * d + 2 * d * f)
    layer_s = layer_hess + layer_factor + layer_blocks
    return dict(layer_s=layer_s, sample_s=t_hess + t_factor + t_blocks,
                phases=dict(hessian_s=layer_hess, factor_s=layer_factor, blocks_s=layer_blocks),
                cores=torch.get_num_threads(),
                sample=(f"CPU port of the reference path: {rows}x{cols} slice of q_proj, Hessian from {nseq}x{SEQLEN} "
                        f"tokens, 4096^2 factorisation, 32-block loop; extrapolated per phase to one "
                        f"{MODEL} layer (forwards excluded)"))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    info = None
    # bounded sample: about 150 s of CPU work for the whole run
    per_step = 150.0 / max(1, args.warmup + args.steps)
    rows = 2048 if per_step >= 14 else 1024 if per_step >= 8 else 512 if per_step >= 5 else 256
    for i in range(args.warmup + args.steps):
        info = cpu_port_sample(rows=rows)
        if i >= args.warmup:
            times.append(info["layer_s"])
    layer_s = sum(times) / len(times)
    value = layer_s * MODEL_LAYERS
    line = {"impl": "reference", "metric": "wall_s_to_binarize_opt_6.7b_crb", "value": value, "unit": "s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": layer_s * 1e3,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(args),
            "cpu_baseline": {"value": value, "unit": "s", "cores": info["cores"], "kind": "port",
                             "sample": info["sample"]},
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
                              device=str(dev), forward_batch=args.forward_batch, verbose=False)
    loader = synthetic_calibration(model.config.vocab_size, args.nsamples, args.seqlen, seed=0)

    # ---- layer-0 inputs of this rank's sequences, kept in pinned host memory ----
    layers, pre = crun._decoder_parts(model)
    mine = parallel.shard_range(len(loader), rank, world)
    sink = {"inps": [], "kwargs": {}}
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
    hidden = model.config.hidden_size
    dtype = next(iter(model.parameters())).dtype
    n_local = len(sink["inps"])
    host_in = torch.empty((n_local, args.seqlen, hidden), dtype=dtype, pin_memory=True)
    for j, x in enumerate(sink["inps"]):
        host_in[j].copy_(x.reshape(args.seqlen, hidden))
    host_out = torch.empty_like(host_in, pin_memory=True)
    dev_in = torch.empty((n_local, args.seqlen, hidden), dtype=dtype, device=dev)
    dev_out = torch.empty_like(dev_in)
    dev_in.copy_(host_in)
    layer_kwargs = sink["kwargs"]
    sink["inps"].clear()
    layer_bytes = sum(p.numel() * p.element_size() for p in layers[0].parameters())
    act_bytes = host_in.numel() * host_in.element_size()

    timer = crun._Timer()
    sampler = ClockSampler(local)
    step_events = []
    errors = []

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- arm 1 (`value`): weights and activations resident in HBM when a step starts ----
    def resident_step(i, timed):
        nonlocal dev_in, dev_out
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        with crun._Resident(layers[i], dev) as layer:
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
    # batch by batch (twice in, once out) and the weights of the next / previous layer move while a
    # layer is being quantized.  Timed as a whole: first copy in to last copy out. ----
    host_in.copy_(dev_in)
    torch.cuda.synchronize()

    def host_steps(first, count):
        nonlocal host_in, host_out
        if count <= 0:
            return
        nxt = crun._Resident(layers[first], dev).prefetch()
        leaving = None
        for i in range(first, first + count):
            res, nxt = nxt, None
            layer = res.__enter__()
            if i + 1 < first + count:
                nxt = crun._Resident(layers[i + 1], dev).prefetch()
            with torch.no_grad():
                crun.quantize_layer(layer, i, host_in, host_out, layer_kwargs, qargs, dev, None)
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

    dev_ms = parallel.max_over_ranks(dev_ms, dev)
    e2e_ms = parallel.max_over_ranks(e2e_ms, dev)
    launches = int(parallel.sum_over_ranks(float(launches), dev))
    err_sum = parallel.sum_over_ranks(float(sum(errors)), dev)
    ms_per_step = dev_ms / args.steps
    value = ms_per_step * MODEL_LAYERS / 1e3
    e2e_value = e2e_ms / args.steps * MODEL_LAYERS / 1e3

    # ---- roofline of the dominant kernel: the tcgen05 Hessian accumulation ----
    peaks = read_peaks()
    d, f = hidden, model.config.ffn_dim if hasattr(model.config, "ffn_dim") else model.config.intermediate_size
    roof = hessian_roofline(dev, d, f, args, peaks)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        info = cpu_port_sample()
        cpu = {"value": info["layer_s"] * MODEL_LAYERS, "unit": "s", "cores": info["cores"], "kind": "port",
               "sample": info["sample"], "sample_s": info["sample_s"]}

    if rank == 0:
        line = {"metric": "wall_s_to_binarize_opt_6.7b_crb", "value": value, "unit": "s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32 (fp16 operands on the Hessian tensor cores)",
                "data": "synthetic", "config": workload_config(args),
                "e2e": {"value": e2e_value, "unit": "s", "h2d_bytes_per_step": layer_bytes + 2 * act_bytes,
                        "d2h_bytes_per_step": layer_bytes + act_bytes + 8 * 6,
                        "note": "same call on pinned host buffers; activations stream in twice (calibration and "
                                "re-propagation pass) and out once per step, copies overlap compute"},
                "gpu_launches": launches, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
                "phases_ms_per_step": {k: v / args.steps for k, v in phases.items()},
                "block_error_sum_per_layer": err_sum / args.steps, "wall_clock_s_timed_region": wall,
                "peaks": peaks["source"]}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of k_hessian_umma_pair on fp16
# X [T, C], from an ncu capture of exactly that launch (profiles/k_hessian_umma_pair_fp16.txt);
# the algorithmic bytes of the launch are T*C*2 + 2 * 4 * C*(C+256)/2 = 1.63e9.
HESSIAN_DRAM_BYTES = {(16384, 16384): 8895349504 + 552018432}


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
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
        run_ours(args)


if __name__ == "__main__":
    main()
