"""The multi-rank path on CPU: two gloo ranks.

Covers the host logic that the GPU runs rely on at N > 1: sequence sharding, summation of the
partial Hessians, owner assignment, weight broadcast and re-propagation on each rank's shard.
The CUDA kernels cannot run here, so `BRAGPTQ` is replaced by a CPU stand-in built on the
oracle; what is tested is the plumbing of `crb_b200.run.quantize_layer`, not the arithmetic.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from crb_b200 import parallel


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_range_partitions_the_sequences():
    for n in (1, 7, 128, 130):
        for ws in (1, 2, 3, 8):
            parts = [list(parallel.shard_range(n, r, ws)) for r in range(ws)]
            assert sum(parts, []) == list(range(n))
            assert max(map(len, parts)) - min(map(len, parts)) <= 1


def test_sized_shards_and_the_plan_for_a_dominant_last_linear():
    assert [list(parallel.shard_range(7, r, 3, [1, 4, 2])) for r in range(3)] == [[0], [1, 2, 3, 4], [5, 6]]
    with pytest.raises(ValueError):
        parallel.shard_range(7, 0, 3, [1, 4, 1])
    opt = {"self_attn.k_proj": (4096, 4096), "self_attn.v_proj": (4096, 4096), "self_attn.q_proj": (4096, 4096),
           "self_attn.out_proj": (4096, 4096), "fc1": (16384, 4096), "fc2": (4096, 16384)}
    # one or two ranks, no shapes, or skew switched off: balanced
    assert parallel.plan_shards(128, 1, opt) == [128]
    assert parallel.plan_shards(128, 2, opt) == [64, 64]
    assert parallel.plan_shards(128, 8, None) == [16] * 8
    assert parallel.plan_shards(128, 8, opt, skew=False) == [16] * 8
    # fc2 is the last and by far the most expensive linear: its owner (rank 0) gets about a third of
    # what the others get (fc2 is a third of the layer's forward work), the rest is balanced
    for ws in (3, 4, 8):
        sizes = parallel.plan_shards(128, ws, opt)
        heavy = parallel.assign_owners(opt, ws)["fc2"]
        assert sum(sizes) == 128 and len(sizes) == ws
        others = [v for r, v in enumerate(sizes) if r != heavy]
        assert max(others) - min(others) <= 1
        assert others[0] / 3 <= sizes[heavy] <= others[0] / 3 + 3
    # the last linear is not the most expensive one: balanced
    flat = {"a": (4096, 16384), "b": (4096, 4096)}
    assert parallel.plan_shards(128, 4, flat) == [32] * 4
    # too few sequences to skew
    assert parallel.plan_shards(6, 4, opt) == [2, 2, 1, 1]


def test_owner_assignment_is_deterministic_and_balanced():
    shapes = {"self_attn.q_proj": (4096, 4096), "self_attn.k_proj": (4096, 4096), "self_attn.v_proj": (4096, 4096),
              "self_attn.out_proj": (4096, 4096), "fc1": (16384, 4096), "fc2": (4096, 16384)}
    a = parallel.assign_owners(shapes, 8)
    assert a == parallel.assign_owners(dict(reversed(list(shapes.items()))), 8)
    assert len(set(a.values())) == 6                      # six linears on six different ranks
    b = parallel.assign_owners(shapes, 2)
    assert set(b.values()) == {0, 1}
    assert all(v == 0 for v in parallel.assign_owners(shapes, 1).values())
    # the most expensive linear (largest in_features) sits alone on its rank when there is room
    assert list(a.values()).count(a["fc2"]) == 1


class _CpuGptq:
    """Interface of crb_b200.BRAGPTQ on CPU tensors, arithmetic by the oracle (test stand-in)."""

    def __init__(self, layer, quantizer, salient_metric, disable_gptq=False):
        self.layer, self.q = layer, quantizer
        self.rows, self.columns = layer.weight.shape
        self._S = torch.zeros(self.columns, self.columns)
        self.nsamples = 0
        self.last_timing = {}
        self.verbose = False

    def add_batch(self, inp, out=None):
        x = inp.reshape(-1, inp.shape[-1]).float()
        self._S += x.t() @ x
        self.nsamples += inp.shape[0] if inp.dim() == 3 else 1

    def fasterquant(self, **kw):
        from oracle import crb_oracle as O
        H = self._S * (2.0 / self.nsamples)
        res = O.quantize_linear(self.layer.weight.data.float(), H, self.q.method, keep_blocks=False,
                                percdamp=kw.get("percdamp", 0.01))
        self.layer.weight.data = res.W.to(self.layer.weight.dtype)
        return {"error": res.error}

    def free(self):
        self._S = None


def _worker(rank, world, port, result_path, shard_sizes=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from crb_b200 import run as crun
    from crb_b200.synth import build_synthetic_model, synthetic_calibration
    crun.BRAGPTQ = _CpuGptq
    model = build_synthetic_model("opt-tiny", n_layers=1, seed=3).float()
    model.seqlen = 64
    loader = synthetic_calibration(model.config.vocab_size, nsamples=8, seqlen=64, seed=1)
    args = crun.default_args(low_quant_method="braq", nsamples=8, forward_batch=2, verbose=False, device="cpu")
    args.percdamp = 0.1          # few calibration tokens: keep the tiny Hessians well conditioned
    args.shard_sizes = shard_sizes
    out = crun.quant_sequential(model, loader, "cpu", args)
    layer = model.model.decoder.layers[0]
    weights = {n: m.weight.data.clone() for n, m in crun.find_layers(layer).items()}
    hidden = out["final_hidden"]
    if world > 1:
        # shards may differ in size: gather through a buffer of the largest one
        n_max = int(parallel.max_over_ranks(float(hidden.shape[0]), "cpu"))
        padded = torch.zeros((n_max,) + tuple(hidden.shape[1:]), dtype=hidden.dtype)
        padded[:hidden.shape[0]] = hidden
        gathered = [torch.zeros_like(padded) for _ in range(world)]
        dist.all_gather(gathered, padded)
        sizes = shard_sizes or [len(parallel.shard_range(8, r, world)) for r in range(world)]
        hidden = torch.cat([g[:k] for g, k in zip(gathered, sizes)], 0)
    errors = {n: parallel.sum_over_ranks(e, "cpu") for n, e in out["errors"][0].items()}
    if rank == 0:
        torch.save({"weights": weights, "hidden": hidden, "error_sum": out["error_sum"],
                    "errors": errors}, result_path)
    if world > 1:
        # every rank must hold the same quantized weights after the broadcast
        for n, w in weights.items():
            ref = w.clone()
            dist.broadcast(ref, src=0)
            assert torch.equal(ref, w), n
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_ranks_reproduce_the_single_rank_run(tmp_path):
    single, double = str(tmp_path / "w1.pt"), str(tmp_path / "w2.pt")
    mp.spawn(_worker, args=(1, _free_port(), single), nprocs=1, join=True)
    mp.spawn(_worker, args=(2, _free_port(), double), nprocs=2, join=True)
    a, b = torch.load(single), torch.load(double)
    # partial Hessians are summed in a different order, so allow rounding-level differences
    assert abs(a["error_sum"] - b["error_sum"]) <= 2e-3 * abs(a["error_sum"])
    assert set(a["errors"]) == set(b["errors"]) and len(a["errors"]) == 6
    for n in a["errors"]:
        # every linear was quantized exactly once, on its owner, from the full (summed) Hessian:
        # a missing all-reduce or a wrong sample count would move these by a factor, not by rounding
        assert abs(a["errors"][n] - b["errors"][n]) <= 2e-2 * abs(a["errors"][n]), (n, a["errors"][n], b["errors"][n])
    assert a["hidden"].shape == b["hidden"].shape
    rel = (a["hidden"] - b["hidden"]).norm() / a["hidden"].norm()
    assert rel < 0.05, float(rel)


@pytest.mark.timeout(600)
def test_three_ranks_with_uneven_shards_reproduce_the_single_rank_run(tmp_path):
    single, triple = str(tmp_path / "w1.pt"), str(tmp_path / "w3.pt")
    mp.spawn(_worker, args=(1, _free_port(), single), nprocs=1, join=True)
    mp.spawn(_worker, args=(3, _free_port(), triple, [1, 4, 3]), nprocs=3, join=True)
    a, b = torch.load(single), torch.load(triple)
    assert abs(a["error_sum"] - b["error_sum"]) <= 2e-3 * abs(a["error_sum"])
    for n in a["errors"]:
        assert abs(a["errors"][n] - b["errors"][n]) <= 2e-2 * abs(a["errors"][n]), (n, a["errors"][n], b["errors"][n])
    assert a["hidden"].shape == b["hidden"].shape
    rel = (a["hidden"] - b["hidden"]).norm() / a["hidden"].norm()
    assert rel < 0.05, float(rel)


def _collectives(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    X = torch.randn(64, 16, generator=g)
    mine = parallel.shard_range(64, rank, world)
    S = X[mine.start:mine.stop].t() @ X[mine.start:mine.stop]
    extra = torch.full((3,), float(rank + 1))
    parallel.allreduce_sum_([S, extra])
    assert torch.allclose(S, X.t() @ X, rtol=1e-5, atol=1e-5)
    assert torch.equal(extra, torch.full((3,), 3.0))
    w = torch.full((4,), float(rank))
    parallel.broadcast_(w, src=1)
    assert torch.equal(w, torch.ones(4))
    assert parallel.max_over_ranks(float(rank), "cpu") == 1.0
    assert parallel.sum_over_ranks(2.0, "cpu") == 4.0
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_collective_helpers_on_two_gloo_ranks():
    mp.spawn(_collectives, args=(2, _free_port()), nprocs=2, join=True)
