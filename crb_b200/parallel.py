"""Sharding of the calibration path across the GPUs of one box (one process per GPU).

Two independent splits, neither of which exists in the single-device reference:

* calibration sequences are split across ranks; each rank accumulates an unscaled partial
  S_r = sum X^T X over its sequences and the partials are summed with one all-reduce per
  distinct layer input (H is a sum over sequences, bigptq.py:50-53);
* the linears of a decoder layer are independent problems once their Hessians exist (all
  hooks see the layer's original weights, run.py:341-353), so each linear is quantized by
  one owner rank and the result is broadcast.

Everything here is host logic on top of torch.distributed and is backend-agnostic (NCCL on
GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def world() -> Tuple[int, int]:
    """(rank, world_size); (0, 1) outside a process group."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_range(n: int, rank: int, world_size: int, sizes: Optional[Sequence[int]] = None) -> range:
    """Contiguous slice of range(n) owned by `rank`: `sizes[r]` items for rank r, or a balanced split
    (the first n % world ranks get one more) when no sizes are given."""
    if sizes is not None:
        if len(sizes) != world_size or sum(sizes) != n or min(sizes) < 0:
            raise ValueError(f"shard sizes {list(sizes)} do not partition {n} items over {world_size} ranks")
        start = sum(sizes[:rank])
        return range(start, start + sizes[rank])
    base, extra = divmod(n, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def linear_cost(rows: int, cols: int) -> float:
    """Seconds one linear takes on a B200 (fitted to measurements, used only to balance ranks).

    Factorisation: products at the split-TF32 GEMM rate (~ cols^3) plus the serial chain of diagonal
    blocks (~ cols): 2.7 ms at 4096 columns, 25.6 ms at 16384.  Block loop: per 128-column block a
    chain of dependent kernels (61 us + 15.4 ns per row) plus the trailing updates (~ rows * cols^2
    at the same GEMM rate)."""
    factor = 3.57e-15 * cols ** 3 + 6.04e-7 * cols
    blocks = (cols / 128) * (6.1e-5 + 1.54e-8 * rows) + rows * cols ** 2 / 1.9e14
    return factor + blocks


def assign_owners(shapes: Dict[str, Tuple[int, int]], world_size: int) -> Dict[str, int]:
    """Greedy longest-processing-time assignment of linears to ranks; deterministic on every rank."""
    load = [0.0] * world_size
    owners: Dict[str, int] = {}
    for name in sorted(shapes, key=lambda n: (-linear_cost(*shapes[n]), n)):
        r = min(range(world_size), key=lambda k: (load[k], k))
        owners[name] = r
        load[r] += linear_cost(*shapes[name])
    return owners


def plan_shards(n: int, world_size: int, shapes: Optional[Dict[str, Tuple[int, int]]] = None,
                skew: bool = True) -> List[int]:
    """Calibration sequences per rank.

    Balanced, unless one linear dominates: when the layer's LAST linear (`shapes` lists the linears
    in the order the layer calls them) is also its most expensive one and its owner would be busy
    for more than 1.5 times as long as any other rank, that owner is the critical path of every
    layer: the other ranks sit idle while it quantizes and can run the second pass of their
    sequences up to that last linear in the meantime (`reprop_overlap` in run.quantize_layer), but
    the owner can only start its own second pass afterwards.  So the owner gets fewer sequences:
    as many as it can re-propagate in the time the others need for the remaining part of theirs
    (the last linear's share of the forward work).  Needs three ranks or more: with two, what the
    single other rank loses in the first pass outweighs what the owner gains."""
    even = [len(shard_range(n, r, world_size)) for r in range(world_size)]
    if not skew or world_size < 3 or not shapes or n < 2 * world_size:
        return even
    names = list(shapes)
    last = names[-1]
    cost = {k: linear_cost(*shapes[k]) for k in names}
    if cost[last] < max(cost.values()):
        return even
    owners = assign_owners(shapes, world_size)
    load = [0.0] * world_size
    for k in names:
        load[owners[k]] += cost[k]
    heavy = owners[last]
    if load[heavy] < 1.5 * max(v for r, v in enumerate(load) if r != heavy):
        return even
    work = {k: float(shapes[k][0]) * shapes[k][1] for k in names}
    tail = work[last] / sum(work.values())
    mine = min(even[heavy], int(n * tail / (world_size - 1 + tail)) + 2)      # + 2: the weight broadcast
    sizes = [len(shard_range(n - mine, r, world_size - 1)) for r in range(world_size - 1)]
    sizes.insert(heavy, mine)
    return sizes


def allreduce_sum_(tensors: Sequence[torch.Tensor]) -> None:
    """In-place sum over ranks of every tensor in the list (no-op for a single rank)."""
    _, ws = world()
    if ws == 1:
        return
    handles = [dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=True) for t in tensors]
    for h in handles:
        h.wait()


def allreduce_hessians_(sums: Sequence[torch.Tensor]) -> None:
    """In-place sum over ranks of partial Hessian sums S [C, C] as `ops.hessian_accumulate` keeps them.

    On CUDA only the maintained part of each S (its 256 x 256 tiles on and above the diagonal) is
    summed: all of them are packed into one buffer, reduced with a single all-reduce and unpacked,
    which moves about half the bytes of the full matrices.  CPU tensors (the gloo tests) take the
    plain route."""
    _, ws = world()
    if ws == 1 or not sums:
        return
    if not all(t.is_cuda and t.dim() == 2 and t.shape[0] == t.shape[1] and t.is_contiguous() for t in sums):
        allreduce_sum_(sums)
        return
    from . import ops
    sizes = [ops.hessian_packed_floats(t.shape[0]) for t in sums]
    buf = torch.empty(sum(sizes), dtype=torch.float32, device=sums[0].device)
    off = 0
    for t, n in zip(sums, sizes):
        ops.hessian_pack(t, buf[off:off + n])
        off += n
    dist.all_reduce(buf, op=dist.ReduceOp.SUM)
    off = 0
    for t, n in zip(sums, sizes):
        ops.hessian_unpack(buf[off:off + n], t)
        off += n


def broadcast_(tensor: torch.Tensor, src: int, group=None) -> None:
    _, ws = world()
    if ws > 1:
        dist.broadcast(tensor, src=src, group=group)


_WEIGHTS_GROUP = None


def weights_group():
    """A process group of all ranks used only for streaming layer weights in (run._Resident): its
    collectives have their own communicator, so a weight broadcast that waits for a copy from host
    memory never holds up the Hessian all-reduce or the broadcast of a finished linear.  Created on
    first use; every rank reaches that point in the same program order."""
    global _WEIGHTS_GROUP
    _, ws = world()
    if ws == 1:
        return None
    if _WEIGHTS_GROUP is None:
        _WEIGHTS_GROUP = dist.new_group()
    return _WEIGHTS_GROUP


def max_over_ranks(value: float, device) -> float:
    _, ws = world()
    if ws == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device) -> float:
    _, ws = world()
    if ws == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
