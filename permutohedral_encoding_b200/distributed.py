"""Data-parallel use of the encoding on the GPUs of one box: points are sharded, the lattice
is replicated, and the only exchange is the all-reduce (sum) of the lattice-value gradient.

The reference has no distributed code (it pins every allocation to cuda:0); this module is the
multi-GPU row of the hot path.  One process per GPU, ``torch.distributed`` for the plumbing
(NCCL over NVLink/NVSwitch on GPUs; gloo works for CPU tests of the host logic).

Overlap: the backward kernel runs level group by level group, so the gradient of the first
levels is final long before the last levels are done.  ``LatticeGradAllReduce`` splits the
levels into buckets, launches the backward of one bucket, then starts that bucket's
all-reduce asynchronously while the next bucket's backward runs; only the last bucket's
all-reduce is exposed.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(nr_positions: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous, even split of ``nr_positions`` points: rank r owns [begin, end).  The first
    ``nr_positions % world_size`` ranks own one point more."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} / world_size {world_size}")
    base, rem = divmod(int(nr_positions), int(world_size))
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def level_buckets(nr_levels: int, nr_buckets: int, policy: str = "halving") -> List[Tuple[int, int]]:
    """Split levels into at most ``nr_buckets`` contiguous buckets whose boundaries are multiples
    of 4 levels (the kernels' level-group size), coarse levels first.

    ``policy="halving"`` (default) makes every bucket about half as long as the one before: the
    all-reduce of a bucket overlaps the backward of the remaining, shorter buckets, and only the
    last, smallest bucket's all-reduce is exposed, while most levels still run in one long sweep
    (long sweeps are the efficient ones).  ``policy="even"`` gives equal buckets."""
    groups = (nr_levels + 3) // 4
    nr_buckets = max(1, min(int(nr_buckets), groups))
    if policy == "even":
        sizes = [groups // nr_buckets + (1 if b < groups % nr_buckets else 0) for b in range(nr_buckets)]
    elif policy == "halving":
        weights = [2.0 ** (nr_buckets - 1 - b) for b in range(nr_buckets)]
        total = sum(weights)
        sizes = [1] * nr_buckets                       # every bucket gets at least one group
        spare = groups - nr_buckets
        ideal = [w / total * groups for w in weights]
        for _ in range(spare):                         # hand out the rest by largest deficit
            b = max(range(nr_buckets), key=lambda i: (ideal[i] - sizes[i], -i))
            sizes[b] += 1
    else:
        raise ValueError(f"unknown bucket policy {policy!r}")
    out, g0 = [], 0
    for sz in sizes:
        out.append((g0 * 4, min((g0 + sz) * 4, nr_levels)))
        g0 += sz
    return [(a, b) for a, b in out if b > a]


class LatticeGradAllReduce:
    """Installs a backward hook on a ``PermutoEncoding`` that computes the lattice gradient in
    level buckets and all-reduces each bucket while the next one is being computed.

    After ``loss.backward()`` the parameter's ``.grad`` holds the sum over ranks (or the mean
    with ``average=True``).  Call ``remove()`` to restore single-GPU behaviour."""

    def __init__(self, encoding, process_group=None, nr_buckets: int = 3, average: bool = False,
                 policy: str = "halving"):
        self.encoding = encoding
        self.group = process_group
        self.average = average
        self.buckets = level_buckets(encoding.nr_levels, nr_buckets, policy)
        encoding.lattice.backward_hook = self._backward
        self.last_works = []

    def remove(self) -> None:
        self.encoding.lattice.backward_hook = None

    def _backward(self, lattice, input_struct, grad_features):
        lv_grad = torch.empty_like(input_struct.m_lattice_values)
        pos_grad = None
        works = []
        for i, (l0, l1) in enumerate(self.buckets):
            _, pg = lattice.backward(input_struct, grad_features, lattice_grad_out=lv_grad, level_begin=l0,
                                     level_end=l1, zero=True, positions_grad_out=pos_grad)
            pos_grad = pg if pg is not None else pos_grad
            # async_op: the collective's stream waits for the kernels enqueued so far and runs
            # beside the next bucket's backward
            works.append(dist.all_reduce(lv_grad[l0:l1], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        for w in works:
            w.wait()
        if self.average:
            lv_grad.div_(dist.get_world_size(self.group))
        self.last_works = works
        return lv_grad, pos_grad


def all_reduce_bucketed(tensor_by_level: torch.Tensor, buckets, group=None) -> None:
    """All-reduce (sum) a ``[L, ...]`` tensor bucket by bucket; host-logic helper shared with
    the CPU tests."""
    works = [dist.all_reduce(tensor_by_level[a:b], op=dist.ReduceOp.SUM, group=group, async_op=True)
             for a, b in buckets]
    for w in works:
        w.wait()
