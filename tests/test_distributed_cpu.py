"""World-size-2 gloo test of the multi-GPU host logic: contiguous point sharding and the
bucketed all-reduce of a per-level gradient.  No GPU involved."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from permutohedral_encoding_b200.distributed import all_reduce_bucketed, level_buckets, shard_bounds
    n_total, nl = 1001, 10
    b, e = shard_bounds(n_total, rank, world)
    gen = torch.Generator().manual_seed(7)
    contrib = torch.randn(n_total, nl, 16, 2, generator=gen)   # same on every rank
    local = contrib[b:e].sum(0)                                 # this rank's partial "table gradient"
    all_reduce_bucketed(local, level_buckets(nl, 3))
    torch.save({"sum": local, "bounds": (b, e), "full": contrib.sum(0)}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds_cover_exactly():
    from permutohedral_encoding_b200.distributed import shard_bounds
    for n in (1, 7, 8, 1000, 2 ** 24):
        for w in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(10, 3, 3)


def test_level_buckets():
    from permutohedral_encoding_b200.distributed import level_buckets
    assert level_buckets(24, 3, "even") == [(0, 8), (8, 16), (16, 24)]
    assert level_buckets(24, 3) == [(0, 12), (12, 20), (20, 24)]
    assert level_buckets(24, 2) == [(0, 16), (16, 24)]
    assert level_buckets(24, 1) == [(0, 24)]
    assert level_buckets(10, 8) == [(0, 4), (4, 8), (8, 10)]
    assert level_buckets(3, 2) == [(0, 3)]
    with pytest.raises(ValueError):
        level_buckets(8, 2, "nope")
    for nl in range(1, 40):
        for nb in range(1, 9):
          for pol in ("halving", "even"):
            bk = level_buckets(nl, nb, pol)
            assert bk[0][0] == 0 and bk[-1][1] == nl
            assert all(a[1] == b[0] for a, b in zip(bk, bk[1:]))
            assert all(a % 4 == 0 for a, _ in bk)


def test_bucketed_allreduce_two_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "r0.pt")
    r1 = torch.load(tmp_path / "r1.pt")
    assert r0["bounds"] == (0, 501) and r1["bounds"] == (501, 1001)
    assert torch.equal(r0["sum"], r1["sum"])
    assert torch.allclose(r0["sum"], r0["full"], rtol=1e-4, atol=1e-4)


class _FakeLattice:
    """Stands in for the native wrapper on CPU: fills the requested level range of the gradient
    buffer with a rank-dependent pattern, like a backward over that bucket would."""

    def __init__(self, rank):
        self.rank, self.calls, self.backward_hook = rank, [], None

    def backward(self, input_struct, grad_features, lattice_grad_out=None, level_begin=None, level_end=None, zero=True,
                 positions_grad_out=None):
        self.calls.append((level_begin, level_end))
        lattice_grad_out[level_begin:level_end] = float(self.rank + 1) * (1 + torch.arange(level_begin, level_end)
                                                                          ).view(-1, 1, 1).float()
        return lattice_grad_out, None


class _FakeEncoding:
    def __init__(self, rank, nr_levels):
        self.nr_levels = nr_levels
        self.lattice = _FakeLattice(rank)
        self.lattice_values = torch.zeros(nr_levels, 8, 2)


class _FakeInput:
    def __init__(self, values):
        self.m_lattice_values = values


def _hook_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from permutohedral_encoding_b200.distributed import LatticeGradAllReduce
    enc = _FakeEncoding(rank, 10)
    hook = LatticeGradAllReduce(enc, nr_buckets=3, average=True, multimem="auto")   # gloo: falls back to all_reduce
    assert hook._symm is None and enc.lattice.backward_hook is not None
    grad, pos_grad = enc.lattice.backward_hook(enc.lattice, _FakeInput(enc.lattice_values), None)
    torch.save({"grad": grad, "calls": enc.lattice.calls, "pos": pos_grad}, os.path.join(out_dir, f"h{rank}.pt"))
    hook.remove()
    assert enc.lattice.backward_hook is None
    dist.barrier()
    dist.destroy_process_group()


def test_gradient_hook_buckets_and_averages_two_ranks(tmp_path):
    """The backward hook of the data-parallel helper on two gloo ranks with a stand-in for the
    native backward: one call per bucket, bucket-wise all-reduce, mean over ranks."""
    port = _free_port()
    mp.spawn(_hook_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    h0, h1 = torch.load(tmp_path / "h0.pt"), torch.load(tmp_path / "h1.pt")
    assert h0["calls"] == [(0, 4), (4, 8), (8, 10)] and h0["pos"] is None
    want = 1.5 * (1 + torch.arange(10)).view(-1, 1, 1).float().expand(10, 8, 2)   # mean of 1x and 2x
    assert torch.equal(h0["grad"], h1["grad"]) and torch.allclose(h0["grad"], want)
