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
