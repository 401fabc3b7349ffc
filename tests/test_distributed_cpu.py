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


class _BilinearLattice:
    """CPU stand-in for the native wrapper with the same three operations on a bilinear toy model:
    features[n, 2l+f] = positions[n, 0] * values[l, 0, f].  Small enough to differentiate by hand,
    rich enough to have a second-order term through the position gradient."""

    def __init__(self):
        self.backward_hook = None
        self.double_backward_hook = None

    def forward(self, inp):
        return inp.m_positions_raw[:, :1] * inp.m_lattice_values.reshape(1, -1)

    def backward(self, inp, grad_features, lattice_grad_out=None, level_begin=None, level_end=None, zero=True,
                 positions_grad_out=None):
        v, x = inp.m_lattice_values, inp.m_positions_raw
        lb = 0 if level_begin is None else level_begin
        le = v.shape[0] if level_end is None else level_end
        lg = lattice_grad_out if lattice_grad_out is not None else torch.zeros_like(v)
        g = grad_features.reshape(x.shape[0], v.shape[0], 2)
        lg[lb:le, 0, :] = (x[:, :1, None] * g[:, lb:le, :]).sum(0)
        pg = None
        if inp.m_require_positions_grad:
            pg = positions_grad_out if positions_grad_out is not None else torch.zeros_like(x)
            pg[:, 0] += (g[:, lb:le, :] * v[None, lb:le, 0, :]).sum((1, 2))
        return (lg if inp.m_require_lattice_values_grad else None), pg

    def double_backward_from_positions(self, inp, dpg, grad_features, need_lattice_grad=True,
                                       need_grad_grad_features=True):
        v, x = inp.m_lattice_values, inp.m_positions_raw
        g = grad_features.reshape(x.shape[0], v.shape[0], 2)
        lg = (dpg[:, :1, None] * g).sum(0).reshape(v.shape) if need_lattice_grad else None
        ggf = (dpg[:, :1] * v.reshape(1, -1)) if need_grad_grad_features else None
        return lg, ggf


class _BilinearEncoding:
    def __init__(self, values):
        self.nr_levels = values.shape[0]
        self.lattice_values = values
        self.lattice = _BilinearLattice()


def _eikonal_grad(values, pos, w, hook_owner=None, n_total=None):
    """lattice_values.grad of mean((|d(F w)/dx| - 1)^2) + mean(F^2) through the package's two
    autograd Functions, on the toy lattice."""
    import permutohedral_encoding_b200.funcs as funcs

    class _Input:   # the Functions build EncodingInput through the native module: replace it for CPU tensors
        def __init__(self, lv, p, aw, a, b, half=None):
            self.m_lattice_values, self.m_positions_raw, self.m_anneal_window = lv, p, aw
            self.m_require_lattice_values_grad, self.m_require_positions_grad = bool(a), bool(b)

    real = funcs._C.EncodingInput
    funcs._C.EncodingInput = _Input
    try:
        enc = hook_owner if hook_owner is not None else _BilinearEncoding(values)
        x = pos.clone().requires_grad_(True)
        out = funcs.PermutoEncodingFunc.apply(enc.lattice, values, x, torch.ones(values.shape[0]), True, True)
        (g,) = torch.autograd.grad((out @ w).sum(), x, create_graph=True)
        n = n_total if n_total is not None else pos.shape[0]
        loss = ((g.norm(dim=1) - 1.0) ** 2).sum() / n + out.square().sum() / n
        loss.backward()
        return values.grad.clone()
    finally:
        funcs._C.EncodingInput = real


def _second_order_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from permutohedral_encoding_b200.distributed import LatticeGradAllReduce, shard_bounds
    gen = torch.Generator().manual_seed(11)
    L, n = 6, 40
    init = torch.randn(L, 1, 2, generator=gen)
    pos_all = torch.randn(n, 3, generator=gen)
    w = torch.randn(2 * L, generator=gen)
    full = _eikonal_grad(init.clone().requires_grad_(True), pos_all, w)          # whole batch, no hook
    values = init.clone().requires_grad_(True)
    enc = _BilinearEncoding(values)
    hook = LatticeGradAllReduce(enc, nr_buckets=2, multimem=False)
    b, e = shard_bounds(n, rank, world)
    sharded = _eikonal_grad(values, pos_all[b:e], w, hook_owner=enc, n_total=n)
    hook.remove()
    assert enc.lattice.backward_hook is None and enc.lattice.double_backward_hook is None
    torch.save({"full": full, "sharded": sharded}, os.path.join(out_dir, f"s{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_second_order_lattice_gradient_is_reduced_two_ranks(tmp_path):
    """Eikonal-style step on two gloo ranks: the lattice gradient from the double backward goes
    through the same sum over ranks as the first-order one, so every rank ends with the gradient
    of the whole batch."""
    port = _free_port()
    mp.spawn(_second_order_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    s0, s1 = torch.load(tmp_path / "s0.pt"), torch.load(tmp_path / "s1.pt")
    assert torch.allclose(s0["sharded"], s0["full"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(s1["sharded"], s0["full"], rtol=1e-5, atol=1e-6)
    assert torch.equal(s0["sharded"], s1["sharded"])
