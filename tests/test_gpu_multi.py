"""Two-GPU check of the data-parallel path: points sharded, lattice replicated, lattice gradient
all-reduced bucket by bucket while backward is still running.  Skipped with fewer than 2 GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir, use_multimem, copy_out, clear):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from permutohedral_encoding_b200 import PermutoEncoding
    from permutohedral_encoding_b200.distributed import LatticeGradAllReduce, shard_bounds
    d, cap, nl, n = 3, 2 ** 16, 12, 50001
    gen = torch.Generator().manual_seed(5)
    table = (torch.rand((nl, cap, 2), generator=gen) * 2 - 1).to(dev)
    shift = (torch.randn((nl, d), generator=gen) * 10).to(dev)
    pos_all = torch.rand((n, d), generator=gen).to(dev)
    go_all = torch.randn((n, 2 * nl), generator=gen).to(dev)
    torch.manual_seed(0)
    m = PermutoEncoding(d, cap, nl, 2, np.geomspace(1.0, 1e-3, nl))
    with torch.no_grad():
        m.lattice_values.copy_(table)
        m.random_shift_per_level.copy_(shift)
    # the whole batch on this GPU alone
    pos = pos_all.clone().requires_grad_(True)
    out_full = m(pos)
    out_full.backward(go_all)
    full_tg, full_pg = m.lattice_values.grad.clone(), pos.grad.clone()
    m.lattice_values.grad = None
    # this rank's shard with the bucketed all-reduce
    hook = LatticeGradAllReduce(m, nr_buckets=3, multimem=use_multimem, copy_out=copy_out, clear=clear)
    b, e = shard_bounds(n, rank, world)
    pos_s = pos_all[b:e].clone().requires_grad_(True)
    out_s = m(pos_s)
    out_s.backward(go_all[b:e])
    torch.cuda.synchronize()
    lvl = full_tg.abs().amax(dim=(1, 2), keepdim=True)
    ok_tg = bool(torch.all((m.lattice_values.grad - full_tg).abs() <= 1e-4 * lvl))
    ok_out = bool(torch.equal(out_s, out_full[b:e]))
    ok_pg = bool(torch.all((pos_s.grad - full_pg[b:e]).abs() <= 1e-4 * full_pg.abs().max()))
    # gradient accumulation: a second backward without clearing .grad doubles it (the buffer that
    # .grad aliases is never the one the next backward writes)
    out_s2 = m(pos_all[b:e])
    out_s2.backward(go_all[b:e])
    torch.cuda.synchronize()
    ok_acc = bool(torch.all((m.lattice_values.grad - 2 * full_tg).abs() <= 2e-4 * lvl))
    # eikonal step: the second-order lattice gradient is summed over the ranks too
    w = torch.randn(2 * nl, generator=gen).to(dev) * 0.2

    def eikonal(points, n_total):
        m.lattice_values.grad = None
        x = points.clone().requires_grad_(True)
        y = m(x)
        (g,) = torch.autograd.grad((y @ w).sum(), x, create_graph=True)
        (((g.norm(dim=1) - 1.0) ** 2).sum() / n_total + y.square().sum() / n_total).backward()
        torch.cuda.synchronize()
        return m.lattice_values.grad.clone()

    sharded_e = eikonal(pos_all[b:e], n)
    hook.remove()
    full_e = eikonal(pos_all, n)
    lvl_e = full_e.abs().amax(dim=(1, 2), keepdim=True)
    ok_eik = bool(torch.all((sharded_e - full_e).abs() <= 2e-4 * lvl_e))
    torch.save({"ok": (ok_tg, ok_out, ok_pg, ok_acc, ok_eik)}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("use_multimem,copy_out,clear", [(False, False, "inline"), ("auto", False, "inline"),
                                                         ("auto", True, "inline"), ("auto", False, "early")])
def test_sharded_step_matches_single_gpu(tmp_path, use_multimem, copy_out, clear):
    """First-order step, gradient accumulation and an eikonal (double-backward) step on two ranks
    against the same batch on one GPU; NCCL all-reduce and the in-switch (multimem) path, the
    latter handing out views of its buffers, copies, and with the early clearing."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path), use_multimem, copy_out, clear), nprocs=2, join=True)
    for r in range(2):
        assert torch.load(tmp_path / f"r{r}.pt")["ok"] == (True, True, True, True, True)


def test_module_on_a_device_that_is_not_current():
    """The reference pins cuda:0; here an encoding lives on whatever device its parameters are on,
    also when another device is current on the calling thread."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    sys.path.insert(0, ROOT)
    from permutohedral_encoding_b200 import PermutoEncoding
    sig = np.geomspace(1.0, 1e-2, 8)
    torch.manual_seed(3)
    with torch.cuda.device(0):
        m0 = PermutoEncoding(3, 2 ** 12, 8, 2, sig)
    pos = torch.rand(5000, 3)
    go = torch.randn(5000, 16)
    out0 = m0(pos.cuda(0))
    out0.backward(go.cuda(0))
    m1 = PermutoEncoding(3, 2 ** 12, 8, 2, sig)
    m1.load_state_dict(m0.state_dict())
    m1 = m1.to("cuda:1")
    torch.cuda.set_device(0)                       # cuda:0 stays current while cuda:1 is used
    out1 = m1(pos.to("cuda:1"))
    out1.backward(go.to("cuda:1"))
    assert out1.device.index == 1 and m1.lattice_values.grad.device.index == 1
    assert torch.equal(out1.cpu(), out0.cpu())
    lvl = m0.lattice_values.grad.abs().amax(dim=(1, 2), keepdim=True).cpu()
    assert torch.all((m1.lattice_values.grad.cpu() - m0.lattice_values.grad.cpu()).abs() <= 1e-4 * lvl + 1e-12)
