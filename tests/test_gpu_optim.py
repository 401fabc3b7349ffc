"""The fused optimizer step on the lattice values (C ABI ``permuto_adam_step``) against the numpy
restatement in oracle/ and against ``torch.optim.AdamW`` on the same device.

Tolerance: rtol 1e-6 (+1e-7 absolute: the moments of O(1) gradients cancel) on parameters and moments (a handful of fp32 roundings differ: the kernel
multiplies by reciprocals where torch divides), with an absolute term of 1e-6 * lr for parameters
that are small against their update.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
REF = dict(lr=1e-3, betas=(0.9, 0.99), eps=1e-15, weight_decay=0.0)       # examples/performance.py:161
TOY = dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2)     # train_toy_example.py:30 (defaults)


@pytest.mark.parametrize("hyper", [REF, TOY])
@pytest.mark.parametrize("n", [1, 3, 4, 1023, 40000])
def test_adam_step_against_oracle(hyper, n):
    from oracle import adam_oracle
    from permutohedral_encoding_b200.optim import adam_step
    rng = np.random.default_rng(n)
    p = (rng.standard_normal(n) * 1e-4).astype(np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    tp, tm, tv = (torch.from_numpy(x.copy()).to(DEV) for x in (p, m, v))
    for step in range(1, 6):
        g = (rng.standard_normal(n) * (rng.random(n) < 0.7)).astype(np.float32)
        tg = torch.from_numpy(g).to(DEV)
        adam_step(tp, tg, tm, tv, step, hyper["lr"], hyper["betas"], hyper["eps"], hyper["weight_decay"])
        p, m, v = adam_oracle.adamw_step(p, g, m, v, step, hyper["lr"], *hyper["betas"], hyper["eps"],
                                         hyper["weight_decay"])
        np.testing.assert_allclose(tp.cpu().numpy(), p, rtol=1e-6, atol=1e-6 * hyper["lr"])
        np.testing.assert_allclose(tm.cpu().numpy(), m, rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(tv.cpu().numpy(), v, rtol=1e-6, atol=1e-7)
        assert torch.equal(tg.cpu(), torch.from_numpy(g))      # the gradient is left alone by default


@pytest.mark.parametrize("hyper", [REF, TOY])
def test_lattice_adamw_matches_torch_adamw_on_a_table(hyper):
    """Same trajectory as torch.optim.AdamW over a [L, C, 2] table with sparse gradients; skipping
    untouched slots and clearing the gradient in the step do not change it."""
    from permutohedral_encoding_b200.optim import LatticeAdamW
    gen = torch.Generator(device="cpu").manual_seed(1)
    init = (torch.randn((6, 4096, 2), generator=gen) * 1e-5).to(DEV)
    a = torch.nn.Parameter(init.clone())
    b = torch.nn.Parameter(init.clone())
    c = torch.nn.Parameter(init.clone())
    opt_a = torch.optim.AdamW([a], **hyper)
    opt_b = LatticeAdamW([b], **hyper)
    opt_c = LatticeAdamW([c], skip_untouched=True, zero_grad_in_step=True, **hyper)
    for _ in range(6):
        g = torch.randn((6, 4096, 2), generator=gen)
        g[3:] *= (torch.rand((3, 4096, 1), generator=gen) < 0.05)   # fine levels: few slots touched
        g[5] = 0
        g = g.to(DEV)
        for prm in (a, b, c):
            prm.grad = g.clone()
        opt_a.step(), opt_b.step(), opt_c.step()
        assert torch.count_nonzero(c.grad) == 0 and torch.equal(b.grad, g)
    for prm in (b, c):
        np.testing.assert_allclose(prm.detach().cpu().numpy(), a.detach().cpu().numpy(), rtol=1e-6,
                                   atol=1e-6 * hyper["lr"])
    sa, sb = opt_a.state[a], opt_b.state[b]
    np.testing.assert_allclose(sb["exp_avg"].cpu().numpy(), sa["exp_avg"].cpu().numpy(), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(sb["exp_avg_sq"].cpu().numpy(), sa["exp_avg_sq"].cpu().numpy(), rtol=1e-6, atol=1e-7)
    if hyper["weight_decay"] == 0.0:
        assert torch.equal(c[5], init[5])                     # never touched: bit-identical


def test_adam_rejects_bad_arguments():
    from permutohedral_encoding_b200 import _native as nat
    from permutohedral_encoding_b200.optim import LatticeAdamW, adam_step
    t = torch.zeros(16, device=DEV)
    with pytest.raises(RuntimeError, match="step counts from 1"):
        adam_step(t, t.clone(), t.clone(), t.clone(), 0, 1e-3)
    with pytest.raises(RuntimeError, match="GPU memory"):
        adam_step(torch.zeros(4), torch.zeros(4), torch.zeros(4), torch.zeros(4), 1, 1e-3)
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        big = torch.zeros(32, device=DEV)
        adam_step(big[1:17], t.clone(), t.clone(), t.clone(), 1, 1e-3)
    assert nat.lib.permuto_adam_step(None, None, None, None, 4, 1e-3, 0.9, 0.99, 1e-8, 0.0, 1, 0, None) \
        == nat.PERMUTO_ERR_INVALID_ARGUMENT
    with pytest.raises(ValueError):
        LatticeAdamW([torch.nn.Parameter(t.clone())], amsgrad=True)


def test_training_loop_with_the_fused_step_reduces_the_loss():
    """The reference's performance-script loop (loss = mean((pred - 10)^2), optimizer step on the
    table) with the fused optimizer."""
    from permutohedral_encoding_b200 import PermutoEncoding
    from permutohedral_encoding_b200.optim import LatticeAdamW
    torch.manual_seed(0)
    m = PermutoEncoding(3, 2 ** 14, 8, 2, np.geomspace(1.0, 1e-2, 8))
    opt = LatticeAdamW([m.lattice_values], lr=2e-1, betas=(0.9, 0.99), eps=1e-15, weight_decay=0.0,
                       skip_untouched=True)
    pts = torch.rand(5000, 3, device=DEV) - 0.5
    losses = []
    for _ in range(100):
        loss = ((m(pts) - 10) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.1 * losses[0], (losses[0], losses[-1])
