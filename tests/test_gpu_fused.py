"""Forward fused with the consumer's first linear layer (C ABI ``permuto_forward_linear``: features
stay in shared memory, the product runs on the tensor cores with tcgen05.mma, accumulator in
tensor memory) against the oracle's features followed by an exact (float64) matrix product.

Tolerance: both operands are rounded to tf32 (10-bit mantissa, round to nearest: relative error
2^-11 each) and accumulated in fp32, so every output must lie within 2e-3 * sum_k |feature_k *
weight_k| of the exact product (+1e-6 of the largest output for sums that cancel).
"""
import numpy as np
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
DEV = "cuda"
TF32_RTOL = 2e-3


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.fixture(scope="module")
def nat():
    from permutohedral_encoding_b200 import _native
    assert torch.cuda.is_available()
    return _native


CASES = {
    # the reference's usage: 24 levels x 2 features into Linear(48, 32) (examples/train_toy_example.py:18-19)
    "toy_mlp": dict(pos_dim=3, capacity=2 ** 16, nr_levels=24, sigma=(1.0, 1e-4), n=5000, box=(0.0, 1.0), table=1.0, h=32, bias=True),
    "wide_64": dict(pos_dim=3, capacity=2 ** 14, nr_levels=24, sigma=(1.0, 1e-3), n=128 * 9, box=(-1.0, 1.0), table=1.0, h=64, bias=False),
    # row width 14 + 4 concat columns = 18 -> padded to 24 columns; odd point count; non-power-of-two capacity
    "padded_concat": dict(pos_dim=4, capacity=30011, nr_levels=7, sigma=(1.0, 1e-2), n=1001, box=(-1.0, 1.0), table=1.0,
                          h=16, bias=True, concat=True, points_scaling=0.5),
    "window": dict(pos_dim=2, capacity=2 ** 12, nr_levels=12, sigma=(1.0, 1e-2), n=777, box=(0.0, 1.0), table=1.0, h=48,
                   bias=True, window_t=0.6),
    "feat4": dict(pos_dim=3, capacity=2 ** 14, nr_levels=12, sigma=(1.0, 1e-3), n=3000, box=(0.0, 1.0), table=1.0, h=32,
                  bias=True, feat=4),
    "feat8_d6": dict(pos_dim=6, capacity=2 ** 14, nr_levels=6, sigma=(1.0, 1e-2), n=2000, box=(0.0, 1.0), table=1.0, h=128,
                     bias=False, feat=8),
    "one_point": dict(pos_dim=3, capacity=2 ** 10, nr_levels=4, sigma=(1.0, 1e-1), n=1, box=(0.0, 1.0), table=1.0, h=256, bias=True),
}


def _setup(nat, name):
    c = CASES[name]
    cases.CASES["fused_" + name] = c
    try:
        inp = cases.make_inputs("fused_" + name)
    finally:
        del cases.CASES["fused_" + name]
    feat = c.get("feat", 2)
    fx = nat.EncodingFixedParams(c["pos_dim"], c["capacity"], c["nr_levels"], feat, inp["sigmas"], T(inp["shift"]),
                                 c.get("concat", False), c.get("points_scaling", 1.0))
    enc = nat.EncodingWrapper.create(c["pos_dim"], feat, fx)
    import zlib
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    width = enc.output_width()
    weight = (rng.standard_normal((c["h"], width)) / np.sqrt(width)).astype(np.float32)
    bias = rng.standard_normal(c["h"]).astype(np.float32) * 0.1 if c["bias"] else None
    return c, inp, enc, fx, weight, bias


def _bound(feats, weight):
    mag = np.abs(feats.astype(np.float64)) @ np.abs(weight.astype(np.float64)).T
    return TF32_RTOL * mag


@pytest.mark.parametrize("name", sorted(CASES))
def test_forward_linear_against_oracle(nat, oracle, name):
    c, inp, enc, fx, weight, bias = _setup(nat, name)
    scale = fx.m_scale_factor_host.numpy()
    feats = oracle.forward(inp["positions"], inp["table"], scale, inp["shift"], inp["anneal"],
                           concat_points=c.get("concat", False), points_scaling=c.get("points_scaling", 1.0))
    want = feats.astype(np.float64) @ weight.astype(np.float64).T + (0 if bias is None else bias.astype(np.float64))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    I = nat.EncodingInput(T(inp["table"]), T(inp["positions"]), T(inp["anneal"]), False, False)
    got = enc.forward_linear(I, T(weight), None if bias is None else T(bias), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "the kernel's bounded wait for the tensor core ran out"
    assert got.shape == (c["n"], c["h"]) and got.dtype == torch.float32
    err = np.abs(got.cpu().numpy().astype(np.float64) - want)
    bound = _bound(feats, weight) + 1e-6 * np.abs(want).max()
    assert np.all(err <= bound), f"worst error / bound = {(err / bound).max():.3f}"
    # and it is not trivially satisfied: errors are well inside but the outputs are not tiny
    assert np.abs(want).max() > 100 * bound.mean()
    # same numbers as the unfused pair (module forward, then an fp32 linear layer)
    unfused = torch.nn.functional.linear(enc.forward(I), T(weight), None if bias is None else T(bias))
    assert np.all(np.abs((got - unfused).cpu().numpy()) <= bound + 1e-5 * np.abs(want).max())
    # repeatable bit for bit (no atomics anywhere on this path)
    assert torch.equal(got, enc.forward_linear(I, T(weight), None if bias is None else T(bias)))


def test_forward_linear_half_table(nat, oracle):
    c, inp, enc, fx, weight, bias = _setup(nat, "toy_mlp")
    rounded = inp["table"].astype(np.float16)
    scale = fx.m_scale_factor_host.numpy()
    feats = oracle.forward(inp["positions"], rounded.astype(np.float32), scale, inp["shift"], inp["anneal"])
    want = feats.astype(np.float64) @ weight.astype(np.float64).T + bias.astype(np.float64)
    I = nat.EncodingInput(T(rounded), T(inp["positions"]), T(inp["anneal"]), False, False)
    got = enc.forward_linear(I, T(weight), T(bias)).cpu().numpy()
    assert np.all(np.abs(got - want) <= _bound(feats, weight) + 1e-6 * np.abs(want).max())


def test_forward_linear_module_and_mlp(nat):
    """Module-level shortcut with a torch.nn.Linear, as in the reference's toy example."""
    from permutohedral_encoding_b200 import PermutoEncoding
    torch.manual_seed(4)
    enc = PermutoEncoding(3, 2 ** 16, 24, 2, np.geomspace(1.0, 1e-4, 24))
    with torch.no_grad():
        enc.lattice_values.uniform_(-1, 1)
    lin = torch.nn.Linear(enc.output_dims(), 32).to(DEV)
    pts = torch.rand(100000, 3, device=DEV)
    with torch.no_grad():
        feats = enc(pts)
        want = torch.nn.functional.linear(feats.double(), lin.weight.double(), lin.bias.double())
        bound = TF32_RTOL * (feats.double().abs() @ lin.weight.double().abs().t()) + 1e-6 * want.abs().max()
    got = enc.forward_linear(pts, lin)
    assert not got.requires_grad and got.shape == (100000, 32)
    assert torch.all((got.double() - want).abs() <= bound)
    got2 = enc.forward_linear(pts, (lin.weight, None))
    assert torch.all((got2.double() - (want - lin.bias.double())).abs() <= bound)


def test_forward_linear_rejects_bad_arguments(nat):
    c, inp, enc, fx, weight, bias = _setup(nat, "toy_mlp")
    I = nat.EncodingInput(T(inp["table"]), T(inp["positions"]), T(inp["anneal"]), False, False)
    with pytest.raises(RuntimeError, match="out_features"):
        enc.forward_linear(I, torch.zeros(24, enc.output_width(), device=DEV))
    with pytest.raises(RuntimeError, match="weight should be"):
        enc.forward_linear(I, torch.zeros(32, enc.output_width() + 1, device=DEV))
    with pytest.raises(RuntimeError, match="bias should have"):
        enc.forward_linear(I, T(weight), torch.zeros(5, device=DEV))
    import ctypes as C
    cfg = nat.PermutoConfig(3, 2, 24, 2 ** 16, 0, 1.0, 0, 0)
    ins = nat.PermutoInputs(16, 256, 3, 1, 256, 256, 256, 256)
    assert nat.lib.permuto_forward_linear(C.byref(cfg), C.byref(ins), None, None, 32, None, None, None) \
        == nat.PERMUTO_ERR_INVALID_ARGUMENT
    assert nat.lib.permuto_forward_linear(C.byref(cfg), C.byref(ins), 256, None, 40, 256, None, None) \
        == nat.PERMUTO_ERR_UNSUPPORTED


# ---------------------------------------------------------------------------------------------
# a whole small MLP behind the encoding
# ---------------------------------------------------------------------------------------------
def _tf32(x):
    """cvt.rna.tf32.f32 in numpy: fp32 rounded to a 10-bit mantissa, ties away from zero."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((bits + np.uint32(0x1000)) & np.uint32(0xFFFFE000)).view(np.float32)


def _mlp_reference(feats, layers, activation):
    """Two float64 evaluations of the layers: exact, and with the operands of every tensor-core
    layer (width a multiple of 16) rounded to tf32 as the kernel rounds them.  Also returns, per
    output, sum|x*w| of the last layer (the magnitude the tolerances are relative to) and a
    worst-case bound on exact-vs-tf32: every tensor-core layer perturbs its output by at most
    TF32_RTOL * sum|x*w|, and a perturbation of a layer's input passes through |W| and an
    activation whose slope is at most 1.13."""
    from scipy.special import erf

    def act(y):
        if activation == "relu":
            return np.maximum(y, 0)
        if activation == "gelu":
            return 0.5 * y * (1 + erf(y / np.sqrt(2.0)))
        return y

    x = xe = feats.astype(np.float64)
    err = np.zeros_like(x)
    for i, (w, b) in enumerate(layers):
        w64 = w.astype(np.float64)
        bias = 0 if b is None else b.astype(np.float64)
        on_tensor_core = w.shape[0] % 16 == 0
        err = err @ np.abs(w64).T + (TF32_RTOL * (np.abs(x) @ np.abs(w64).T) if on_tensor_core else 0)
        mag = np.abs(xe) @ np.abs(w64).T
        if on_tensor_core:
            xe = _tf32(xe.astype(np.float32)).astype(np.float64) @ _tf32(w).astype(np.float64).T + bias
        else:
            xe = xe.astype(np.float32).astype(np.float64) @ w64.T + bias
        x = x @ w64.T + bias
        if i + 1 < len(layers):
            x, xe, err = act(x), act(xe), err * 1.13
    return x, err, xe, mag


MLP_CASES = {
    # the reference's toy example: 48 -> 32 -> 32 -> 32 -> 1 with GELU (examples/train_toy_example.py:18-26)
    "toy_example": ("toy_mlp", [32, 32, 32, 1], "gelu", True),
    "relu_two_outputs": ("toy_mlp", [64, 16, 3], "relu", True),
    "wide_last": ("wide_64", [48, 32], "gelu", False),
    "linear_chain": ("padded_concat", [16, 16], "none", True),
    "feat4_hidden64": ("feat4", [64, 64, 4], "gelu", True),
}


@pytest.mark.parametrize("name", sorted(MLP_CASES))
def test_forward_mlp_against_oracle(nat, oracle, name):
    base, widths, activation, with_bias = MLP_CASES[name]
    c, inp, enc, fx, _, _ = _setup(nat, base)
    import zlib
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    layers, fan_in = [], enc.output_width()
    for h in widths:
        w = (rng.standard_normal((h, fan_in)) * np.sqrt(2.0 / fan_in)).astype(np.float32)
        b = (rng.standard_normal(h) * 0.2).astype(np.float32) if with_bias else None
        layers.append((w, b))
        fan_in = h
    scale = fx.m_scale_factor_host.numpy()
    feats = oracle.forward(inp["positions"], inp["table"], scale, inp["shift"], inp["anneal"],
                           concat_points=c.get("concat", False), points_scaling=c.get("points_scaling", 1.0))
    want, err, emulated, mag = _mlp_reference(feats, layers, activation)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    I = nat.EncodingInput(T(inp["table"]), T(inp["positions"]), T(inp["anneal"]), False, False)
    dev_layers = [(T(w), None if b is None else T(b)) for w, b in layers]
    got = enc.forward_mlp(I, dev_layers, activation, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert got.shape == (c["n"], widths[-1])
    got64 = got.cpu().numpy().astype(np.float64)
    # sharp: the same roundings emulated in float64 -- what is left is fp32 accumulation and the odd
    # hidden unit that lands on the other side of a tf32 rounding boundary
    sharp = 1e-3 * mag + 1e-6 * np.abs(want).max()
    assert np.all(np.abs(got64 - emulated) <= sharp), f"worst error / tolerance = {(np.abs(got64 - emulated) / sharp).max():.3f}"
    assert np.abs(want).max() > 50 * sharp.mean()            # ... and that tolerance is not vacuous
    # loose: the exact network, within the worst-case cost of tf32 operands
    bound = err + 1e-5 * np.abs(want).max()
    assert np.all(np.abs(got64 - want) <= bound)
    # against the unfused evaluation in fp32 on the device
    x = enc.forward(I)
    for i, (w, b) in enumerate(dev_layers):
        x = torch.nn.functional.linear(x, w, b)
        if i + 1 < len(dev_layers):
            x = {"gelu": torch.nn.functional.gelu, "relu": torch.relu, "none": lambda v: v}[activation](x)
    assert np.all(np.abs((got - x).cpu().numpy()) <= bound + 1e-5 * np.abs(want).max())
    assert torch.equal(got, enc.forward_mlp(I, dev_layers, activation))


def test_forward_mlp_module_with_the_toy_example_network(nat):
    from permutohedral_encoding_b200 import PermutoEncoding
    torch.manual_seed(5)
    enc = PermutoEncoding(3, 2 ** 16, 24, 2, np.geomspace(1.0, 1e-4, 24))
    with torch.no_grad():
        enc.lattice_values.uniform_(-1, 1)
    mlp = torch.nn.Sequential(torch.nn.Linear(enc.output_dims(), 32), torch.nn.GELU(), torch.nn.Linear(32, 32),
                              torch.nn.GELU(), torch.nn.Linear(32, 32), torch.nn.GELU(), torch.nn.Linear(32, 1)).to(DEV)
    pts = torch.rand(70001, 3, device=DEV)
    with torch.no_grad():
        want = mlp(enc(pts))
    got = enc.forward_mlp(pts, mlp)
    assert got.shape == (70001, 1) and not got.requires_grad
    assert torch.allclose(got, want, rtol=0, atol=5e-3 * float(want.abs().max()))
    with pytest.raises(RuntimeError, match="end with a Linear"):
        enc.forward_mlp(pts, torch.nn.Sequential(torch.nn.Linear(48, 32), torch.nn.GELU()).to(DEV))
    with pytest.raises(RuntimeError, match="cannot fuse"):
        enc.forward_mlp(pts, torch.nn.Sequential(torch.nn.Linear(48, 32), torch.nn.Tanh(), torch.nn.Linear(32, 1)).to(DEV))
    with pytest.raises(RuntimeError, match="hidden width"):
        enc.forward_mlp(pts, torch.nn.Sequential(torch.nn.Linear(48, 24), torch.nn.ReLU(), torch.nn.Linear(24, 1)).to(DEV))
