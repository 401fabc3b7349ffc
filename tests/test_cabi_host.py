"""CPU-only checks of the C-ABI library and the host-side Python mirror: the library loads,
exports every function the header declares, validates arguments before touching CUDA, and the
host scale-factor routine has the reference's bits.  No kernel runs here."""
import ctypes as C
import math
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "permuto_b200.h")


@pytest.fixture(scope="module")
def nat():
    from permutohedral_encoding_b200 import _native
    return _native


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(permuto_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(nat):
    names = declared_functions()
    assert len(names) >= 8
    for n in names:
        assert hasattr(nat.lib, n), f"{n} declared in include/permuto_b200.h but not exported"
    assert nat.lib.permuto_abi_version() == nat.ABI_VERSION == 2


def test_extra_levels(nat):
    assert [nat.extra_levels(d, True) for d in range(2, 8)] == [1, 2, 2, 3, 3, 4]
    assert [nat.extra_levels(d, True, 4) for d in range(2, 8)] == [1, 1, 1, 2, 2, 2]
    assert nat.extra_levels(7, True, 8) == 1
    assert nat.extra_levels(3, False) == 0


@pytest.mark.parametrize("d", [2, 3, 4, 5, 6, 7])
def test_scale_factor_matches_oracle_bits(nat, oracle, d):
    sig = np.geomspace(1.0, 1e-4, 24)
    a, b = nat.scale_factor(sig, d), oracle.scale_factor(sig, d)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_scale_factor_matches_reference_fixture(nat):
    import cases
    g = np.load(os.path.join(ROOT, "tests", "golden", "dim6.npz"))
    mine = nat.scale_factor(cases.sigmas_of(cases.CASES["dim6"]), 6)
    assert np.array_equal(mine.view(np.uint32), g["aten_scale"].view(np.uint32))


def test_argument_validation_without_gpu(nat):
    lib = nat.lib
    assert lib.permuto_forward(None, None, None, None) == nat.PERMUTO_ERR_INVALID_ARGUMENT
    assert "NULL" in nat.last_error()
    cfg = nat.PermutoConfig(8, 2, 4, 1024, 0, 1.0, 0, 0)
    ins = nat.PermutoInputs(10, 8, 3, 1, 8, 8, 8, 8)
    assert lib.permuto_forward(C.byref(cfg), C.byref(ins), C.c_void_p(8), None) == nat.PERMUTO_ERR_UNSUPPORTED
    assert "pos_dim must be 2,3,4,5,6 or 7" in nat.last_error()
    cfg = nat.PermutoConfig(3, 3, 4, 1024, 0, 1.0, 0, 0)
    assert lib.permuto_forward(C.byref(cfg), C.byref(ins), C.c_void_p(8), None) == nat.PERMUTO_ERR_UNSUPPORTED
    assert "nr_feat_per_level must be 2, 4 or 8" in nat.last_error()
    cfg = nat.PermutoConfig(3, 2, 4, 1024, 0, 1.0, 0, 0)
    ins0 = nat.PermutoInputs(0, 8, 3, 1, 8, 8, 8, 8)
    assert lib.permuto_forward(C.byref(cfg), C.byref(ins0), C.c_void_p(8), None) == nat.PERMUTO_ERR_INVALID_ARGUMENT
    assert "0 points" in nat.last_error()
    big = nat.PermutoInputs(2 ** 31, 8, 3, 1, 8, 8, 8, 8)
    assert lib.permuto_forward(C.byref(cfg), C.byref(big), C.c_void_p(8), None) == nat.PERMUTO_ERR_INVALID_ARGUMENT
    assert "2^31" in nat.last_error()
    odd = nat.PermutoInputs(10, 8, 3, 1, 12, 8, 8, 8)   # lattice_values not 8-byte aligned
    assert lib.permuto_forward(C.byref(cfg), C.byref(odd), C.c_void_p(8), None) == nat.PERMUTO_ERR_INVALID_ARGUMENT
    assert lib.permuto_backward(C.byref(cfg), C.byref(ins), C.c_void_p(8), None, None, 2, 9, 0, None) \
        == nat.PERMUTO_ERR_INVALID_ARGUMENT
    assert "level range" in nat.last_error()
    assert lib.permuto_double_backward(C.byref(cfg), C.byref(ins), None, None, None, None, 0, None) \
        == nat.PERMUTO_ERR_INVALID_ARGUMENT
    with pytest.raises(RuntimeError):
        nat.check(nat.PERMUTO_ERR_INVALID_ARGUMENT)


def test_wrapper_rejects_what_the_reference_rejects(nat):
    shift = torch.zeros(4, 3)
    fx = nat.EncodingFixedParams(3, 1024, 4, 2, np.geomspace(1, 0.1, 4), shift, False, 1.0)
    with pytest.raises(RuntimeError, match="nr_feat_per_level must be 2, 4 or 8"):
        nat.EncodingWrapper.create(3, 3, fx)
    with pytest.raises(RuntimeError, match="pos_dim must be"):
        nat.EncodingWrapper.create(8, 2, fx)
    enc = nat.EncodingWrapper.create(3, 2, fx)
    table = torch.zeros(4, 1024, 2)
    with pytest.raises(RuntimeError, match="GPU memory"):   # CPU tensors: no fallback, loud error
        enc.forward(nat.EncodingInput(table, torch.zeros(5, 3), torch.ones(4), False, False))


def test_python_helpers():
    from permutohedral_encoding_b200 import Coarse2Fine, map_range_val
    from permutohedral_encoding_b200.utils import cosine_easing_window
    assert map_range_val(5.0, 0.0, 10.0, 0.0, 1.0) == pytest.approx(0.5)
    assert map_range_val(-3.0, 0.0, 10.0, 2.0, 4.0) == 2.0 and map_range_val(30.0, 0.0, 10.0, 2.0, 4.0) == 4.0
    c2f = Coarse2Fine(8)
    w = c2f(0.5)
    assert w.shape == (8,) and c2f.get_last_t() == 0.5
    assert torch.allclose(w[:4], torch.ones(4)) and torch.allclose(w[4:], torch.zeros(4), atol=1e-7)
    w = cosine_easing_window(4, torch.tensor(1.5))
    assert w[0] == 1 and w[1] == pytest.approx(0.5 * (1 + math.cos(math.pi * 0.5 + math.pi))) and w[2] == 0
    with pytest.raises(AssertionError):
        c2f(1.5)


def test_module_needs_cuda_and_has_no_cpu_fallback():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from permutohedral_encoding_b200 import PermutoEncoding
    with pytest.raises((RuntimeError, AssertionError)):
        PermutoEncoding(3, 1024, 4, 2, np.geomspace(1, 0.1, 4))


def test_header_is_plain_c_and_library_links_from_c(tmp_path, nat):
    """The boundary is a C ABI: the header compiles as C99, and a C program linked against the
    library can call the host-side entry points (no GPU needed for these)."""
    import subprocess
    src = tmp_path / "use_abi.c"
    src.write_text(
        '#include <stdio.h>\n#include "permuto_b200.h"\n'
        "int main(void) {\n"
        "  double sig[2] = {1.0, 0.5}; float out[6];\n"
        "  if (permuto_abi_version() != PERMUTO_ABI_VERSION) return 1;\n"
        "  if (permuto_scale_factor(sig, 2, 3, out) != PERMUTO_OK) return 2;\n"
        "  if (permuto_scale_factor(sig, 2, 9, out) != PERMUTO_ERR_UNSUPPORTED) return 3;\n"
        "  if (permuto_forward(NULL, NULL, NULL, NULL) != PERMUTO_ERR_INVALID_ARGUMENT) return 4;\n"
        '  printf("%.9g %.9g %s\\n", out[0], out[5], permuto_last_error());\n'
        "  return 0;\n}\n")
    exe = tmp_path / "use_abi"
    lib_dir = os.path.dirname(nat.LIB_PATH)
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", lib_dir, "-l:libpermuto_b200.so", f"-Wl,-rpath,{lib_dir}"], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    a, b = res.stdout.split()[:2]
    want = nat.scale_factor([1.0, 0.5], 3)
    assert np.float32(a) == want[0, 0] and np.float32(b) == want[1, 2]
    assert "NULL" in res.stdout
