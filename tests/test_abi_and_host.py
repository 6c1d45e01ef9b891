"""CPU-side tests: the C-ABI library loads and exports what the header declares, the host
wrappers validate arguments like the reference does, and nothing silently falls back to CPU."""
import ctypes
import os
import re

import pytest
import torch

from sparsespline_ffn_b200 import _lib, build, ops
from sparsespline_ffn_b200 import (FlashSplineDelta, FlashSplineFeature, flash_spline_delta,
                                   flash_spline_feature)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "splinekv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(skv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = _declared_functions()
    assert set(_lib.EXPORTS) <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/splinekv_b200.h but not exported"


def test_abi_version_and_error_strings(lib):
    assert lib.skv_abi_version() == 4
    for code in range(0, -8, -1):
        assert lib.skv_error_string(code)
    assert b"unknown" in lib.skv_error_string(-99)


def test_problem_struct_matches_header(lib):
    text = open(os.path.join(ROOT, "include", "splinekv_b200.h")).read()
    body = re.search(r"typedef struct skv_problem \{(.*?)\} skv_problem;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b(?:int64_t|int32_t|float)\s+(\w+);", body)
    assert fields == [f[0] for f in _lib.Problem._fields_]


def test_validation_without_a_gpu(lib):
    p = _lib.Problem(N=128, h=64, L=22, r=32, grid_lo=-3.0, scale=20 / 6, lambda_scale=1.0,
                     activation=0, dtype=0, impl=0, delta_f32=0)
    assert lib.skv_resolve_impl(ctypes.byref(p)) in (1, 2)
    assert lib.skv_scratch_bytes(ctypes.byref(p), 1) > 0
    p.impl = 1
    assert lib.skv_resolve_impl(ctypes.byref(p)) == 1
    bad = _lib.Problem(N=128, h=64, L=3, r=32, grid_lo=-3.0, scale=1.0, lambda_scale=1.0,
                       activation=0, dtype=0, impl=0, delta_f32=0)
    assert lib.skv_resolve_impl(ctypes.byref(bad)) == -2
    bad2 = _lib.Problem(N=128, h=64, L=22, r=32, grid_lo=-3.0, scale=1.0, lambda_scale=1.0,
                        activation=7, dtype=0, impl=0, delta_f32=0)
    assert lib.skv_resolve_impl(ctypes.byref(bad2)) == -3
    assert lib.skv_resolve_impl(None) == -1
    # a float32 problem can never take the tcgen05 kernels
    p32 = _lib.Problem(N=128, h=64, L=22, r=32, grid_lo=-3.0, scale=1.0, lambda_scale=1.0,
                       activation=0, dtype=1, impl=2, delta_f32=0)
    assert lib.skv_resolve_impl(ctypes.byref(p32)) == -3


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_device_is_an_error_not_a_fallback(lib):
    assert lib.skv_device_ok() == -6
    p = _lib.Problem(N=4, h=8, L=22, r=16, grid_lo=-3.0, scale=1.0, lambda_scale=1.0,
                     activation=0, dtype=0, impl=0, delta_f32=0)
    assert lib.skv_feature_forward(ctypes.byref(p), None, 8, None, None, 0, None, 16, None, 0, None, None) == -6


def test_cpu_tensors_raise_instead_of_falling_back():
    z = torch.randn(4, 8)
    C = torch.randn(8, 22, 16)
    with pytest.raises(RuntimeError, match="CUDA-only"):
        flash_spline_feature(z, C, use_kernel=True)
    with pytest.raises(RuntimeError, match="use_kernel=False"):
        flash_spline_feature(z, C, use_kernel=False)
    with pytest.raises(RuntimeError, match="CUDA-only"):
        flash_spline_delta(z, C)
    with pytest.raises(RuntimeError, match="CUDA-only"):
        ops.feature_forward(z, C, -3, 3, 20)


def test_argument_validation_matches_the_reference():
    # shape checks come before the device check, as in flash_spline_feature_reference
    # (src/sparsespline_ffn/rl_spline_kv_reference.py:162-171)
    with pytest.raises(ValueError, match="2D"):
        ops.feature_forward(torch.randn(2, 4, 8), torch.randn(8, 22, 16), -3, 3, 20)
    with pytest.raises(ValueError, match="!= h"):
        ops.feature_forward(torch.randn(4, 8), torch.randn(9, 22, 16), -3, 3, 20)
    with pytest.raises(ValueError, match=r"G\+spline_order"):
        ops.feature_forward(torch.randn(4, 8), torch.randn(8, 21, 16), -3, 3, 20)
    with pytest.raises(ValueError, match="activation"):
        ops.feature_forward(torch.randn(4, 8), torch.randn(8, 22, 16), -3, 3, 20, activation="swish")
    with pytest.raises(ValueError, match="fwd_kernel"):
        FlashSplineFeature.apply(torch.randn(4, 8).requires_grad_(), torch.randn(8, 22, 16), -3, 3, 20,
                                 "relu_sq", 1.0, True, "triton", "no_such_kernel")
    with pytest.raises(ValueError, match="bwd_kernel"):
        FlashSplineDelta.apply(torch.randn(4, 8), torch.randn(8, 22, 16), -3, 3, 20, 1.0, "no_such_kernel")


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU or eager fallback"):
        _lib.load()


def test_package_does_not_import_the_oracle():
    import subprocess
    import sys
    code = ("import sys; import sparsespline_ffn_b200, sparsespline_ffn_b200.ops, sparsespline_ffn_b200.sharded; "
            "bad = [m for m in sys.modules if m == 'oracle' or m.startswith('oracle.')]; "
            "assert not bad, bad")
    subprocess.run([sys.executable, "-c", code], check=True, cwd=ROOT)
    for dirpath, _, files in os.walk(os.path.join(ROOT, "sparsespline_ffn_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
