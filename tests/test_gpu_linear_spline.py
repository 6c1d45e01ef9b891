"""The linear B-spline (spline_order = 1, L = G + 1: weights 1 - tau and tau at rows bin, bin + 1) through
the C ABI, against the reference's own outputs (tests/golden/b1_golden.npz, written by
tests/golden/make_golden.py from flash_spline_feature_reference(spline_order=1) and autograd,
src/sparsespline_ffn/rl_spline_kv_reference.py:125-142, 178-187) and against the CPU oracle on larger
seeded inputs.  It runs on the CUDA-core kernels (float32 arithmetic, bf16 or float32 I/O)."""
import os

import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("sparsespline_ffn_b200.ops")


@pytest.fixture(scope="module")
def b1_golden():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "b1_golden.npz")
    data = np.load(path)
    cases = {}
    for key in data.files:
        case, name = key.split("/")
        cases.setdefault(case, {})[name] = data[key]
    return cases


@pytest.mark.parametrize("case", ["uniform", "d20_like", "gelu", "edges"])
def test_linear_spline_matches_the_reference_outputs(b1_golden, case):
    c = b1_golden[case]
    lo, hi, G, lam = float(c["meta"][0]), float(c["meta"][1]), int(c["meta"][2]), float(c["meta"][3])
    act = {0: "relu_sq", 1: "identity", 2: "gelu"}[int(c["meta"][4])]
    z = torch.from_numpy(c["z"]).cuda()
    C = torch.from_numpy(c["C"]).cuda()
    go = torch.from_numpy(c["go"]).cuda()
    h = z.shape[1]
    assert ops.resolve_impl(z, C, lo, hi, G + 0, "auto") in ("simt", "tcgen05") if C.shape[1] == G + 2 else True
    f = ops.feature_forward(z, C, lo, hi, G, act, lam, spline_order=1)
    dz, dC, _ = ops.feature_backward(z, C, go, lo, hi, G, act, lam, spline_order=1)
    finite = np.isfinite(c["z"])
    fa = util.f32(f)
    np.testing.assert_allclose(fa[:, :h][finite], c["f"][:, :h][finite], rtol=1e-5, atol=1e-6)
    util.assert_parity("lambda*delta", f[:, h:], c["f"][:, h:], torch.float32)
    np.testing.assert_allclose(util.f32(dz)[finite], c["dz"][finite], rtol=2e-4, atol=2e-5)
    util.assert_parity("dC", dC, c["dC"], torch.float32, bias=True)
    assert not util.f32(dC)[:, -1].any()             # the last knot row never gets a weight


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(1024, 256, 32, 21), (333, 72, 16, 9), (64, 40, 64, 41)],
                         ids=lambda s: "N%d_h%d_r%d_L%d" % s)
def test_linear_spline_against_the_oracle(shape, dtype):
    N, h, r, L = shape
    G = L - 1
    g = torch.Generator().manual_seed(4)
    z = (torch.randn(N, h, generator=g) * 2.0).to(dtype).cuda()
    C = (torch.randn(h, L, r, generator=g) * 0.1).to(dtype).cuda()
    go = torch.randn(N, h + r, generator=g).to(dtype).cuda()
    f = ops.feature_forward(z, C, -3.0, 3.0, G, "relu_sq", 0.75, spline_order=1)
    dz, dC, _ = ops.feature_backward(z, C, go, -3.0, 3.0, G, "relu_sq", 0.75, spline_order=1)
    a_ref, d_ref = util.oc.feature_forward(util.f32(z), util.f32(C), -3.0, 3.0, G, "relu_sq", 0.75, spline_order=1)
    gof = util.f32(go)
    dz_ref, dC_ref = util.oc.feature_backward(util.f32(z), util.f32(C), gof[:, h:], gof[:, :h], -3.0, 3.0, G,
                                              "relu_sq", 0.75, spline_order=1)
    util.assert_parity("phi(z)", f[:, :h], a_ref, dtype)
    util.assert_parity("lambda*delta", f[:, h:], d_ref, dtype)
    util.assert_parity("dz", dz, dz_ref, dtype)
    util.assert_parity("dC", dC, dC_ref, dtype, bias=True)
    # the quadratic table shape is refused for the linear spline and vice versa
    with pytest.raises(ValueError):
        ops.feature_forward(z, C, -3.0, 3.0, G, "relu_sq", 1.0)
    ops.check_status(z.device)


def test_linear_spline_autograd_function():
    from sparsespline_ffn_b200 import flash_spline_feature
    g = torch.Generator().manual_seed(8)
    z = (torch.randn(200, 48, generator=g) * 1.5).cuda().requires_grad_(True)
    C = (torch.randn(48, 13, 8, generator=g) * 0.1).cuda().requires_grad_(True)
    go = torch.randn(200, 56, generator=g).cuda()
    f = flash_spline_feature(z, C, -3.0, 3.0, 12, "identity", 0.5, True, spline_order=1)
    f.backward(go)
    gof = util.f32(go)
    dz_ref, dC_ref = util.oc.feature_backward(util.f32(z), util.f32(C), gof[:, 48:], gof[:, :48], -3.0, 3.0, 12,
                                              "identity", 0.5, spline_order=1)
    util.assert_parity("dz", z.grad, dz_ref, torch.float32)
    util.assert_parity("dC", C.grad, dC_ref, torch.float32)
