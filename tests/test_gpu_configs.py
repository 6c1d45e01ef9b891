"""The benchmark configurations other than the headline, as parity cases at their own sizes:

* the CPU-runnable case: one layer, float32, N = 4096 tokens, d = 256, h = 1024, grid [-5, 5], G = 20,
  r = 32, lambda = 1, with z = ReLU^2(x W_in) clamped to the grid as the operator's input (so about half
  the entries are exactly 0: knot interval 10, tau = 0), in float32 (CUDA-core kernels) and bf16
  (tcgen05 kernels), full size against the CPU oracle;
* the boundary-heavy case: lambda = 0.25 and pre-activations four times as wide, so that a few per
  cent of z fall outside the grid, on a 4096-token slice of the production width (h = 5120).
Inputs are seeded synthetic tensors of those shapes and distributions.
"""
import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("sparsespline_ffn_b200.ops")


def _layer_inputs(N, d, h, r, G, x_std, relu2, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, d, generator=g) * x_std
    W_in = torch.randn(d, h, generator=g) / d ** 0.5
    pre = x @ W_in
    z = torch.where(pre > 0, pre * pre, torch.zeros_like(pre)).clamp(-5.0, 5.0) if relu2 else pre
    C = torch.randn(h, G + 2, r, generator=g) * 0.02
    go = torch.randn(N, h + r, generator=g)
    return z, C, go


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_cpu_runnable_configuration_full_size(dtype):
    N, d, h, r, G = 4096, 256, 1024, 32, 20
    z, C, go = (t.to(dtype).cuda() for t in _layer_inputs(N, d, h, r, G, 1.0, relu2=True))
    assert ops.resolve_impl(z, C, -5.0, 5.0, G) == ("simt" if dtype == torch.float32 else "tcgen05")
    bins = ops.knot_index(z, -5.0, 5.0, G).cpu().numpy()
    assert np.array_equal(bins, util.oc.knot_index(util.f32(z), -5.0, 5.0, G))
    assert (bins == 10).mean() > 0.45                  # the exact zeros of ReLU^2 sit on a knot
    # the operator input is already ReLU^2(pre): identity base path, as the survey's "relu2" z-mode
    f = ops.feature_forward(z, C, -5.0, 5.0, G, "identity", 1.0)
    dz, dC, _ = ops.feature_backward(z, C, go, -5.0, 5.0, G, "identity", 1.0)
    a_ref, d_ref = util.oracle_forward(z, C, -5.0, 5.0, G, "identity", 1.0)
    dz_ref, dC_ref = util.oracle_backward(z, C, go, -5.0, 5.0, G, "identity", 1.0)
    util.assert_parity("phi(z)", f[:, :h], a_ref, dtype)
    util.assert_parity("lambda*delta", f[:, h:], d_ref, dtype)
    util.assert_parity("dz", dz, dz_ref, dtype)
    util.assert_parity("dC", dC, dC_ref, dtype, bias=True)
    ops.check_status(z.device)


def test_boundary_heavy_configuration_slice():
    N, d, h, r, G, lam = 4096, 1280, 5120, 32, 20, 0.25
    z, C, go = (t.to(torch.bfloat16).cuda() for t in _layer_inputs(N, d, h, r, G, 2.0, relu2=False, seed=1))
    zf = util.f32(z)
    outside = float(((zf < -5.0) | (zf > 5.0)).mean())
    assert 0.005 < outside < 0.1                      # the clamp and boundary intervals are exercised
    bins = ops.knot_index(z, -5.0, 5.0, G).cpu().numpy()
    assert np.array_equal(bins, util.oc.knot_index(zf, -5.0, 5.0, G))
    _, d32 = ops.feature_forward(z, C, -5.0, 5.0, G, "relu_sq", lam, delta_f32=True)
    dz, dC, _ = ops.feature_backward(z, C, go, -5.0, 5.0, G, "relu_sq", lam)
    _, d_ref = util.oracle_forward(z, C, -5.0, 5.0, G, "relu_sq", lam)
    dz_ref, dC_ref = util.oracle_backward(z, C, go, -5.0, 5.0, G, "relu_sq", lam)
    util.assert_parity("delta f32", d32, d_ref, torch.bfloat16, bias=True)
    util.assert_parity("dz", dz, dz_ref, torch.bfloat16)
    util.assert_parity("dC", dC, dC_ref, torch.bfloat16, bias=True)
    # tokens outside the grid contribute exactly nothing to the residual and to dz's spline term
    far = torch.full_like(z, 100.0)
    assert float(ops.feature_forward(far, C, -5.0, 5.0, G, "relu_sq", lam)[:, h:].abs().max()) == 0.0
    ops.check_status(z.device)
