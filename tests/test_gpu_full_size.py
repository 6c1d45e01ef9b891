"""The d20 production shape (N = 65536 tokens, h = 5120, G = 20, r = 32, bf16) on the GPU.

At this size the oracle is applied where it finishes in seconds (the C/OpenMP restatement on all
tokens for dC, a token subset for f and dz) and size-independent properties cover the rest:
exact linearity in C, exact zeros, bitwise run-to-run determinism.
"""
import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("sparsespline_ffn_b200.ops")

N, H, R, G = 65536, 5120, 32, 20
LO, HI = -5.0, 5.0


@pytest.fixture(scope="module")
def data():
    g = torch.Generator(device="cuda").manual_seed(5)
    z = (torch.randn(N, H, generator=g, device="cuda") * 1.5).to(torch.bfloat16)
    C = (torch.randn(H, G + 2, R, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    go = torch.randn(N, H + R, generator=g, device="cuda").to(torch.bfloat16)
    return z, C, go


def test_forward_properties_and_sampled_parity(data):
    z, C, _ = data
    assert ops.resolve_impl(z, C, LO, HI, G) == "tcgen05"
    f = ops.feature_forward(z, C, LO, HI, G, "relu_sq", 1.0)
    # bitwise determinism
    assert torch.equal(f, ops.feature_forward(z, C, LO, HI, G, "relu_sq", 1.0))
    # exact linearity in C: a power of two commutes with every rounding on the path as long as no
    # table entry is an f16 subnormal, so use entries k * 2^-12 with |k| <= 127
    gq = torch.Generator(device="cuda").manual_seed(6)
    Cq = (torch.randint(-127, 128, C.shape, generator=gq, device="cuda").float() / 4096).to(torch.bfloat16)
    f1 = ops.feature_forward(z, Cq, LO, HI, G, "relu_sq", 1.0)
    f2 = ops.feature_forward(z, Cq * 2, LO, HI, G, "relu_sq", 1.0)
    assert torch.equal(f2[:, H:].float(), 2 * f1[:, H:].float())
    assert torch.equal(f2[:, :H], f[:, :H])
    # exact zeros
    f0 = ops.feature_forward(z, torch.zeros_like(C), LO, HI, G, "relu_sq", 1.0)
    assert torch.count_nonzero(f0[:, H:]) == 0
    # a token subset against the oracle; indices bit for bit
    idx = torch.randperm(N, generator=torch.Generator().manual_seed(1))[:512].cuda()
    zs = z[idx].contiguous()
    assert np.array_equal(ops.knot_index(zs, LO, HI, G).cpu().numpy(), util.oc.knot_index(util.f32(zs), LO, HI, G))
    a_ref, d_ref = util.oracle_forward(zs, C, LO, HI, G, "relu_sq", 1.0)
    util.assert_parity("phi(z)", f[idx][:, :H], a_ref, torch.bfloat16)
    util.assert_parity("delta", f[idx][:, H:], d_ref, torch.bfloat16)
    _, d32 = ops.feature_forward(z, C, LO, HI, G, "relu_sq", 1.0, delta_f32=True)
    util.assert_parity("delta f32", d32[idx], d_ref, torch.bfloat16, bias=True)
    ops.check_status(z.device)


def test_backward_properties_and_parity(data):
    z, C, go = data
    dz, dC, dC_cast = ops.feature_backward(z, C, go, LO, HI, G, "relu_sq", 0.5)
    dz_b, dC_b, _ = ops.feature_backward(z, C, go, LO, HI, G, "relu_sq", 0.5)
    assert torch.equal(dz, dz_b) and torch.equal(dC, dC_b)            # bitwise determinism
    assert torch.count_nonzero(dC[:, -1, :]) == 0                     # last knot row never gets weight
    assert torch.equal(dC_cast, dC.to(torch.bfloat16))
    # dC against the oracle on all tokens (float64 accumulate), dz on a token subset
    go32 = util.f32(go)
    dz_ref_unused, dC_ref = util.oc.feature_backward(util.f32(z), util.f32(C), go32[:, H:], None, LO, HI, G,
                                                     "identity", 0.5)
    util.assert_parity("dC", dC, dC_ref, torch.bfloat16, bias=True)
    idx = torch.randperm(N, generator=torch.Generator().manual_seed(2))[:512].cuda()
    dz_ref, _ = util.oracle_backward(z[idx].contiguous(), C, go[idx].contiguous(), LO, HI, G, "relu_sq", 0.5)
    util.assert_parity("dz", dz[idx], dz_ref, torch.bfloat16)
    # dC is linear in the upstream gradient: doubling it doubles dC exactly
    _, dC2, _ = ops.feature_backward(z, C, go * 2, LO, HI, G, "relu_sq", 0.5, need_dz=False)
    assert torch.equal(dC2, 2 * dC)
    ops.check_status(z.device)


@pytest.mark.parametrize("r,G", [(16, 20), (64, 20), (128, 20), (32, 40)], ids=["r16", "r64", "r128", "G40"])
def test_other_ranks_and_grids_at_full_key_count(r, G):
    """Code ranks 16 / 64 / 128 at G = 20 and rank 32 at G = 40, all h = 5120 keys wide, on 4096 tokens:
    forward, dz and dC against the oracle on every token, indices bit for bit, exact zeros."""
    n = 4096
    g = torch.Generator(device="cuda").manual_seed(100 + r + G)
    z = (torch.randn(n, H, generator=g, device="cuda") * 2.0).to(torch.bfloat16)
    C = (torch.randn(H, G + 2, r, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    go = torch.randn(n, H + r, generator=g, device="cuda").to(torch.bfloat16)
    assert ops.resolve_impl(z, C, LO, HI, G) == "tcgen05"
    assert np.array_equal(ops.knot_index(z, LO, HI, G).cpu().numpy(), util.oc.knot_index(util.f32(z), LO, HI, G))
    f = ops.feature_forward(z, C, LO, HI, G, "relu_sq", 0.25)
    a_ref, d_ref = util.oracle_forward(z, C, LO, HI, G, "relu_sq", 0.25)
    util.assert_parity("phi(z)", f[:, :H], a_ref, torch.bfloat16)
    util.assert_parity("delta", f[:, H:], d_ref, torch.bfloat16)
    dz, dC, _ = ops.feature_backward(z, C, go, LO, HI, G, "relu_sq", 0.25)
    dz_ref, dC_ref = util.oracle_backward(z, C, go, LO, HI, G, "relu_sq", 0.25)
    util.assert_parity("dz", dz, dz_ref, torch.bfloat16)
    util.assert_parity("dC", dC, dC_ref, torch.bfloat16, bias=True)
    assert torch.count_nonzero(dC[:, -1, :]) == 0
    f0 = ops.feature_forward(z, torch.zeros_like(C), LO, HI, G, "relu_sq", 0.25)
    assert torch.count_nonzero(f0[:, H:]) == 0
    ops.check_status(z.device)


def test_fused_readout_properties_and_sampled_parity(data):
    """y = [phi(z); lambda*delta] W_out^T at d_out = h / 4 without the feature tensor: determinism, exact
    doubling in W_out (a power of two commutes with every rounding), independence of the tokens from one
    another (a reversed token order gives the reversed rows, bit for bit, although every token lands in
    another tile and lane), the feature followed by a float64 product on a token subset."""
    z, C, _ = data
    D = H // 4
    g = torch.Generator(device="cuda").manual_seed(8)
    W = (torch.randn(D, H + R, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    y = ops.feature_readout_forward(z, C, W, LO, HI, G, "relu_sq", 1.0)
    assert y.shape == (N, D)
    assert torch.equal(y, ops.feature_readout_forward(z, C, W, LO, HI, G, "relu_sq", 1.0))
    assert torch.equal(ops.feature_readout_forward(z, C, W * 2, LO, HI, G, "relu_sq", 1.0).float(), 2 * y.float())
    yr = ops.feature_readout_forward(z.flip(0).contiguous(), C, W, LO, HI, G, "relu_sq", 1.0)
    assert torch.equal(yr.flip(0), y)
    idx = torch.randperm(N, generator=torch.Generator().manual_seed(2))[:1024].cuda()
    f = ops.feature_forward(z[idx].contiguous(), C, LO, HI, G, "relu_sq", 1.0)
    ref = f.double() @ W.double().t()
    err = (y[idx].double() - ref)
    assert float(err.norm() / ref.norm()) < 4e-3
    assert float(err.abs().max() / ref.abs().max()) < 8e-3
    ops.check_status(z.device)
