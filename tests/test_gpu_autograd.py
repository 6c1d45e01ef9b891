"""The operator classes on a GPU: same call shapes as the reference's boundary tests
(tests/test_flash_spline_feature_autograd.py:34-117), gradients checked against the oracle."""
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

skv = pytest.importorskip("sparsespline_ffn_b200")
LO, HI, G = -3.0, 3.0, 20


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_feature_function_forward_backward(dtype):
    N, h, r = 512, 128, 32
    z, C, go = util.make_inputs(N, h, r, G, dtype)
    z.requires_grad_(True)
    C.requires_grad_(True)
    f = skv.FlashSplineFeature.apply(z, C, LO, HI, G, "relu_sq", 0.5, True, "triton", "auto")
    assert f.shape == (N, h + r) and f.dtype == dtype
    f.backward(go)
    assert z.grad.dtype == dtype and C.grad.dtype == dtype and C.grad.shape == C.shape
    a_ref, d_ref = util.oracle_forward(z, C, LO, HI, G, "relu_sq", 0.5)
    dz_ref, dC_ref = util.oracle_backward(z, C, go, LO, HI, G, "relu_sq", 0.5)
    util.assert_parity("a", f[:, :h], a_ref, dtype)
    util.assert_parity("delta", f[:, h:], d_ref, dtype)
    util.assert_parity("dz", z.grad, dz_ref, dtype)
    util.assert_parity("dC", C.grad, dC_ref, dtype)


def test_functional_wrappers_and_defaults():
    N, h, r = 256, 64, 32
    z, C, go = util.make_inputs(N, h, r, G, torch.bfloat16)
    f = skv.flash_spline_feature(z, C)                      # defaults: grid [-3, 3], G=20, relu_sq
    a_ref, d_ref = util.oracle_forward(z, C, -3.0, 3.0, 20)
    util.assert_parity("delta", f[:, h:], d_ref, torch.bfloat16)
    d = skv.flash_spline_delta(z, C, lambda_scale=0.25)
    _, d_ref2 = util.oracle_forward(z, C, -3.0, 3.0, 20, "identity", 0.25)
    assert d.shape == (N, r)
    util.assert_parity("delta only", d, d_ref2, torch.bfloat16)


def test_delta_function_backward():
    N, h, r = 384, 64, 64
    z, C, go = util.make_inputs(N, h, r, G, torch.bfloat16)
    z.requires_grad_(True)
    C.requires_grad_(True)
    d = skv.FlashSplineDelta.apply(z, C, LO, HI, G, 0.5, "wgmma_cuda")
    d.backward(go[:, h:].contiguous())
    dz_ref, dC_ref = util.oracle_backward(z, C, go[:, h:], LO, HI, G, "identity", 0.5, with_base=False)
    util.assert_parity("dz", z.grad, dz_ref, torch.bfloat16)
    util.assert_parity("dC", C.grad, dC_ref, torch.bfloat16)


def test_gradients_only_where_required():
    N, h, r = 128, 64, 32
    z, C, go = util.make_inputs(N, h, r, G, torch.bfloat16)
    z.requires_grad_(True)
    f = skv.flash_spline_feature(z, C, LO, HI, G)
    f.backward(go)
    assert z.grad is not None and C.grad is None
    z2 = z.detach().clone()
    C2 = C.detach().clone().requires_grad_(True)
    skv.flash_spline_feature(z2, C2, LO, HI, G).backward(go)
    assert C2.grad is not None and z2.grad is None


def test_non_contiguous_grad_output():
    N, h, r = 128, 64, 32
    z, C, go = util.make_inputs(N, h, r, G, torch.bfloat16)
    z.requires_grad_(True)
    wide = torch.zeros(N, 2 * (h + r), dtype=go.dtype, device=go.device)
    wide[:, ::2] = go
    f = skv.flash_spline_feature(z, C, LO, HI, G)
    f.backward(wide[:, ::2])
    dz_ref, _ = util.oracle_backward(z, C, go, LO, HI, G)
    util.assert_parity("dz", z.grad, dz_ref, torch.bfloat16)


def test_forced_kernel_names_and_env_override(monkeypatch):
    N, h, r = 128, 64, 32
    z, C, _ = util.make_inputs(N, h, r, G, torch.bfloat16)
    f_auto = skv.flash_spline_feature(z, C, LO, HI, G)
    f_simt = skv.flash_spline_feature(z, C, LO, HI, G, fwd_kernel="simt", bwd_kernel="simt")
    util.assert_parity("simt vs auto", f_simt, util.f32(f_auto), torch.bfloat16)
    monkeypatch.setenv("SPARSE_SPLINE_FWD_KERNEL", "simt")
    assert torch.equal(skv.flash_spline_feature(z, C, LO, HI, G), f_simt)
    monkeypatch.setenv("SPARSE_SPLINE_FWD_KERNEL", "bogus")
    with pytest.raises(ValueError):
        skv.flash_spline_feature(z, C, LO, HI, G)


def test_forward_backward_under_cuda_graph_capture():
    """The operator enqueues on the current stream without host synchronisation, so a training step
    can be captured into a CUDA graph; during capture dC is accumulated into the preallocated
    ``C.grad`` as the reference does (flash_spline_feature_autograd.py:154-172).  The replayed
    graph must give the eager results for new input values."""
    N, h, r = 640, 128, 32
    z_a, C, go = util.make_inputs(N, h, r, G, torch.bfloat16, seed=11)
    z_b, _, _ = util.make_inputs(N, h, r, G, torch.bfloat16, seed=12)
    C.requires_grad_(True)
    z_static = z_a.clone().requires_grad_(True)
    # eager warm-up on a side stream (allocates the status word and the caching allocator's blocks)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            f = skv.flash_spline_feature(z_static, C, LO, HI, G, "relu_sq", 0.5, True)
            f.backward(go)
    torch.cuda.current_stream().wait_stream(s)
    z_static.grad.zero_()
    C.grad.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        f_static = skv.flash_spline_feature(z_static, C, LO, HI, G, "relu_sq", 0.5, True)
        f_static.backward(go)
    for z_new in (z_a, z_b):
        with torch.no_grad():
            z_static.copy_(z_new)
            z_static.grad.zero_()
            C.grad.zero_()
        graph.replay()
        torch.cuda.synchronize()
        a_ref, d_ref = util.oracle_forward(z_new, C, LO, HI, G, "relu_sq", 0.5)
        dz_ref, dC_ref = util.oracle_backward(z_new, C, go, LO, HI, G, "relu_sq", 0.5)
        util.assert_parity("delta", f_static[:, h:], d_ref, torch.bfloat16)
        util.assert_parity("a", f_static[:, :h], a_ref, torch.bfloat16)
        util.assert_parity("dz", z_static.grad, dz_ref, torch.bfloat16)
        util.assert_parity("dC", C.grad, dC_ref, torch.bfloat16)
    skv.ops.check_status(z_static.device)
