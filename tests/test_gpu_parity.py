"""GPU parity tests: the CUDA library (through its C ABI) against the CPU oracle.

Shapes, input distributions and edge cases follow the reference's own kernel tests
(tests/test_rlkv_kernel_parity.py:109-150, 459-514; tests/test_flash_spline_feature_forward.py:89-169;
tests/test_flash_spline_feature_backward_kernel.py:19-164).  Knot-interval indices are compared
bit for bit; floating-point outputs against the gates in tests/util.py.
"""
import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("sparsespline_ffn_b200.ops")

# (N, h, r, L) of the reference's parity harness plus ragged / wide cases
SHAPES = [
    (64, 64, 8, 8),
    (256, 128, 16, 16),
    (1024, 256, 32, 22),
    (4096, 256, 32, 22),
    (333, 72, 32, 22),       # ragged token count, h not a multiple of 32
    (130, 40, 64, 22),
    (96, 24, 128, 42),       # widest code dimension, G = 40
    (1, 8, 16, 22),          # a single token
    (600, 64, 128, 22),      # rank sweep of the d20 width: r = 128, 64, 16 and G = 40
    (520, 64, 64, 22),
    (260, 64, 16, 22),
    (300, 64, 32, 42),
    (512, 64, 32, 23),       # odd knot-row counts (one zero pad row in the operand images) and L = 24, 32
    (300, 40, 16, 31),
    (200, 24, 32, 9),
    (512, 64, 32, 24),
    (512, 64, 32, 32),
]
DTYPES = [torch.float32, torch.bfloat16]
IMPLS = ["simt", "tcgen05"]
LO, HI = -3.0, 3.0


def _impl_or_skip(impl, z, C, G):
    if impl == "tcgen05" and ops.resolve_impl(z, C, LO, HI, G, "auto") != "tcgen05":
        pytest.skip("shape/dtype not eligible for the tcgen05 kernels")
    return impl


def _sid(s):
    return "N%d_h%d_r%d_L%d" % s


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", SHAPES, ids=_sid)
def test_knot_index_bit_exact(shape, dtype):
    N, h, r, L = shape
    z, _, _ = util.make_inputs(N, h, r, L - 2, dtype)
    got = ops.knot_index(z, LO, HI, L - 2).cpu().numpy()
    ref = util.oc.knot_index(util.f32(z), LO, HI, L - 2)
    assert np.array_equal(got, ref)


def test_knot_index_edges_bit_exact(golden):
    c = golden["edges"]
    lo, hi, G = float(c["meta"][0]), float(c["meta"][1]), int(c["meta"][2])
    z = torch.from_numpy(c["z"]).cuda()
    assert np.array_equal(ops.knot_index(z, lo, hi, G).cpu().numpy(), c["bins"])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", SHAPES, ids=_sid)
def test_forward_parity(shape, dtype, impl):
    N, h, r, L = shape
    G = L - 2
    z, C, _ = util.make_inputs(N, h, r, G, dtype)
    impl = _impl_or_skip(impl, z, C, G)
    f = ops.feature_forward(z, C, LO, HI, G, "relu_sq", 0.75, with_base=True, impl=impl)
    assert f.shape == (N, h + r) and f.dtype == dtype
    a_ref, d_ref = util.oracle_forward(z, C, LO, HI, G, "relu_sq", 0.75)
    util.assert_parity("phi(z)", f[:, :h], a_ref, dtype)
    util.assert_parity("lambda*delta", f[:, h:], d_ref, dtype)
    # float32 residual output: this is where the signed-bias gate applies
    a2, d32 = ops.feature_forward(z, C, LO, HI, G, "relu_sq", 0.75, with_base=True, impl=impl, delta_f32=True)
    assert d32.dtype == torch.float32 and d32.shape == (N, r)
    assert torch.equal(a2, f[:, :h])
    util.assert_parity("delta f32", d32, d_ref, dtype, bias=True)
    ops.check_status(z.device)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", SHAPES, ids=_sid)
def test_backward_parity(shape, dtype, impl):
    N, h, r, L = shape
    G = L - 2
    z, C, go = util.make_inputs(N, h, r, G, dtype)
    impl = _impl_or_skip(impl, z, C, G)
    dz, dC, dC_cast = ops.feature_backward(z, C, go, LO, HI, G, "relu_sq", 0.5, with_base=True, impl=impl)
    dz_ref, dC_ref = util.oracle_backward(z, C, go, LO, HI, G, "relu_sq", 0.5)
    assert dz.dtype == dtype and dC.dtype == torch.float32
    util.assert_parity("dz", dz, dz_ref, dtype)
    util.assert_parity("dC", dC, dC_ref, dtype, bias=True)
    if dtype == torch.bfloat16:
        assert dC_cast is not None and dC_cast.dtype == dtype
        assert torch.equal(dC_cast, dC.to(dtype))
    # residual-only operator: no base path in dz
    dz2, dC2, _ = ops.feature_backward(z, C, go[:, h:], LO, HI, G, "identity", 0.5, with_base=False, impl=impl)
    dz2_ref, dC2_ref = util.oracle_backward(z, C, go[:, h:], LO, HI, G, "identity", 0.5, with_base=False)
    util.assert_parity("dz_spline", dz2, dz2_ref, dtype)
    util.assert_parity("dC (delta only)", dC2, dC2_ref, dtype, bias=True)
    ops.check_status(z.device)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("workload", ["skewed", "collapsed"])
def test_backward_stress_distributions(workload, impl):
    """Skewed N(2, 0.5) and collapsed N(0, 0.05) pre-activations: every token lands in a few knot
    intervals, the worst case for the dC reduction."""
    N, h, r, G = 2048, 128, 32, 20
    g = torch.Generator().manual_seed(3)
    base = torch.randn(N, h, generator=g)
    z = (base * 0.5 + 2.0 if workload == "skewed" else base * 0.05).to(torch.bfloat16).cuda()
    C = (torch.randn(h, G + 2, r, generator=g) * 0.1).to(torch.bfloat16).cuda()
    go = torch.randn(N, h + r, generator=g).to(torch.bfloat16).cuda()
    impl = _impl_or_skip(impl, z, C, G)
    dz, dC, _ = ops.feature_backward(z, C, go, LO, HI, G, "relu_sq", 1.0, impl=impl)
    dz_ref, dC_ref = util.oracle_backward(z, C, go, LO, HI, G)
    util.assert_parity("dz", dz, dz_ref, torch.bfloat16)
    util.assert_parity("dC", dC, dC_ref, torch.bfloat16, bias=True)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("name", ["uniform", "d20_like", "skewed", "collapsed", "gelu"])
def test_golden_vectors_on_gpu(golden, name, impl):
    """The stored outputs of the reference itself, float32 end to end."""
    c = golden[name]
    lo, hi, G, lam = float(c["meta"][0]), float(c["meta"][1]), int(c["meta"][2]), float(c["meta"][3])
    act = ("relu_sq", "identity", "gelu")[int(c["meta"][4])]
    z = torch.from_numpy(c["z"]).cuda()
    C = torch.from_numpy(c["C"]).cuda()
    go = torch.from_numpy(c["go"]).cuda()
    dtype = torch.float32
    if impl == "tcgen05":
        z, C, go, dtype = z.bfloat16(), C.bfloat16(), go.bfloat16(), torch.bfloat16
        if ops.resolve_impl(z, C, lo, hi, G, "auto") != "tcgen05":
            pytest.skip("not eligible")
        if name != "d20_like":
            pytest.skip("inputs of this case are not bf16-representable")
    assert np.array_equal(ops.knot_index(z, lo, hi, G).cpu().numpy(), c["bins"])
    f = ops.feature_forward(z, C, lo, hi, G, act, lam, impl=impl)
    util.assert_parity("f", f, c["f"], dtype)
    dz, dC, _ = ops.feature_backward(z, C, go, lo, hi, G, act, lam, impl=impl)
    util.assert_parity("dz", dz, c["dz"], dtype)
    util.assert_parity("dC", dC, c["dC"], dtype)
    h = z.shape[1]
    d = ops.feature_forward(z, C, lo, hi, G, "identity", lam, with_base=False, impl=impl)
    util.assert_parity("delta only", d, c["delta_only"], dtype)
    dz2, dC2, _ = ops.feature_backward(z, C, go[:, h:], lo, hi, G, "identity", lam, with_base=False, impl=impl)
    util.assert_parity("delta dz", dz2, c["delta_dz"], dtype)
    util.assert_parity("delta dC", dC2, c["delta_dC"], dtype)


@pytest.mark.parametrize("impl", IMPLS)
def test_gelu_base_path(impl):
    """activation="gelu" (the exact erf form of F.gelu, as rl_spline_kv_reference.py:81-82) in bf16 at a
    shape the tcgen05 family takes: base half of f and the g_a * phi'(z) term of dz."""
    N, h, r, G = 300, 64, 32, 20
    z, C, go = util.make_inputs(N, h, r, G, torch.bfloat16, seed=5)
    impl = _impl_or_skip(impl, z, C, G)
    f = ops.feature_forward(z, C, LO, HI, G, "gelu", 0.5, impl=impl)
    a_ref, d_ref = util.oracle_forward(z, C, LO, HI, G, "gelu", 0.5)
    util.assert_parity("phi", f[:, :h], a_ref, torch.bfloat16)
    util.assert_parity("delta", f[:, h:], d_ref, torch.bfloat16)
    dz, dC, _ = ops.feature_backward(z, C, go, LO, HI, G, "gelu", 0.5, impl=impl)
    dz_ref, dC_ref = util.oracle_backward(z, C, go, LO, HI, G, "gelu", 0.5)
    util.assert_parity("dz", dz, dz_ref, torch.bfloat16)
    util.assert_parity("dC", dC, dC_ref, torch.bfloat16, bias=True)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_edge_cases(dtype, impl):
    N, h, r, G = 256, 64, 32, 20
    z, C, go = util.make_inputs(N, h, r, G, dtype)
    impl = _impl_or_skip(impl, z, C, G)
    # C = 0: the residual is exactly zero, dz of the spline path exactly zero, dC is not
    f0 = ops.feature_forward(z, torch.zeros_like(C), LO, HI, G, impl=impl)
    assert torch.count_nonzero(f0[:, h:]) == 0
    zf = z.float()
    assert torch.equal(f0[:, :h], torch.where(zf > 0, zf * zf, torch.zeros_like(zf)).to(dtype))
    dz0, dC0, _ = ops.feature_backward(z, torch.zeros_like(C), go[:, h:], LO, HI, G, "identity",
                                       with_base=False, impl=impl)
    assert torch.count_nonzero(dz0) == 0
    assert dC0.abs().max() > 0
    # every token far outside the grid: residual exactly zero and finite
    zfar = torch.full_like(z, 100.0)
    f1 = ops.feature_forward(zfar, C, LO, HI, G, impl=impl)
    assert torch.count_nonzero(f1[:, h:]) == 0 and torch.isfinite(f1).all()
    _, dCfar, _ = ops.feature_backward(zfar, C, go, LO, HI, G, impl=impl)
    assert torch.count_nonzero(dCfar) == 0
    # z exactly on the grid ends
    zedge = z.clone()
    zedge[:, ::2] = LO
    zedge[:, 1::2] = HI
    f2 = ops.feature_forward(zedge, C, LO, HI, G, impl=impl)
    _, d_ref = util.oracle_forward(zedge, C, LO, HI, G)
    assert torch.isfinite(f2).all()
    util.assert_parity("delta at grid ends", f2[:, h:], d_ref, dtype)
    # lambda scales the residual half only
    fa = ops.feature_forward(z, C, LO, HI, G, lambda_scale=1.0, impl=impl)
    fb = ops.feature_forward(z, C, LO, HI, G, lambda_scale=0.25, impl=impl)
    assert torch.equal(fa[:, :h], fb[:, :h])
    assert torch.allclose(fb[:, h:].float(), 0.25 * fa[:, h:].float(), rtol=2e-2, atol=1e-3)
    # the last knot row never receives weight
    _, dC, _ = ops.feature_backward(z, C, go, LO, HI, G, impl=impl)
    assert torch.count_nonzero(dC[:, -1, :]) == 0
    # partition of unity: C constant along the knot axis gives dz_spline = 0 inside the grid
    Cc = C[:, :1, :].expand(-1, G + 2, -1).contiguous()
    zin = z.clamp(-2.9, 2.9)
    dzc, _, _ = ops.feature_backward(zin, Cc, go[:, h:], LO, HI, G, "identity", with_base=False, impl=impl)
    assert dzc.float().abs().max() < (1e-4 if dtype == torch.float32 else 5e-2)
    ops.check_status(z.device)


def test_non_contiguous_and_strided_inputs():
    N, h, r, G = 128, 64, 32, 20
    z, C, go = util.make_inputs(N, 2 * h, r, G, torch.bfloat16)
    z_view = z[:, :h]                         # row stride 2h, unit inner stride: passed through
    z_t = z[:, :h].t().contiguous().t()       # inner stride != 1: copied
    Ch = C[:h].contiguous()
    f_ref = ops.feature_forward(z[:, :h].contiguous(), Ch, LO, HI, G)
    assert torch.equal(ops.feature_forward(z_view, Ch, LO, HI, G), f_ref)
    assert torch.equal(ops.feature_forward(z_t, Ch, LO, HI, G), f_ref)


def test_empty_input():
    h, r, G = 64, 32, 20
    z = torch.empty(0, h, dtype=torch.bfloat16, device="cuda")
    C = torch.zeros(h, G + 2, r, dtype=torch.bfloat16, device="cuda")
    f = ops.feature_forward(z, C, LO, HI, G)
    assert f.shape == (0, h + r)
    dz, dC, _ = ops.feature_backward(z, C, torch.empty(0, h + r, dtype=torch.bfloat16, device="cuda"), LO, HI, G)
    assert dz.shape == (0, h) and torch.count_nonzero(dC) == 0


def test_run_to_run_determinism():
    N, h, r, G = 4096, 256, 32, 20
    z, C, go = util.make_inputs(N, h, r, G, torch.bfloat16)
    f1 = ops.feature_forward(z, C, LO, HI, G)
    f2 = ops.feature_forward(z, C, LO, HI, G)
    assert torch.equal(f1, f2)
    a = ops.feature_backward(z, C, go, LO, HI, G)
    b = ops.feature_backward(z, C, go, LO, HI, G)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


@pytest.mark.parametrize("c_scale", [1e-6, 1e-7, "mixed"], ids=["1e-6", "1e-7", "mixed"])
def test_small_code_table_magnitudes(c_scale):
    """A freshly initialised code table is near zero (the reference starts from C = 0,
    src/sparsespline_ffn/rl_spline_kv_reference.py:44,285): the f16 operand images are range-scaled, so
    tiny entries keep their precision.  Errors are judged relative to the largest reference value."""
    N, h, r, G = 1024, 256, 32, 20
    g = torch.Generator().manual_seed(17)
    z = (torch.randn(N, h, generator=g) * 1.5).to(torch.bfloat16).cuda()
    C = torch.randn(h, G + 2, r, generator=g)
    if c_scale == "mixed":
        C = C * torch.logspace(-6, -1, h).reshape(h, 1, 1)      # per-key magnitudes from 1e-6 to 0.1
    else:
        C = C * c_scale
    C = C.to(torch.bfloat16).cuda()
    go = torch.randn(N, h + r, generator=g).to(torch.bfloat16).cuda()
    _, d32 = ops.feature_forward(z, C, LO, HI, G, "relu_sq", 1.0, delta_f32=True, impl="tcgen05")
    dz, dC, _ = ops.feature_backward(z, C, go[:, h:], LO, HI, G, "identity", 1.0, with_base=False, impl="tcgen05")
    _, d_ref = util.oracle_forward(z, C, LO, HI, G, "relu_sq", 1.0)
    dz_ref, dC_ref = util.oracle_backward(z, C, go[:, h:], LO, HI, G, "identity", 1.0, with_base=False)
    assert np.abs(d_ref).max() > 0 and np.abs(dz_ref).max() > 0
    util.assert_parity("delta f32", d32, d_ref, torch.bfloat16, rel_gate=2e-3)
    util.assert_parity("dz_spline", dz, dz_ref, torch.bfloat16)
    util.assert_parity("dC", dC, dC_ref, torch.bfloat16)
    ops.check_status(z.device)


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[1] % 16 == 0 and s[2] <= 32 and s[3] <= 22 and s[3] % 2 == 0]
                         + [(1, 16, 16, 22), (129, 32, 32, 22), (385, 48, 32, 10)], ids=_sid)
def test_fused_backward_matches_the_two_kernel_backward(shape):
    """The one-kernel form of the backward (dz and dC roles in one CTA) against the default two
    kernels and the oracle: dz bit for bit, dC up to the order of the token sum."""
    from sparsespline_ffn_b200 import _lib
    N, h, r, L = shape
    G = L - 2
    z, C, go = util.make_inputs(N, h, r, G, torch.bfloat16)
    _impl_or_skip("tcgen05", z, C, G)
    lib = _lib.load()
    dz0, dC0, _ = ops.feature_backward(z, C, go, LO, HI, G, "relu_sq", 0.5, impl="tcgen05")
    lib.skv_debug_set(_lib.SKV_DEBUG_FUSED_BACKWARD, 1)
    try:
        launches = int(lib.skv_kernel_launches())
        dz1, dC1, _ = ops.feature_backward(z, C, go, LO, HI, G, "relu_sq", 0.5, impl="tcgen05")
        launches = int(lib.skv_kernel_launches()) - launches
        dz2, dC2, _ = ops.feature_backward(z, C, go[:, h:], LO, HI, G, "identity", 0.5, with_base=False,
                                           impl="tcgen05")
    finally:
        lib.skv_debug_set(_lib.SKV_DEBUG_FUSED_BACKWARD, 0)
    assert launches == 6, "the fused path launches amax x2, two packs, the fused kernel and the reduce"
    assert torch.equal(dz0, dz1)
    scale = dC0.abs().max().item()
    assert (dC0 - dC1).abs().max().item() <= 1e-5 * scale
    dz_ref, dC_ref = util.oracle_backward(z, C, go, LO, HI, G, "relu_sq", 0.5)
    util.assert_parity("dz (fused)", dz1, dz_ref, torch.bfloat16)
    util.assert_parity("dC (fused)", dC1, dC_ref, torch.bfloat16, bias=True)
    dz2_ref, dC2_ref = util.oracle_backward(z, C, go[:, h:], LO, HI, G, "identity", 0.5, with_base=False)
    util.assert_parity("dz_spline (fused)", dz2, dz2_ref, torch.bfloat16)
    util.assert_parity("dC delta-only (fused)", dC2, dC2_ref, torch.bfloat16, bias=True)
    ops.check_status(z.device)


@pytest.mark.parametrize("L", [9, 15, 21, 22, 23, 24, 31, 32, 33, 41, 42])
def test_knot_counts_resolve_to_the_tensor_core_kernels(L):
    """Odd knot-row counts and every count up to the G = 40 grid get the tcgen05 kernels, not the
    CUDA-core fallback (the reference's fastest forward takes L = 16, 22 and 32 only,
    src/sparsespline_ffn/cuda_ext/spline_kv_fwd_v11.cu:382-392)."""
    z = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
    C = torch.zeros(64, L, 32, dtype=torch.bfloat16, device="cuda")
    assert ops.resolve_impl(z, C, LO, HI, L - 2) == "tcgen05"
