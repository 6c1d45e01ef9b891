"""The oracle (numpy and C restatements) against outputs of the reference itself.

The fixture ``tests/golden/spline_kv_golden.npz`` was produced by importing the
reference's PyTorch oracle (see ``tests/golden/make_golden.py``).  Every case
and every stored output is checked here, so the oracle's parity is pinned.
"""
import numpy as np
import pytest

from oracle import c_binding as oc
from oracle import spline_kv_oracle as onp

CASES = ["uniform", "d20_like", "skewed", "collapsed", "edges", "gelu"]


def _meta(c):
    lo, hi, G, lam, act, finite = c["meta"]
    return float(lo), float(hi), int(G), float(lam), ("relu_sq", "identity", "gelu")[int(act)], bool(finite)


def _close(a, b, rtol=2e-5, atol=2e-6):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    fin = np.isfinite(b)
    assert np.array_equal(np.isfinite(a), fin)
    np.testing.assert_allclose(a[fin], b[fin], rtol=rtol, atol=atol)


@pytest.mark.parametrize("name", CASES)
def test_knot_index_bit_exact(golden, name):
    c = golden[name]
    lo, hi, G, *_ = _meta(c)
    assert np.array_equal(onp.knot_index(c["z"], lo, hi, G), c["bins"])
    assert np.array_equal(oc.knot_index(c["z"], lo, hi, G), c["bins"])


@pytest.mark.parametrize("name", CASES)
def test_basis_weights(golden, name):
    c = golden[name]
    lo, hi, G, *_ = _meta(c)
    b, B, dB, in_range, clamp_active = onp.knot_index_and_basis(c["z"], lo, hi, G)
    assert np.array_equal(in_range.astype(np.uint8), c["in_range"])
    np.testing.assert_allclose(B, c["B"], rtol=0, atol=1e-7)
    # partition of unity
    np.testing.assert_allclose(B.sum(0), 1.0, atol=1e-6)


@pytest.mark.parametrize("name", CASES)
def test_forward(golden, name):
    c = golden[name]
    lo, hi, G, lam, act, _ = _meta(c)
    f = onp.feature_forward(c["z"], c["C"], lo, hi, G, act, lam)
    _close(f, c["f"])
    a, d = oc.feature_forward(c["z"], c["C"], lo, hi, G, act, lam)
    h = c["z"].shape[1]
    _close(a, c["f"][:, :h])
    _close(d, c["f"][:, h:])
    # the delta-only operator of the reference returns the same residual
    _close(d, c["delta_only"])


@pytest.mark.parametrize("name", CASES)
def test_backward(golden, name):
    c = golden[name]
    lo, hi, G, lam, act, finite = _meta(c)
    z, C, go = c["z"], c["C"], c["go"]
    h = z.shape[1]
    if not finite:
        # gradients at infinite z are inf/nan in the reference too; compare finite rows only
        rows = np.isfinite(z).all(axis=1)
        z, go = z[rows], go[rows]
        ref_dz = c["dz"][rows]
        dz, _ = onp.feature_backward(z, C, go, lo, hi, G, act, lam)
        _close(dz, ref_dz, rtol=1e-4, atol=1e-5)
        return
    dz, dC = onp.feature_backward(z, C, go, lo, hi, G, act, lam)
    _close(dz, c["dz"], rtol=1e-4, atol=1e-5)
    _close(dC, c["dC"], rtol=1e-4, atol=1e-5)
    dz_c, dC_c = oc.feature_backward(z, C, go[:, h:], go[:, :h], lo, hi, G, act, lam)
    _close(dz_c, c["dz"], rtol=1e-4, atol=1e-5)
    _close(dC_c, c["dC"], rtol=1e-4, atol=1e-5)
    # delta-only operator: no base path
    dz_d, dC_d = oc.feature_backward(z, C, go[:, h:], None, lo, hi, G, act, lam)
    _close(dz_d, c["delta_dz"], rtol=1e-4, atol=1e-5)
    _close(dC_d, c["delta_dC"], rtol=1e-4, atol=1e-5)
    # analytic reference (gradient w.r.t. the unscaled residual)
    dC_an, dzs_an = onp.delta_backward(z, C, go[:, h:], lo, hi, G)
    _close(dC_an, c["analytic_dC"], rtol=1e-4, atol=1e-5)
    _close(dzs_an, c["analytic_dz_spline"], rtol=1e-4, atol=1e-5)


def test_last_row_of_dC_is_never_touched(golden):
    # bin <= G-1 and k <= 2 reach row G+1 = L-1 only with weight B2(tau=0)=0 at u in (G-1, G]
    c = golden["d20_like"]
    assert np.all(c["dC"][:, -1, :] == 0) or np.abs(c["dC"][:, -1, :]).max() < 1e-6


def test_reference_invariants_hold_for_the_oracle():
    """Properties the reference's own CPU tests assert (tests/test_rl_spline_kv_reference.py:50-146)."""
    rng = np.random.default_rng(0)
    N, h, r, G = 16, 12, 8, 20
    z = rng.standard_normal((N, h)).astype(np.float32) * 2
    C = rng.standard_normal((h, G + 2, r)).astype(np.float32) * 0.1
    # C = 0 => delta exactly 0 and the base half is ReLU^2
    f0 = onp.feature_forward(z, np.zeros_like(C), -3, 3, G)
    assert np.all(f0[:, h:] == 0)
    np.testing.assert_array_equal(f0[:, :h], np.where(z > 0, z * z, 0).astype(np.float32))
    # linearity in C and lambda
    f1 = onp.feature_forward(z, C, -3, 3, G)
    f2 = onp.feature_forward(z, 2 * C, -3, 3, G)
    np.testing.assert_allclose(f2[:, h:], 2 * f1[:, h:], rtol=1e-5, atol=1e-7)
    f3 = onp.feature_forward(z, C, -3, 3, G, lambda_scale=0.25)
    np.testing.assert_allclose(f3[:, h:], 0.25 * f1[:, h:], rtol=1e-5, atol=1e-7)
    # partition of unity: C constant along the knot axis => delta constant in z, dz_spline = 0
    Cc = np.broadcast_to(rng.standard_normal((h, 1, r)).astype(np.float32), (h, G + 2, r)).copy()
    zin = np.clip(z, -2.9, 2.9)
    dC, dzs = onp.delta_backward(zin, Cc, rng.standard_normal((N, r)).astype(np.float32), -3, 3, G)
    assert np.abs(dzs).max() < 1e-5
    assert np.abs(dC).max() > 0
    # all tokens far outside the grid => delta exactly 0, finite
    f4 = onp.feature_forward(np.full((N, h), 100.0, np.float32), C, -3, 3, G)
    assert np.all(f4[:, h:] == 0) and np.isfinite(f4).all()


# ---------------------------------------------------------------------------------------------
# linear spline (spline_order = 1): the C oracle against the reference's own outputs
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def b1_golden():
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "b1_golden.npz")
    data = np.load(path)
    cases = {}
    for key in data.files:
        case, name = key.split("/")
        cases.setdefault(case, {})[name] = data[key]
    return cases


@pytest.mark.parametrize("case", ["uniform", "d20_like", "gelu", "edges"])
def test_c_oracle_linear_spline_matches_the_reference(b1_golden, case):
    from oracle import c_binding as oc
    c = b1_golden[case]
    lo, hi, G, lam = float(c["meta"][0]), float(c["meta"][1]), int(c["meta"][2]), float(c["meta"][3])
    act = {0: "relu_sq", 1: "identity", 2: "gelu"}[int(c["meta"][4])]
    z, C, go = c["z"], c["C"], c["go"]
    h = z.shape[1]
    a, d = oc.feature_forward(z, C, lo, hi, G, act, lam, spline_order=1)
    f_ref = c["f"]
    finite = np.isfinite(z)
    np.testing.assert_allclose(a[finite], f_ref[:, :h][finite], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(d, f_ref[:, h:], rtol=1e-4, atol=1e-6)
    dz, dC = oc.feature_backward(z, C, go[:, h:], go[:, :h], lo, hi, G, act, lam, spline_order=1)
    np.testing.assert_allclose(dz[finite], c["dz"][finite], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dC, c["dC"], rtol=1e-4, atol=1e-5)
    assert not dC[:, -1].any()                      # the last knot row never gets a weight
