"""Signed-bias report of the tensor-core kernels on their float32 outputs.

The reference gates the mean signed error of its kernels against each other at 5e-6
(tests/test_rlkv_kernel_parity.py:342-371, "Regime B"); a systematic (non-zero-mean) error is what
made its bf16-basis forward diverge in training (src/sparsespline_ffn/cuda_ext/spline_kv_fwd_v11.cu:3-6).
Here every output is compared before its rounding to bf16: the residual (``delta_f32``), ``dz``
(``dz_f32``) and ``dC`` (always float32).  The gate is |mean signed error| <= 5e-6 x max(1, maxabs(ref)):
absolute where the reference values are O(1) or smaller, relative to the largest reference value where
they are larger (dC grows with the token count: one bf16 ulp of a value near 100 is already 0.5).  The
measured numbers are printed (run with -s to see them) for both forms of the backward.
"""
import json

import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("sparsespline_ffn_b200.ops")
_lib = pytest.importorskip("sparsespline_ffn_b200._lib")

# name -> (N, h, r, G, grid, lambda, z mean, z std)
CASES = {
    "config1_like": (2048, 512, 32, 20, (-5.0, 5.0), 1.0, 0.0, 1.0),
    "config2_like": (2048, 512, 32, 20, (-5.0, 5.0), 0.25, 0.0, 2.0),     # ~1 % of z outside the grid
    "G40": (1024, 256, 32, 40, (-5.0, 5.0), 1.0, 0.0, 1.0),
    "r128": (1024, 256, 128, 20, (-5.0, 5.0), 1.0, 0.0, 1.0),
    "skewed": (2048, 256, 32, 20, (-3.0, 3.0), 1.0, 2.0, 0.5),
    "collapsed": (2048, 256, 32, 20, (-3.0, 3.0), 1.0, 0.0, 0.05),
}


def _inputs(N, h, r, G, mean, std, seed=5):
    g = torch.Generator().manual_seed(seed)
    z = (torch.randn(N, h, generator=g) * std + mean).to(torch.bfloat16).cuda()
    C = (torch.randn(h, G + 2, r, generator=g) * 0.02).to(torch.bfloat16).cuda()
    go = torch.randn(N, h + r, generator=g).to(torch.bfloat16).cuda()
    return z, C, go


def _entry(test, ref):
    rel, _, bias = util.stats(test, ref)
    ref_max = float(np.abs(ref).max())
    return dict(rel=rel, mean_signed=bias, mean_signed_rel=bias / max(1.0, ref_max), ref_max=ref_max)


@pytest.mark.parametrize("fused", [False, True], ids=["two_kernels", "fused"])
@pytest.mark.parametrize("case", sorted(CASES))
def test_signed_bias_of_float32_outputs(case, fused):
    N, h, r, G, (lo, hi), lam, mean, std = CASES[case]
    z, C, go = _inputs(N, h, r, G, mean, std)
    if ops.resolve_impl(z, C, lo, hi, G) != "tcgen05":
        pytest.skip("shape not eligible for the tcgen05 kernels")
    lib = _lib.load()
    lib.skv_debug_set(_lib.SKV_DEBUG_FUSED_BACKWARD, 1 if fused else 0)
    try:
        _, d32 = ops.feature_forward(z, C, lo, hi, G, "relu_sq", lam, delta_f32=True, impl="tcgen05")
        dz32, dC32, _ = ops.feature_backward(z, C, go, lo, hi, G, "relu_sq", lam, impl="tcgen05", dz_f32=True)
    finally:
        lib.skv_debug_set(_lib.SKV_DEBUG_FUSED_BACKWARD, 0)
    ops.check_status(z.device)
    assert dz32.dtype == torch.float32
    _, d_ref = util.oracle_forward(z, C, lo, hi, G, "relu_sq", lam)
    dz_ref, dC_ref = util.oracle_backward(z, C, go, lo, hi, G, "relu_sq", lam)
    report = dict(case=case, backward="fused" if fused else "two kernels",
                  delta=_entry(d32, d_ref), dz=_entry(dz32, dz_ref), dC=_entry(dC32, dC_ref))
    print("BIAS " + json.dumps(report))
    for name in ("delta", "dz", "dC"):
        e = report[name]
        assert e["rel"] <= 1e-2, (name, e)
        assert abs(e["mean_signed_rel"]) <= util.BIAS_GATE, (name, e)


def test_dz_f32_rounds_to_the_bf16_result():
    """The float32 dz is the same arithmetic as the bf16 one: rounding it gives the bf16 tensor."""
    z, C, go = _inputs(512, 128, 32, 20, 0.0, 1.5)
    dz32, _, _ = ops.feature_backward(z, C, go, -5.0, 5.0, 20, "relu_sq", 0.5, impl="tcgen05", dz_f32=True)
    dz16, _, _ = ops.feature_backward(z, C, go, -5.0, 5.0, 20, "relu_sq", 0.5, impl="tcgen05")
    assert torch.equal(dz32.to(torch.bfloat16), dz16)
