"""Helpers shared by the GPU parity tests: seeded inputs and the oracle as checker."""
from __future__ import annotations

import numpy as np
import torch

from oracle import c_binding as oc
from oracle import spline_kv_oracle as onp

# Gates.  Stated tolerance of the target: maxabs(diff)/maxabs(ref) <= 1e-2 for bf16 I/O against the float32
# oracle and |mean signed error| <= 5e-6 (relative to maxabs(ref) when that exceeds 1) on float32
# kernel outputs.  float32 I/O is held to 1e-4.
REL_GATE = {torch.bfloat16: 1e-2, torch.float32: 1e-4}
BIAS_GATE = 5e-6


def make_inputs(N, h, r, G, dtype, seed=0, z_scale=2.0, C_scale=0.1, device="cuda"):
    """z ~ z_scale*N(0,1) [N,h], C ~ C_scale*N(0,1) [h,G+2,r], grad [N,h+r]; CPU generator, so the
    values do not depend on the GPU, rounded to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    z = (torch.randn(N, h, generator=g) * z_scale).to(dtype)
    C = (torch.randn(h, G + 2, r, generator=g) * C_scale).to(dtype)
    go = torch.randn(N, h + r, generator=torch.Generator().manual_seed(seed + 7)).to(dtype)
    return z.to(device), C.to(device), go.to(device)


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def oracle_forward(z, C, lo, hi, G, act="relu_sq", lam=1.0):
    """(phi(z) [N,h], lambda*delta [N,r]) from the C oracle on the up-cast inputs."""
    return oc.feature_forward(f32(z), f32(C), lo, hi, G, act, lam)


def oracle_backward(z, C, go, lo, hi, G, act="relu_sq", lam=1.0, with_base=True):
    h = z.shape[1]
    g = f32(go)
    if with_base:
        return oc.feature_backward(f32(z), f32(C), g[:, h:], g[:, :h], lo, hi, G, act, lam)
    return oc.feature_backward(f32(z), f32(C), g, None, lo, hi, G, act, lam)


def stats(test, ref):
    return onp.parity_stats(f32(test) if isinstance(test, torch.Tensor) else test, ref)


def assert_parity(name, test, ref, dtype, bias=False, rel_gate=None):
    rel, elem_rel, mean_signed = stats(test, ref)
    gate = REL_GATE[dtype] if rel_gate is None else rel_gate
    msg = f"{name}: maxabs(diff)/maxabs(ref)={rel:.3e} (gate {gate:.0e}), elementwise rel={elem_rel:.3e}, mean signed={mean_signed:+.3e}"
    assert rel <= gate, msg
    if bias:
        scale = max(1.0, float(np.abs(ref).max()))
        assert abs(mean_signed) <= BIAS_GATE * scale, msg
    return msg
