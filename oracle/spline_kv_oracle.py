"""CPU oracle for the RL-Spline-KV feature path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain numpy, the algorithm of the reference package's
PyTorch oracle.  It is the checker that the CUDA kernels are compared against;
nothing in the shipped package may import it.  Only ``tests/``, the smoke entry
and the benchmark's CPU-baseline leg use it.

Reference functions restated here (paths inside the reference project):

* knot interval + quadratic B-spline weights
    ``src/sparsespline_ffn/rl_spline_kv_reference.py:88-109`` (``_b2_basis_and_bins``)
    ``src/sparsespline_ffn/kernels/flash_spline_feature_backward_ref.py:48-68``
* base-path activation
    ``src/sparsespline_ffn/rl_spline_kv_reference.py:78-85`` (``_activation``)
* feature forward ``f = [phi(z); lambda * delta]``
    ``src/sparsespline_ffn/rl_spline_kv_reference.py:145-203``
* analytic backward ``dC``/``dz_spline`` and the two masks (forward mask for
  ``dC``, clamp mask for ``dz``)
    ``src/sparsespline_ffn/kernels/flash_spline_feature_backward_ref.py:71-150``
* base-path gradient, lambda chain rule, split of ``grad_output``
    ``src/sparsespline_ffn/kernels/flash_spline_feature_autograd.py:146-152, 226-242``

Parity is pinned: ``tests/golden/`` holds outputs of the reference itself
(imported from its source tree by ``tests/golden/make_golden.py``) and
``tests/test_oracle_golden.py`` checks this module against every one of them.

Arithmetic conventions.  All inputs are taken as float32 (bf16 tensors are
up-cast by the caller before they get here, which is exact).  The knot index
is computed exactly as the reference does it in float32:
``u = fl(fl(z - lo) * scale)`` with ``scale = float32(G / (hi - lo))`` where the
division is done in double; the index is therefore bit-reproducible.  Sums
over keys (forward) and over tokens (``dC``) are accumulated in float64, so the
oracle is closer to the exact value than any float32 summation order.
"""
from __future__ import annotations

import math

import numpy as np

_erf = np.vectorize(math.erf, otypes=[np.float64])

ACTIVATIONS = ("relu_sq", "identity", "gelu")


def grid_scale(grid_lo: float, grid_hi: float, G: int) -> np.float32:
    """``scale = G / (hi - lo)`` in double, rounded once to float32."""
    return np.float32(float(G) / (float(grid_hi) - float(grid_lo)))


def knot_index_and_basis(z32: np.ndarray, grid_lo: float, grid_hi: float, G: int):
    """Knot interval and the three non-zero quadratic B-spline weights.

    Returns ``(bin, B, dB, in_range, clamp_active)`` where ``bin`` is int32 in
    ``[0, G-1]``, ``B`` and ``dB`` are ``[3, ...]`` float32 stacks *without* any
    mask applied, ``in_range = 0 <= u <= G`` (masks the forward weights and so
    ``dC``) and ``clamp_active = 0 <= u <= G-1`` (masks ``dz``: it is where the
    derivative of ``clamp(u, 0, G-1)`` is one).
    """
    z32 = np.asarray(z32, dtype=np.float32)
    lo = np.float32(grid_lo)
    scale = grid_scale(grid_lo, grid_hi, G)
    u = (z32 - lo) * scale                      # two float32 roundings, no fma
    in_range = (u >= np.float32(0.0)) & (u <= np.float32(G))
    clamp_active = (u >= np.float32(0.0)) & (u <= np.float32(G - 1))
    u_c = np.minimum(np.maximum(u, np.float32(0.0)), np.float32(G - 1))
    b = np.floor(u_c)
    tau = np.clip(u_c - b, np.float32(0.0), np.float32(1.0)).astype(np.float32)
    omt = np.float32(1.0) - tau
    half = np.float32(0.5)
    two = np.float32(2.0)
    B0 = half * omt * omt
    B1 = half * (np.float32(1.0) + two * tau - two * tau * tau)
    B2 = half * tau * tau
    dB0 = -omt
    dB1 = np.float32(1.0) - two * tau
    dB2 = tau
    return (b.astype(np.int32), np.stack([B0, B1, B2]), np.stack([dB0, dB1, dB2]),
            in_range, clamp_active)


def knot_index(z32: np.ndarray, grid_lo: float, grid_hi: float, G: int) -> np.ndarray:
    """Only the knot-interval index (int32), for the bit-exact comparison."""
    return knot_index_and_basis(z32, grid_lo, grid_hi, G)[0]


def activation(z32: np.ndarray, name: str) -> np.ndarray:
    if name == "relu_sq":
        return np.where(z32 > 0, z32 * z32, np.float32(0.0)).astype(np.float32)
    if name == "identity":
        return np.asarray(z32, dtype=np.float32)
    if name == "gelu":          # F.gelu: the exact erf form
        z = np.asarray(z32, dtype=np.float64)
        return (0.5 * z * (1.0 + _erf(z * 0.7071067811865476))).astype(np.float32)
    raise ValueError(name)


def activation_grad(z32: np.ndarray, name: str) -> np.ndarray:
    if name == "relu_sq":
        return np.where(z32 > 0, np.float32(2.0) * z32, np.float32(0.0)).astype(np.float32)
    if name == "identity":
        return np.ones_like(z32, dtype=np.float32)
    if name == "gelu":          # Phi(z) + z * pdf(z), what autograd returns for F.gelu
        z = np.asarray(z32, dtype=np.float64)
        return (0.5 * (1.0 + _erf(z * 0.7071067811865476))
                + z * np.exp(-0.5 * z * z) * 0.3989422804014327).astype(np.float32)
    raise ValueError(name)


def _check_shapes(z32, C32, G):
    if z32.ndim != 2:
        raise ValueError(f"z must be 2D [N, h], got {z32.shape}")
    N, h = z32.shape
    hC, L, r = C32.shape
    if hC != h:
        raise ValueError(f"C[0]={hC} != h={h}")
    if L != G + 2:
        raise ValueError(f"L={L} should equal G+2={G + 2}")
    return N, h, L, r


def delta_forward(z32, C32, grid_lo, grid_hi, G, chunk: int = 256) -> np.ndarray:
    """Unscaled spline residual ``delta[N, r]`` as float64 (sum over keys in double)."""
    z32 = np.asarray(z32, dtype=np.float32)
    C32 = np.asarray(C32, dtype=np.float32)
    N, h, L, r = _check_shapes(z32, C32, G)
    out = np.zeros((N, r), dtype=np.float64)
    keys = np.arange(h)[None, :]
    C64 = C32.astype(np.float64)
    for s in range(0, N, chunk):
        zz = z32[s:s + chunk]
        b, B, _, in_range, _ = knot_index_and_basis(zz, grid_lo, grid_hi, G)
        acc = np.zeros((zz.shape[0], r), dtype=np.float64)
        for k in range(3):
            w = (B[k] * in_range.astype(np.float32)).astype(np.float64)     # [n, h]
            acc += np.einsum("nj,njc->nc", w, C64[keys, b + k, :])
        out[s:s + chunk] = acc
    return out


def feature_forward(z32, C32, grid_lo, grid_hi, G, activation_name="relu_sq",
                    lambda_scale=1.0, chunk: int = 256) -> np.ndarray:
    """``f = [phi(z); lambda * delta]`` as float32 ``[N, h + r]``."""
    z32 = np.asarray(z32, dtype=np.float32)
    a = activation(z32, activation_name)
    d = delta_forward(z32, C32, grid_lo, grid_hi, G, chunk) * float(lambda_scale)
    return np.concatenate([a, d.astype(np.float32)], axis=1)


def delta_backward(z32, C32, g_delta32, grid_lo, grid_hi, G, chunk: int = 256):
    """Analytic ``(dC [h, L, r] float64, dz_spline [N, h] float64)`` for a gradient
    ``g_delta`` taken with respect to the *unscaled* ``delta``."""
    z32 = np.asarray(z32, dtype=np.float32)
    C32 = np.asarray(C32, dtype=np.float32)
    g = np.asarray(g_delta32, dtype=np.float32).astype(np.float64)
    N, h, L, r = _check_shapes(z32, C32, G)
    if g.shape != (N, r):
        raise ValueError(f"g_delta must be [N, r]={(N, r)}, got {g.shape}")
    scale = float(grid_scale(grid_lo, grid_hi, G))
    C64 = C32.astype(np.float64)
    dC = np.zeros((h, L, r), dtype=np.float64)
    dz = np.zeros((N, h), dtype=np.float64)
    keys = np.arange(h)[None, :]
    for s in range(0, N, chunk):
        zz = z32[s:s + chunk]
        gg = g[s:s + chunk]
        n = zz.shape[0]
        b, B, dB, in_range, clamp_active = knot_index_and_basis(zz, grid_lo, grid_hi, G)
        kk = np.broadcast_to(keys, (n, h))
        for k in range(3):
            w = (B[k] * in_range.astype(np.float32)).astype(np.float64)
            contrib = w[:, :, None] * gg[:, None, :]                       # [n, h, r]
            np.add.at(dC, (kk.reshape(-1), (b + k).reshape(-1)), contrib.reshape(n * h, r))
            dw = (dB[k] * clamp_active.astype(np.float32)).astype(np.float64)
            inner = np.einsum("njc,nc->nj", C64[keys, b + k, :], gg)
            dz[s:s + chunk] += dw * inner
    dz *= scale
    return dC, dz


def feature_backward(z32, C32, grad_out32, grid_lo, grid_hi, G, activation_name="relu_sq",
                     lambda_scale=1.0, chunk: int = 256):
    """Gradients of ``feature_forward`` for an upstream ``grad_out [N, h + r]``.

    Returns ``(dz [N, h] float64, dC [h, L, r] float64)``:
    ``dz = g_a * phi'(z) + dz_spline`` and both spline terms carry the lambda
    chain-rule factor.
    """
    z32 = np.asarray(z32, dtype=np.float32)
    go = np.asarray(grad_out32, dtype=np.float32)
    h = z32.shape[1]
    g_a = go[:, :h].astype(np.float64)
    g_d = go[:, h:]
    dC, dz_s = delta_backward(z32, C32, g_d, grid_lo, grid_hi, G, chunk)
    lam = float(lambda_scale)
    dz = g_a * activation_grad(z32, activation_name).astype(np.float64) + lam * dz_s
    return dz, lam * dC


def parity_stats(test, ref):
    """``(maxabs(diff)/maxabs(ref), max elementwise rel with 1e-6 floor, mean signed diff)``.

    The first is the gated figure (the reference's probe scripts gate on it,
    ``benchmarks/modal_h100_bwd_v5_n_scaling.py:75-89``); the other two are the
    statistics of ``tests/test_rlkv_kernel_parity.py:153-168``.
    """
    t = np.asarray(test, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    d = t - r
    ref_max = max(float(np.abs(r).max()), 1e-30)
    return (float(np.abs(d).max()) / ref_max,
            float((np.abs(d) / np.maximum(np.abs(r), 1e-6)).max()),
            float(d.mean()))
