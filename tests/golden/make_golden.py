"""Generate the golden vectors in this folder by running the reference itself.

Run where the reference source tree is available:

    python tests/golden/make_golden.py --reference-src <reference>/src

It imports the reference's own PyTorch oracle (``flash_spline_feature_reference``,
``_b2_basis_and_bins``, ``flash_spline_delta_backward_ref`` and the CPU path of
``FlashSplineFeature`` / ``FlashSplineDelta``), evaluates it in float32 on small
seeded inputs and stores inputs and outputs in ``spline_kv_golden.npz``; a second
file, ``module_golden.npz``, holds one forward + backward of the reference's
``RLSplineKVReference`` layer per mode (additive, gelu base, no_base, multiplicative
gate), and ``b1_golden.npz`` the linear spline (``spline_order = 1``) of the reference's
oracle with its autograd gradients.  The fixtures travel with the repository; the reference does not have to be
present when the tests run.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def cases():
    g = torch.Generator().manual_seed(0)

    def rn(*shape, scale=1.0):
        return torch.randn(*shape, generator=g, dtype=torch.float32) * scale

    out = {}
    # the reference parity harness distribution: z = 2*randn, C = 0.1*randn, grid [-3, 3]
    out["uniform"] = dict(z=rn(48, 24, scale=2.0), C=rn(24, 10, 8, scale=0.1), lo=-3.0, hi=3.0,
                          G=8, act="relu_sq", lam=1.0)
    # production-like: G=20, r=32, grid [-5, 5], lambda warm-up value, bf16-representable inputs
    out["d20_like"] = dict(z=bf16_round(rn(32, 40, scale=2.5)), C=bf16_round(rn(40, 22, 32, scale=0.02)),
                           lo=-5.0, hi=5.0, G=20, act="relu_sq", lam=0.25)
    # skewed and collapsed pre-activations (the reference's backward stress workloads)
    out["skewed"] = dict(z=rn(40, 16, scale=0.5) + 2.0, C=rn(16, 22, 16, scale=0.1), lo=-3.0, hi=3.0,
                         G=20, act="relu_sq", lam=1.0)
    out["collapsed"] = dict(z=rn(40, 16, scale=0.05), C=rn(16, 22, 16, scale=0.1), lo=-3.0, hi=3.0,
                            G=20, act="identity", lam=0.5)
    # edge values: knots, grid ends, one ulp either side, far outside, infinities
    lo, hi, G = -3.0, 3.0, 12
    knots = torch.linspace(lo, hi, G + 1, dtype=torch.float32)
    specials = torch.cat([
        knots,
        torch.nextafter(knots, torch.full_like(knots, 10.0)),
        torch.nextafter(knots, torch.full_like(knots, -10.0)),
        torch.tensor([0.0, -0.0, 2.5, 2.4999998, 2.5000002, 100.0, -100.0, 1e30, -1e30,
                      float("inf"), float("-inf"), 1e-30, -1e-30], dtype=torch.float32),
    ])
    n = specials.numel()
    h = 6
    z = specials[:, None].repeat(1, h) + torch.arange(h, dtype=torch.float32)[None, :] * 0.0
    z[:, 1] = specials.flip(0)
    z[:, 2] = rn(n, scale=3.0)
    out["edges"] = dict(z=z, C=rn(h, G + 2, 8, scale=0.1), lo=lo, hi=hi, G=G, act="relu_sq", lam=1.0)
    # gelu base path (drawn last, so that the cases above keep their values)
    out["gelu"] = dict(z=rn(36, 24, scale=1.5), C=rn(24, 18, 16, scale=0.1), lo=-4.0, hi=4.0,
                       G=16, act="gelu", lam=0.75)
    return out


MODULE_CASES = {
    # name -> extra config fields of the reference's RLSplineKVConfig
    "additive": dict(),
    "additive_gelu": dict(activation="gelu"),
    "no_base": dict(no_base=True),
    "multiplicative": dict(gating_mode="multiplicative"),
    "additive_linear": dict(spline_order=1),
}


def module_fixture(reference_src):
    """One forward + backward of the reference's RLSplineKVReference module (CPU, float32, its own
    PyTorch path) per mode: inputs, parameters, output and every gradient, in module_golden.npz."""
    sys.path.insert(0, reference_src)
    from sparsespline_ffn.rl_spline_kv_reference import RLSplineKVConfig, RLSplineKVReference  # noqa: E402

    store = {}
    for i, (name, extra) in enumerate(MODULE_CASES.items()):
        torch.manual_seed(100 + i)
        cfg = RLSplineKVConfig(d=32, h_ratio=2.0, r=16, G=20, grid_lo=-3.0, grid_hi=3.0, lambda_scale=0.5,
                               c_init_std=0.05, use_kernel=False, **extra)
        m = RLSplineKVReference(cfg)
        m.train()                                        # no diagnostics pass
        with torch.no_grad():
            m.K.weight.mul_(2.0)                         # spread z over more knot intervals
            if m.W_d_proj is not None:
                m.W_d_proj.weight.mul_(30.0)             # a gate that visibly departs from 1
        x = torch.randn(3, 16, cfg.d).requires_grad_(True)
        gy = torch.randn(3, 16, cfg.d)
        y = m(x)
        y.backward(gy)
        rec = dict(x=x.detach(), gy=gy, y=y.detach(), dx=x.grad)
        for pname, prm in m.named_parameters():
            rec["param." + pname] = prm.detach()
            rec["grad." + pname] = prm.grad
        for k, v in rec.items():
            store[f"{name}/{k}"] = v.numpy()
    path = os.path.join(HERE, "module_golden.npz")
    np.savez_compressed(path, **store)
    print(path, os.path.getsize(path), "bytes;", len(store), "arrays")


def b1_fixture(reference_src):
    """The linear B-spline (spline_order = 1, L = G + 1) of the reference's PyTorch oracle
    (rl_spline_kv_reference.py:125-142, 178-187): f and, through autograd, dz and dC, in b1_golden.npz."""
    sys.path.insert(0, reference_src)
    from sparsespline_ffn.rl_spline_kv_reference import flash_spline_feature_reference  # noqa: E402

    g = torch.Generator().manual_seed(11)

    def rn(*shape, scale=1.0):
        return torch.randn(*shape, generator=g, dtype=torch.float32) * scale

    cases = {
        "uniform": dict(z=rn(48, 24, scale=2.0), C=rn(24, 9, 8, scale=0.1), lo=-3.0, hi=3.0, G=8, act="relu_sq", lam=1.0),
        "d20_like": dict(z=bf16_round(rn(32, 40, scale=2.5)), C=bf16_round(rn(40, 21, 32, scale=0.02)),
                         lo=-5.0, hi=5.0, G=20, act="relu_sq", lam=0.25),
        "gelu": dict(z=rn(36, 24, scale=1.5), C=rn(24, 17, 16, scale=0.1), lo=-4.0, hi=4.0, G=16, act="gelu", lam=0.75),
    }
    lo, hi, G = -3.0, 3.0, 12
    knots = torch.linspace(lo, hi, G + 1, dtype=torch.float32)
    specials = torch.cat([knots, torch.nextafter(knots, torch.full_like(knots, 10.0)),
                          torch.nextafter(knots, torch.full_like(knots, -10.0)),
                          torch.tensor([0.0, -0.0, 100.0, -100.0, 1e30, -1e30, 1e-30], dtype=torch.float32)])
    cases["edges"] = dict(z=specials[:, None].repeat(1, 4), C=rn(4, G + 1, 8, scale=0.1), lo=lo, hi=hi, G=G,
                          act="identity", lam=1.0)
    store = {}
    for name, c in cases.items():
        z, C = c["z"], c["C"]
        N, h = z.shape
        r = C.shape[-1]
        go = torch.randn(N, h + r, generator=g, dtype=torch.float32)
        zt = z.clone().requires_grad_(True)
        Ct = C.clone().requires_grad_(True)
        f = flash_spline_feature_reference(zt, Ct, c["lo"], c["hi"], c["G"], activation=c["act"],
                                           lambda_scale=c["lam"], spline_order=1)
        f.backward(go)
        rec = dict(z=z, C=C, go=go, f=f.detach(), dz=zt.grad, dC=Ct.grad,
                   meta=torch.tensor([c["lo"], c["hi"], float(c["G"]), c["lam"],
                                      {"relu_sq": 0.0, "identity": 1.0, "gelu": 2.0}[c["act"]]], dtype=torch.float64))
        for k, v in rec.items():
            store[f"{name}/{k}"] = v.detach().numpy()
    path = os.path.join(HERE, "b1_golden.npz")
    np.savez_compressed(path, **store)
    print(path, os.path.getsize(path), "bytes;", len(store), "arrays")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True)
    ap.add_argument("--only", choices=["operator", "module", "b1"], help="regenerate one of the fixture files")
    args = ap.parse_args()
    torch.set_num_threads(1)          # the reference's scatter-add backward is order-dependent across threads
    if args.only in (None, "module"):
        module_fixture(args.reference_src)
    if args.only in (None, "b1"):
        b1_fixture(args.reference_src)
    if args.only in ("module", "b1"):
        return
    sys.path.insert(0, args.reference_src)
    from sparsespline_ffn.rl_spline_kv_reference import (  # noqa: E402
        _b2_basis_and_bins, flash_spline_feature_reference)
    from sparsespline_ffn.kernels.flash_spline_feature_backward_ref import (  # noqa: E402
        flash_spline_delta_backward_ref)
    from sparsespline_ffn.kernels.flash_spline_feature_autograd import (  # noqa: E402
        flash_spline_delta, flash_spline_feature)

    torch.set_num_threads(1)
    store = {}
    gg = torch.Generator().manual_seed(7)
    for name, c in cases().items():
        z, C = c["z"], c["C"]
        N, h = z.shape
        r = C.shape[-1]
        lo, hi, G, act, lam = c["lo"], c["hi"], c["G"], c["act"], c["lam"]
        go = torch.randn(N, h + r, generator=gg, dtype=torch.float32)
        bins, B0, B1, B2, in_range = _b2_basis_and_bins(z, lo, hi, G)
        f = flash_spline_feature_reference(z, C, lo, hi, G, activation=act, lambda_scale=lam)
        # gradients through the reference Function's CPU path (reference recomputation)
        finite = torch.isfinite(z).all()
        zt = z.clone().requires_grad_(True)
        Ct = C.clone().requires_grad_(True)
        fo = flash_spline_feature(zt, Ct, lo, hi, G, act, lam, use_kernel=False)
        fo.backward(go)
        dz, dC = zt.grad.clone(), Ct.grad.clone()
        # delta-only operator
        zt2 = z.clone().requires_grad_(True)
        Ct2 = C.clone().requires_grad_(True)
        d = flash_spline_delta(zt2, Ct2, lo, hi, G, lam, "triton")
        d.backward(go[:, h:].contiguous())
        # analytic backward reference (gradient w.r.t. unscaled delta)
        dC_an, dzs_an = flash_spline_delta_backward_ref(z, C, go[:, h:].contiguous(), lo, hi, G)
        rec = dict(z=z, C=C, go=go, bins=bins.to(torch.int32), B=torch.stack([B0, B1, B2]),
                   in_range=in_range.to(torch.uint8), f=f, dz=dz, dC=dC,
                   delta_only=d.detach(), delta_dz=zt2.grad, delta_dC=Ct2.grad,
                   analytic_dC=dC_an, analytic_dz_spline=dzs_an,
                   meta=torch.tensor([lo, hi, float(G), lam, {"relu_sq": 0.0, "identity": 1.0, "gelu": 2.0}[act],
                                      1.0 if bool(finite) else 0.0], dtype=torch.float64))
        for k, v in rec.items():
            store[f"{name}/{k}"] = v.detach().numpy()
    path = os.path.join(HERE, "spline_kv_golden.npz")
    np.savez_compressed(path, **store)
    print(path, os.path.getsize(path), "bytes;", len(store), "arrays")


if __name__ == "__main__":
    main()
