"""A stack of RL-Spline-KV layers (the late-layer configuration of the reference's d20 runs, at a
small size): x -> z = x W_in^T -> f = feature(z, C) -> y = f W_out^T, x <- x + y, three times,
forward and backward, against the same chain evaluated with the CPU oracle in float64/float32.
The GEMMs around the operator are plain torch matmuls; what is under test is that the operator
composes correctly with autograd across layers (saved tensors, gradient splitting, dtypes)."""
import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

skv = pytest.importorskip("sparsespline_ffn_b200")

LAYERS, N, D, H, R, G = 3, 384, 96, 256, 32, 20
LO, HI, LAM = -5.0, 5.0, 0.25


def _params():
    g = torch.Generator().manual_seed(21)
    x = torch.randn(N, D, generator=g) * 2.0
    W_in = [torch.randn(H, D, generator=g) / D ** 0.5 for _ in range(LAYERS)]
    C = [torch.randn(H, G + 2, R, generator=g) * 0.02 for _ in range(LAYERS)]
    # small read-out weights keep the residual stream, and with it z, at O(1) across layers (the stack
    # has no normalisation; with large updates z leaves the grid and the comparison becomes ill-conditioned)
    W_out = [torch.randn(D, H + R, generator=g) * 0.05 / (H + R) ** 0.5 for _ in range(LAYERS)]
    go = torch.randn(N, D, generator=g)
    bf = lambda t: t.to(torch.bfloat16)
    return bf(x), [bf(w) for w in W_in], [bf(c) for c in C], [bf(w) for w in W_out], bf(go)


def _oracle_chain(x, W_in, C, W_out, go):
    """float64 chain; the operator's inputs are rounded to bf16 where the GPU path rounds them."""
    bf = lambda a: torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)
    xs, zs = [x.astype(np.float64)], []
    for l in range(LAYERS):
        z = bf(bf(xs[-1]) @ W_in[l].T)
        a, d = util.oc.feature_forward(z, C[l], LO, HI, G, "relu_sq", LAM)
        f = bf(np.concatenate([a, d], axis=1))
        y = bf(f @ W_out[l].T)
        zs.append(z)
        xs.append(bf(xs[-1] + y))
    gx = go.astype(np.float64)
    dCs = [None] * LAYERS
    for l in reversed(range(LAYERS)):
        gf = gx @ W_out[l]                                   # dL/df
        dz, dC = util.oc.feature_backward(zs[l], C[l], gf[:, H:], gf[:, :H], LO, HI, G, "relu_sq", LAM)
        dCs[l] = dC
        gx = gx + dz.astype(np.float64) @ W_in[l]
    return xs[-1], gx, dCs


def test_three_layer_stack_forward_backward():
    x, W_in, C, W_out, go = _params()
    xg = x.cuda().requires_grad_(True)
    Cg = [c.cuda().requires_grad_(True) for c in C]
    Wi = [w.cuda() for w in W_in]
    Wo = [w.cuda() for w in W_out]
    h = xg
    for l in range(LAYERS):
        z = h @ Wi[l].T
        f = skv.flash_spline_feature(z, Cg[l], LO, HI, G, "relu_sq", LAM, True)
        h = h + f @ Wo[l].T
    h.backward(go.cuda())
    f64 = lambda t: t.float().numpy().astype(np.float64)
    out_ref, gx_ref, dC_ref = _oracle_chain(f64(x), [f64(w) for w in W_in], [c.float().numpy() for c in C],
                                            [f64(w) for w in W_out], f64(go))
    util.assert_parity("stack output", h, out_ref, torch.bfloat16, rel_gate=2e-2)
    util.assert_parity("dL/dx", xg.grad, gx_ref, torch.bfloat16, rel_gate=3e-2)
    for l in range(LAYERS):
        util.assert_parity(f"dC layer {l}", Cg[l].grad, dC_ref[l], torch.bfloat16, rel_gate=3e-2)
