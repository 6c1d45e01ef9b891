"""The two sharded modes rehearsed with CPU ranks over gloo (world size 2): the local compute is
replaced by the oracle so that only the partitioning and the collectives are under test."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import c_binding as oc

LO, HI, G, ACT, LAM = -3.0, 3.0, 20, "relu_sq", 0.5


def _oracle_forward(z, C, lo, hi, G_, act, lam, with_base, delta_f32):
    a, d = oc.feature_forward(z.float().numpy(), C.float().numpy(), lo, hi, G_, act, lam)
    a_t = torch.from_numpy(a).to(z.dtype) if with_base else None
    d_t = torch.from_numpy(d)
    if delta_f32:
        return a_t, d_t
    return torch.cat([a_t, d_t.to(z.dtype)], dim=1) if with_base else d_t.to(z.dtype)


def _oracle_backward(z, C, go, lo, hi, G_, act, lam, with_base, need_dz, need_dC):
    h = z.shape[1]
    if isinstance(go, (tuple, list)):                 # the key-sharded mode passes (g_act, g_delta)
        g_a, g_d = go[0].float().numpy(), go[1].float().numpy()
    else:
        g = go.float().numpy()
        g_a, g_d = (g[:, :h], g[:, h:]) if with_base else (None, g)
    dz, dC = oc.feature_backward(z.float().numpy(), C.float().numpy(), g_d, g_a, lo, hi, G_, act, lam)
    return (torch.from_numpy(dz).to(z.dtype) if need_dz else None,
            torch.from_numpy(dC.astype(np.float32)) if need_dC else None)


def _inputs():
    g = torch.Generator().manual_seed(11)
    N, h, r = 96, 48, 16
    z = torch.randn(N, h, generator=g) * 2
    C = torch.randn(h, G + 2, r, generator=g) * 0.1
    go = torch.randn(N, h + r, generator=g)
    return z, C, go


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sparsespline_ffn_b200 import sharded
        sharded._local_forward = _oracle_forward
        sharded._local_backward = _oracle_backward
        z, C, go = _inputs()
        N, h = z.shape
        # token-sharded: local tokens, replicated C, dC all-reduced
        ts = sharded.token_slice(N, world, rank)
        zl = z[ts].clone().requires_grad_(True)
        Cr = C.clone().requires_grad_(True)
        f = sharded.token_sharded_spline_feature(zl, Cr, LO, HI, G, ACT, LAM)
        f.backward(go[ts])
        # key-sharded: local keys, all tokens, partial residual all-reduced
        ks = sharded.key_slice(h, world, rank)
        zk = z[:, ks].clone().requires_grad_(True)
        Ck = C[ks].clone().requires_grad_(True)
        a_loc, delta = sharded.key_sharded_spline_feature(zk, Ck, LO, HI, G, ACT, LAM)
        (a_loc * go[:, :h][:, ks]).sum().backward(retain_graph=True)
        delta.backward(go[:, h:])
        results[rank] = dict(ts=(ts.start, ts.stop), ks=(ks.start, ks.stop), f=f.detach(), dz=zl.grad,
                             dC=Cr.grad, delta=delta.detach(), a_loc=a_loc.detach(), dzk=zk.grad, dCk=Ck.grad)
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_slices_cover_everything():
    from sparsespline_ffn_b200 import sharded
    for n, w in [(65536, 8), (10, 4), (7, 8), (96, 2)]:
        idx = [i for r in range(w) for i in range(*sharded.token_slice(n, w, r).indices(n))]
        assert idx == list(range(n))
    for h, w in [(5120, 8), (48, 2), (40, 4), (8, 4)]:
        idx = [i for r in range(w) for i in range(*sharded.key_slice(h, w, r).indices(h))]
        assert idx == list(range(h))
        assert all(sharded.key_slice(h, w, r).start % 8 == 0 for r in range(w))


@pytest.mark.timeout(300)
def test_token_and_key_sharded_modes_world2():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    z, C, go = _inputs()
    N, h = z.shape
    f_ref = _oracle_forward(z, C, LO, HI, G, ACT, LAM, True, False)
    dz_ref, dC_ref = _oracle_backward(z, C, go, LO, HI, G, ACT, LAM, True, True, True)
    for rank in range(world):
        r = results[rank]
        ts = slice(*r["ts"])
        ks = slice(*r["ks"])
        # token-sharded
        assert torch.allclose(r["f"], f_ref[ts], atol=1e-6)
        assert torch.allclose(r["dz"], dz_ref[ts], atol=1e-5)
        assert torch.allclose(r["dC"], dC_ref, rtol=1e-5, atol=1e-5)       # identical on every rank
        # key-sharded
        assert torch.allclose(r["delta"], f_ref[:, h:], rtol=1e-5, atol=1e-6)
        assert torch.allclose(r["a_loc"], f_ref[:, :h][:, ks], atol=1e-6)
        assert torch.allclose(r["dzk"], dz_ref[:, ks], rtol=1e-4, atol=1e-5)
        assert torch.allclose(r["dCk"], dC_ref[ks], rtol=1e-4, atol=1e-5)
    assert torch.equal(results[0]["dC"], results[1]["dC"])
