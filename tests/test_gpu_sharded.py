"""The two sharded modes on real GPUs (NCCL), one process per GPU; needs at least two GPUs and
is skipped otherwise.  Every rank checks its results against the unsharded operator run locally."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

LO, HI, G, LAM = -5.0, 5.0, 20, 0.25


def _worker(rank, world, port, ok):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sparsespline_ffn_b200 import flash_spline_feature, sharded
        g = torch.Generator().manual_seed(3)
        N, h, r = 1024, 256, 32
        z = (torch.randn(N, h, generator=g) * 2).to(torch.bfloat16).cuda()
        C = (torch.randn(h, G + 2, r, generator=g) * 0.02).to(torch.bfloat16).cuda()
        go = torch.randn(N, h + r, generator=g).to(torch.bfloat16).cuda()
        zf = z.clone().requires_grad_(True)
        Cf = C.clone().requires_grad_(True)
        f_full = flash_spline_feature(zf, Cf, LO, HI, G, "relu_sq", LAM, True)
        f_full.backward(go)
        # token-sharded
        ts = sharded.token_slice(N, world, rank)
        zl = z[ts].clone().requires_grad_(True)
        Cl = C.clone().requires_grad_(True)
        f = sharded.token_sharded_spline_feature(zl, Cl, LO, HI, G, "relu_sq", LAM)
        f.backward(go[ts])
        # a different token count may split the keys differently, so sums can differ in the last bit
        assert torch.equal(f[:, :h], f_full[ts][:, :h])
        dmax = f_full[:, h:].float().abs().max().item()
        assert (f[:, h:].float() - f_full[ts][:, h:].float()).abs().max().item() <= 1e-2 * dmax
        gmax = zf.grad.float().abs().max().item()
        assert (zl.grad.float() - zf.grad[ts].float()).abs().max().item() <= 1e-2 * gmax
        assert torch.allclose(Cl.grad.float(), Cf.grad.float(), rtol=2e-2, atol=2e-2 * Cf.grad.float().abs().max().item())
        # key-sharded
        ks = sharded.key_slice(h, world, rank)
        zk = z[:, ks].contiguous().requires_grad_(True)
        Ck = C[ks].contiguous().requires_grad_(True)
        a_loc, delta = sharded.key_sharded_spline_feature(zk, Ck, LO, HI, G, "relu_sq", LAM)
        (a_loc.float() * go[:, :h][:, ks].float()).sum().backward(retain_graph=True)
        delta.backward(go[:, h:])
        assert torch.equal(a_loc, f_full[:, :h][:, ks])
        assert (delta.float() - f_full[:, h:].float()).abs().max().item() <= 1e-2 * dmax
        assert (zk.grad.float() - zf.grad[:, ks].float()).abs().max().item() <= 1e-2 * gmax
        cmax = Cf.grad.float().abs().max().item()
        assert (Ck.grad.float() - Cf.grad[ks].float()).abs().max().item() <= 1e-2 * cmax
        ok[rank] = True
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_token_and_key_sharded_on_gpus():
    import torch.multiprocessing as mp
    world = 2
    ok = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ok), nprocs=world, join=True)
    assert all(ok.get(r) for r in range(world))
