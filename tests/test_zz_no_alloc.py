"""The allocation-free forward entry point, called through the C ABI.

`skv_feature_forward_noalloc` is for hosts that cannot call cudaMalloc where the operator runs
(servers and plugin sandboxes with a fixed device-memory budget, latency-critical loops): it carries its scratch as a fixed array inside the library.  Here it is compared with the
regular entry point (caller-owned scratch) on two calls in a row with different inputs, since all
calls share the one array, and the size limit is checked.  The file is named so that pytest
collects it last.
"""
import ctypes

import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

LO, HI, G = -3.0, 3.0, 20


def _call_noalloc(lib, _lib, z, C, lam, with_base=True):
    N, h = z.shape
    r = C.shape[2]
    p = _lib.Problem(N=N, h=h, L=G + 2, r=r, grid_lo=LO, scale=float(G) / (HI - LO), lambda_scale=lam,
                     activation=_lib.SKV_ACT["relu_sq"], dtype=_lib.SKV_BF16, impl=0, delta_f32=0)
    f = torch.empty(N, h + r if with_base else r, dtype=z.dtype, device=z.device)
    vp = ctypes.c_void_p
    act_ptr = vp(f.data_ptr()) if with_base else None
    delta_ptr = vp(f.data_ptr() + (2 * h if with_base else 0))
    rc = lib.skv_feature_forward_noalloc(ctypes.byref(p), vp(z.data_ptr()), z.stride(0), vp(C.data_ptr()),
                                         act_ptr, f.stride(0), delta_ptr, f.stride(0), None,
                                         vp(torch.cuda.current_stream().cuda_stream))
    return rc, f


def test_noalloc_forward_matches_regular_entry_point_twice_in_a_row():
    from sparsespline_ffn_b200 import _lib, ops
    lib = _lib.load()
    shapes = [(1024, 256, 32), (777, 128, 64)]
    for call, (N, h, r) in enumerate(shapes):
        z, C, _ = util.make_inputs(N, h, r, G, torch.bfloat16, seed=call + 1)
        assert ops.resolve_impl(z, C, LO, HI, G) == "tcgen05"     # the variant that uses scratch
        rc, f = _call_noalloc(lib, _lib, z, C, 0.5)
        assert rc == 0, lib.skv_error_string(rc)
        torch.cuda.synchronize()
        f_ref = ops.feature_forward(z, C, LO, HI, G, "relu_sq", 0.5)
        util.assert_parity(f"call {call}: phi(z)", f[:, :h], util.f32(f_ref[:, :h]), torch.bfloat16)
        util.assert_parity(f"call {call}: lambda*delta", f[:, h:], util.f32(f_ref[:, h:]), torch.bfloat16)
        assert torch.equal(f, f_ref)                               # same kernels, same order of sums
        # and against the oracle, like every other forward test
        _, d_ref = util.oracle_forward(z, C, LO, HI, G, "relu_sq", 0.5)
        util.assert_parity(f"call {call}: delta vs oracle", f[:, h:], d_ref, torch.bfloat16)


def test_noalloc_refuses_problems_beyond_its_array():
    from sparsespline_ffn_b200 import _lib
    lib = _lib.load()
    p = _lib.Problem(N=65536, h=5120, L=22, r=32, grid_lo=-5.0, scale=2.0, lambda_scale=1.0,
                     activation=0, dtype=_lib.SKV_BF16, impl=0, delta_f32=0)
    assert lib.skv_scratch_bytes(ctypes.byref(p), 0) > _lib.SKV_NOALLOC_SCRATCH_BYTES
    # the boundary the header documents for this width: 4096 tokens fit, 8192 do not
    p.N = 4096
    assert 0 < lib.skv_scratch_bytes(ctypes.byref(p), 0) <= _lib.SKV_NOALLOC_SCRATCH_BYTES
    p.N = 8192
    assert lib.skv_scratch_bytes(ctypes.byref(p), 0) > _lib.SKV_NOALLOC_SCRATCH_BYTES
    p.N = 65536
    rc = lib.skv_feature_forward_noalloc(ctypes.byref(p), None, 5120, None, None, 0, None, 32, None, None)
    assert rc == -8
    assert b"SKV_NOALLOC_SCRATCH_BYTES" in lib.skv_error_string(rc)
