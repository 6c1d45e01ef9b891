"""The bounded device-side waits: a wait that can never be satisfied runs out, the kernel returns
by itself with the time-out bit in the caller's status word, and the next call on the same device
works.  The failure is made on the host side of the kernel's own protocol (a test hook makes the
loader warp leave out one bulk copy, so a barrier never completes although nothing is in flight);
nothing faults, traps or hangs.  The reference's kernels spin on their barriers without a limit
(src/sparsespline_ffn/cuda_ext/spline_kv_bwd_v6.cu:159-172)."""
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

ops = pytest.importorskip("sparsespline_ffn_b200.ops")
_lib = pytest.importorskip("sparsespline_ffn_b200._lib")


def test_a_wait_that_runs_out_sets_the_status_word_and_the_device_stays_usable():
    lib = _lib.load()
    N, h, r, G = 256, 64, 32, 20
    z, C, _ = util.make_inputs(N, h, r, G, torch.bfloat16)
    assert ops.resolve_impl(z, C, -3.0, 3.0, G) == "tcgen05"
    ops.check_status(z.device)                                   # clean before the experiment
    assert lib.skv_debug_set(_lib.SKV_DEBUG_WAIT_CYCLES, 2_000_000) == 0      # about a millisecond
    assert lib.skv_debug_set(_lib.SKV_DEBUG_SKIP_FIRST_COPY, 1) == 0
    try:
        ops.feature_forward(z, C, -3.0, 3.0, G, impl="tcgen05")  # returns: the kernel drains by itself
        torch.cuda.synchronize()
    finally:
        lib.skv_debug_set(_lib.SKV_DEBUG_SKIP_FIRST_COPY, 0)
        lib.skv_debug_set(_lib.SKV_DEBUG_WAIT_CYCLES, 4_000_000_000)
    assert int(ops.status_word(z.device).item()) & 0x1, "the forward's time-out bit is not set"
    with pytest.raises(RuntimeError, match="bounded wait"):
        ops.check_status(z.device)
    ops.check_status(z.device)                                   # the word was cleared by the raise
    # the context is intact: a normal call gives the right answer
    f = ops.feature_forward(z, C, -3.0, 3.0, G, "relu_sq", 0.75, impl="tcgen05")
    a_ref, d_ref = util.oracle_forward(z, C, -3.0, 3.0, G, "relu_sq", 0.75)
    util.assert_parity("phi(z)", f[:, :h], a_ref, torch.bfloat16)
    util.assert_parity("lambda*delta", f[:, h:], d_ref, torch.bfloat16)
    ops.check_status(z.device)


def test_the_readout_gemm_drains_when_its_first_stage_never_arrives():
    lib = _lib.load()
    N, h, r, G, d_out = 512, 128, 32, 20, 256
    z, C, _ = util.make_inputs(N, h, r, G, torch.bfloat16)
    W = (torch.randn(d_out, h + r, device=z.device) * 0.04).to(torch.bfloat16)
    ops.check_status(z.device)
    assert lib.skv_debug_set(_lib.SKV_DEBUG_WAIT_CYCLES, 2_000_000) == 0
    assert lib.skv_debug_set(_lib.SKV_DEBUG_SKIP_FIRST_COPY, 2) == 0          # the feature kernels run normally
    try:
        ops.feature_readout_forward(z, C, W, -3.0, 3.0, G, "relu_sq", 1.0)
        torch.cuda.synchronize()
    finally:
        lib.skv_debug_set(_lib.SKV_DEBUG_SKIP_FIRST_COPY, 0)
        lib.skv_debug_set(_lib.SKV_DEBUG_WAIT_CYCLES, 4_000_000_000)
    assert int(ops.status_word(z.device).item()) == 0x10, "only the read-out GEMM's time-out bit should be set"
    with pytest.raises(RuntimeError, match="bounded wait"):
        ops.check_status(z.device)
    y = ops.feature_readout_forward(z, C, W, -3.0, 3.0, G, "relu_sq", 1.0)
    f = ops.feature_forward(z, C, -3.0, 3.0, G, "relu_sq", 1.0)
    ref = f.double() @ W.double().t()
    assert float((y.double() - ref).norm() / ref.norm()) < 4e-3
    ops.check_status(z.device)


def test_debug_set_rejects_unknown_settings():
    lib = _lib.load()
    assert lib.skv_debug_set(99, 1) < 0
    assert lib.skv_debug_set(_lib.SKV_DEBUG_WAIT_CYCLES, 5) < 0   # a limit too short to be useful
