"""Host-side behaviour of the RLSplineKV module that needs no GPU: configuration checks, parameter
names and shapes (those of the reference's RLSplineKVReference, so that its checkpoints load), and
the refusal to run without the CUDA kernels."""
import pytest
import torch

from sparsespline_ffn_b200.rl_spline_kv import RLSplineKV, RLSplineKVConfig


def test_config_validation_matches_the_reference_rules():
    RLSplineKVConfig(d=16)
    for bad in (dict(G=1), dict(grid_lo=1.0, grid_hi=1.0), dict(h_ratio=0.0), dict(h_ratio=5.0), dict(r=0),
                dict(spline_order=3), dict(activation="tanh"), dict(gating_mode="other"), dict(c_init_std=-1.0),
                dict(gating_mode="multiplicative", no_base=True)):
        with pytest.raises(ValueError):
            RLSplineKVConfig(d=16, **bad)


@pytest.mark.parametrize("mode,readout_in", [("additive", 32 + 8), ("no_base", 8), ("multiplicative", 32)])
def test_parameter_names_and_shapes(mode, readout_in):
    extra = dict(no_base=True) if mode == "no_base" else dict(gating_mode=mode) if mode == "multiplicative" else {}
    m = RLSplineKV(RLSplineKVConfig(d=16, h_ratio=2.0, r=8, G=20, **extra))
    shapes = {k: tuple(v.shape) for k, v in m.state_dict().items()}
    assert shapes["K.weight"] == (32, 16)
    assert shapes["C"] == (32, 22, 8)
    assert shapes["W_out.weight"] == (16, readout_in)
    assert ("W_d_proj.weight" in shapes) == (mode == "multiplicative")
    assert {"grid_lo_buf", "grid_hi_buf"} <= set(shapes)
    assert float(m.C.abs().max()) == 0.0                 # cold start: C = 0 unless a std is given
    assert m.num_params() == sum(p.numel() for p in m.parameters())


def test_linear_spline_modes_and_cpu_input():
    assert tuple(RLSplineKV(RLSplineKVConfig(d=16, r=8, spline_order=1)).C.shape) == (16, 21, 8)   # L = G + 1
    with pytest.raises(NotImplementedError):
        RLSplineKV(RLSplineKVConfig(d=16, spline_order=1, no_base=True))
    with pytest.raises(NotImplementedError):
        RLSplineKV(RLSplineKVConfig(d=16, spline_order=1, gating_mode="multiplicative"))
    m = RLSplineKV(RLSplineKVConfig(d=16, r=8))
    with pytest.raises(RuntimeError, match="CUDA-only"):
        m(torch.randn(4, 16))
    with pytest.raises(ValueError):
        m(torch.randn(4, 15))
