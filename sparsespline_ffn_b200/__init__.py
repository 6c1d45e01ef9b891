"""B200 (sm_100a) implementation of the RL-Spline-KV ``flash_spline_feature`` operator.

The package is a drop-in for one operator of the reference project
(``sparsespline_ffn.kernels.flash_spline_feature_autograd``): the same
``torch.autograd.Function`` classes and functional wrappers, backed by a C-ABI CUDA library
(``libsplinekv_b200.so``, built from ``csrc/``).  There is no CPU or eager fallback: the
operators raise when the library or a B200 is missing.
"""
from .kernels.flash_spline_feature_autograd import (  # noqa: F401
    FlashSplineDelta,
    FlashSplineFeature,
    flash_spline_delta,
    flash_spline_feature,
)

from .rl_spline_kv import RLSplineKV, RLSplineKVConfig  # noqa: F401,E402

__all__ = ["FlashSplineFeature", "flash_spline_feature", "FlashSplineDelta", "flash_spline_delta",
           "RLSplineKV", "RLSplineKVConfig"]
