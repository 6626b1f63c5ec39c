"""flaggems_b200: the FP8 quantized-inference hot path of FlagGems on B200 (sm_100a).

The public names, signatures and registration behaviour follow the reference's
``flag_gems`` package (src/flag_gems/__init__.py) for the functions on that path; the
top-level ``flag_gems`` module of this repository re-exports everything here so that
``import flag_gems`` keeps working.  All device work goes through the C-ABI library
``flaggems_b200/lib/libflaggems_b200.so`` (hand-written CUDA for sm_100a).
"""
from . import _cabi  # noqa: F401
from .fused import *  # noqa: F401,F403
from .ops import *  # noqa: F401,F403
from .registration import (  # noqa: F401
    all_registered_keys,
    all_registered_ops,
    aten_lib,
    enable,
    only_enable,
    use_gems,
)
from .patches import apply_gems_patches_to_vllm, patch_empty_vllm  # noqa: F401

__version__ = "0.1.0"
device = "cuda"
vendor_name = "nvidia"
