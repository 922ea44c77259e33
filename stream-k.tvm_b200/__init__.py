"""streamk_b200: B200-native Stream-K GEMM library (fp32 / fp16 / W4A16).

The directory is named after the reference project; import it as `streamk_b200`
(the repository root holds a small loader module of that name).
"""
from .ops import *  # noqa: F401,F403
from .ops import __all__  # noqa: F401
from .gather import (GatheredResult, ScatteredResult, column_block, peer_order,  # noqa: F401
                     streamk_fp16_nt_gather, streamk_fp16_nt_reduce_scatter)
from . import build as build_recipe  # noqa: F401
