"""streamk_b200: B200-native Stream-K GEMM library (fp32 / fp16 / W4A16).

The directory is named after the reference project; import it as `streamk_b200`
(the repository root holds a small loader module of that name).
"""
from .ops import *  # noqa: F401,F403
from .ops import __all__  # noqa: F401
from .gather import GatheredResult, column_block, peer_order, streamk_fp16_nt_gather  # noqa: F401
from . import build as build_recipe  # noqa: F401
