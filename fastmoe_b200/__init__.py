"""fastmoe_b200: the MoE token dispatch/combine hot path of polkadot21/fastmoe,
rebuilt for NVIDIA B200 (sm_100a) as hand-written CUDA behind the reference's
Python API.

    from fastmoe_b200.kernels.ops import grouped_weighted_scatter_add
    from fastmoe_b200.models.tiny_model import MoEFeedForward, PipelinedMoEBlock
    from fastmoe_b200.consts import MoEImplementation

The CUDA kernels live in `libfastmoe_b200.so` (C ABI: include/fastmoe_b200.h),
which is loaded on first use.
"""

from . import consts  # noqa: F401
from .consts import MoEImplementation  # noqa: F401

__version__ = "0.1.0"
