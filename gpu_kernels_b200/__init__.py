"""B200-native NVFP4 path: quantise/pack, block-scaled GEMM, N-sharded multi-GPU GEMM.

Everything here drives hand-written sm_100a kernels through a C ABI
(include/nvfp4_capi.h). There is no CPU or eager fallback.
"""
from .nvfp4 import dequantize, dequantize_mx, pack_scales, quantize, quantize_mx, unpack_scales  # noqa: F401
from . import gemm, nvfp4  # noqa: F401
from .gemm import Nvfp4Gemm, gemm_host  # noqa: F401
from .sharded import GatheredOutput, ShardedNvfp4Gemm, gather_columns, shard_b, slab_rows  # noqa: F401
from .moe import Nvfp4MoE, route  # noqa: F401
from .peer import PeerGroup, SharedBuffer  # noqa: F401
