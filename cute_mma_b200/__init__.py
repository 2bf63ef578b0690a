"""B200-native GEMM and OFT fused block-diagonal GEMM: host-side mirror of the reference operators.

The compute path is the CUDA library built from cute_mma_b200/csrc (C ABI in include/cute_mma_b200.h).
This package only loads that library and forwards device pointers to it; there is no CPU fallback.
"""
from .ops import (  # noqa: F401
    Error,
    device_status,
    gemm,
    gemm_nt,
    gemm_tn,
    library_path,
    load_library,
    oft_tn,
    oft_tn_host,
    shard_range,
    tile_coord,
    kernel_info,
)
