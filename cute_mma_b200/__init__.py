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
    gemm_rowmajor,
    gemm_tn_acc2,
    kernel_info,
    lora_tn,
    oft_plan,
    oft_tn,
    oft_tn_a_rw,
    oft_tn_host,
    oft_tn_static,
    oft_tn_two_pass,
    rotate,
    shard_range,
    tile_coord,
    transform_weight,
)
