"""glowq_b200: B200 (sm_100a) implementation of GlowQ's corrected W4A16 linear behind GlowQ's own Python surface."""
from .cuda_w4a16 import CudaW4A16Linear, convert_to_cuda_w4a16, load_w4a16_extension
from .correction import (AddSVDCorrection, MiniGroupCache, clear_group_cache, patch_svd_correction_wrappers,
                         patch_svd_correction_wrappers_cumulative)
from .artifacts import load_packed, save_packed

__all__ = ["load_w4a16_extension", "CudaW4A16Linear", "convert_to_cuda_w4a16", "AddSVDCorrection", "MiniGroupCache",
           "patch_svd_correction_wrappers", "patch_svd_correction_wrappers_cumulative", "clear_group_cache",
           "save_packed", "load_packed"]
