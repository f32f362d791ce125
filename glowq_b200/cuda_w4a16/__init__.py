"""Drop-in replacement of GlowQ's ``cuda_w4a16`` package (src/cuda_w4a16/__init__.py:1-8)."""
from .kernels import load_w4a16_extension
from .linear import CudaW4A16Linear, convert_to_cuda_w4a16

__all__ = ["load_w4a16_extension", "CudaW4A16Linear", "convert_to_cuda_w4a16"]
