"""Dense NVFP4 GEMM."""

from .runtime import DenseNvfp4Gemm

__all__ = ["DenseNvfp4Gemm"]
