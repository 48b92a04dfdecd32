"""Grouped NVFP4 GEMM."""

from .runtime import GroupedNvfp4Gemm, grouped_nvfp4_gemm

__all__ = ["GroupedNvfp4Gemm", "grouped_nvfp4_gemm"]
