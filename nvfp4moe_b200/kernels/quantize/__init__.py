"""NVFP4 quantization kernels (inference subset of ``lightmoe.kernels.quantize``)."""

from .decode import (nvfp4_decode_prepare, nvfp4_direct_decode_prepare, nvfp4_dispatch_quantize_decode,
                     nvfp4_quantize_decode)
from .runtime import nvfp4_quantize_batched, nvfp4_quantize_rowwise

__all__ = ["nvfp4_decode_prepare", "nvfp4_direct_decode_prepare", "nvfp4_dispatch_quantize_decode",
           "nvfp4_quantize_batched", "nvfp4_quantize_decode", "nvfp4_quantize_rowwise"]
