"""Host side of the decode quantizer.

Mirrors ``nvfp4_quantize_decode`` of the reference
(``lightmoe/kernels/quantize/decode.py:1108-1165``): every token row is
quantized once and written to each of its destination slots.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ... import _lib


def nvfp4_quantize_decode(
    x: Tensor,
    topk_ids: Tensor,
    slots: Tensor,
    m_indptr: Tensor,
    padded_offsets: Tensor,
    scale_pair: Tensor,
    q_out: Tensor,
    sf_out: Tensor,
    sf_tile_rows: int = 128,
) -> None:
    if sf_tile_rows != 128:
        raise NotImplementedError("decode scale factors use 128-row atoms in this build")
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or not x.is_cuda:
        raise ValueError("x must be contiguous CUDA BF16")
    tokens, features = x.shape
    top_k = topk_ids.shape[1]
    _lib.check(
        _lib.lib().lm_quantize_decode(
            x.data_ptr(), tokens, features, top_k, slots.data_ptr(), topk_ids.data_ptr(),
            m_indptr.data_ptr(), m_indptr.numel() - 1, scale_pair.data_ptr(), q_out.data_ptr(),
            sf_out.data_ptr(), _lib.stream_handle(),
        )
    )


def nvfp4_dispatch_quantize_decode(
    x: Tensor,
    topk_ids: Tensor,
    topk_weights: Tensor,
    parts: Tensor,
    gather: Tensor,
    m_indptr: Tensor,
    probs: Tensor,
    slots: Tensor,
    padded_offsets: Tensor,
    scale_pair: Tensor,
    q_out: Tensor,
    sf_out: Tensor,
    plan_tile_rows: int = 128,
) -> None:
    """Dispatch, decode plan and quantization of a decode batch in one launch.

    Same call as ``nvfp4_dispatch_quantize_decode`` of the reference
    (``lightmoe/kernels/quantize/decode.py:1168-1257``); here the packed rows
    and scale factors land directly in expert-major order, so the GEMM needs no
    token gather.  At most 1024 assignments.
    """
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or not x.is_cuda:
        raise ValueError("x must be contiguous CUDA BF16")
    tokens, features = x.shape
    top_k = topk_ids.shape[1]
    if tokens * top_k > 1024:
        raise ValueError("fused decode preparation handles at most 1024 assignments")
    experts = m_indptr.numel() - 1
    _lib.check(
        _lib.lib().lm_dispatch_quantize_decode(
            x.data_ptr(), topk_ids.data_ptr(), topk_weights.data_ptr(), tokens, top_k, experts,
            features, gather.data_ptr(), m_indptr.data_ptr(), probs.data_ptr(), slots.data_ptr(),
            padded_offsets.data_ptr(), parts.data_ptr(), parts.numel(), plan_tile_rows,
            scale_pair.data_ptr(), q_out.data_ptr(), sf_out.data_ptr(), _lib.stream_handle(),
        )
    )


__all__ = ["nvfp4_dispatch_quantize_decode", "nvfp4_quantize_decode"]
