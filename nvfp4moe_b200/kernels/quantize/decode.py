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


__all__ = ["nvfp4_quantize_decode"]
