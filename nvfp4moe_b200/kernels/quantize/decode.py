"""Host side of the decode quantizer.

Mirrors ``nvfp4_quantize_decode`` of the reference
(``lightmoe/kernels/quantize/decode.py:1108-1165``): every token row is
quantized once and written to each of its destination slots.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ... import _lib
from ...tracing import traced


@traced("lightmoe.quantize")
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


@traced("lightmoe.decode_prepare")
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


@traced("lightmoe.decode_prepare")
def _one_token_prepare(x, topk_ids, topk_weights, gather, slots, table, probs, padded_offsets, scale,
                       q_out, sf_out, direct: bool, label: str) -> None:
    tokens, features = x.shape
    topk = topk_ids.shape[1]
    experts = padded_offsets.numel()
    rows = tokens * topk
    table_shape = (topk,) if direct else (experts + 1,)
    expected = (
        tokens == 1
        and 0 < experts <= 256
        and 0 < topk <= min(experts, 32)
        and x.dtype == torch.bfloat16
        and features % 64 == 0
        and topk_ids.dtype == torch.int32
        and tuple(topk_ids.shape) == (1, topk)
        and topk_weights.dtype == torch.float32
        and tuple(topk_weights.shape) == (1, topk)
        and gather.dtype == torch.int32
        and gather.numel() == rows
        and slots.dtype == torch.int32
        and slots.numel() == rows
        and table.dtype == torch.int32
        and tuple(table.shape) == table_shape
        and probs.dtype == torch.float32
        and probs.numel() == rows
        and padded_offsets.dtype == torch.int32
        and scale.dtype == torch.float32
        and tuple(scale.shape) == (2,)
        and q_out.dtype in (torch.uint8, torch.float4_e2m1fn_x2)
        and q_out.numel() == rows * features // 2
        and sf_out.dtype == torch.float8_e4m3fn
    )
    if not expected:
        raise ValueError(f"{label} tensors do not match the configured shape")
    tensors = (x, topk_ids, topk_weights, gather, slots, table, probs, padded_offsets, scale, q_out, sf_out)
    if any(not t.is_cuda or not t.is_contiguous() or t.device != x.device for t in tensors):
        raise ValueError(f"{label} tensors must be contiguous on one CUDA device")
    # scale factors: atom row e for expert-major rows (row 0 with direct routes)
    need = ((1 if direct else experts) * (features // 64)) * 512
    if sf_out.numel() < need:
        raise ValueError(f"{label} tensors do not match the configured shape")
    with torch.cuda.device(x.device):
        _lib.check(
            _lib.lib().lm_decode_prepare(
                x.data_ptr(), topk_ids.data_ptr(), topk_weights.data_ptr(), topk, experts, features,
                int(direct), gather.data_ptr(), slots.data_ptr(), table.data_ptr(), probs.data_ptr(),
                padded_offsets.data_ptr(), scale.data_ptr(), q_out.data_ptr(), sf_out.data_ptr(),
                _lib.stream_handle(),
            )
        )


def nvfp4_decode_prepare(
    x: Tensor,
    topk_ids: Tensor,
    topk_weights: Tensor,
    gather: Tensor,
    slots: Tensor,
    cu: Tensor,
    probs: Tensor,
    padded_offsets: Tensor,
    scale: Tensor,
    q_out: Tensor,
    sf_out: Tensor,
    *,
    use_pdl: bool = True,
) -> None:
    """Build batch-size-one expert assignments and quantize in one launch.

    Same call as ``nvfp4_decode_prepare`` of the reference
    (``lightmoe/kernels/quantize/decode.py:946-1024``): one token, its ``top_k`` routes sorted
    expert-major (``gather``, ``slots``, ``cu`` = m_indptr, ``probs``, ``padded_offsets``), the
    row quantized with the multiply chain and written to each of its expert-major rows with
    varlen scale-factor atoms.  ``use_pdl`` is accepted for the signature; the launch is a
    plain one (nothing it could overlap precedes it in a decode step).
    """
    if x.ndim != 2 or topk_ids.ndim != 2:
        raise ValueError("decode input and expert ids must be matrices")
    if x.shape[0] != 1 or cu.numel() - 1 <= 0 or cu.numel() - 1 > 256 or not (
            0 < topk_ids.shape[1] <= min(cu.numel() - 1, 32)):
        raise ValueError("fused decode requires one token, 1-256 experts, and top-k at most 32")
    if padded_offsets.numel() != cu.numel() - 1:
        raise ValueError("fused decode tensors do not match the configured shape")
    _one_token_prepare(x, topk_ids, topk_weights, gather, slots, cu, probs, padded_offsets, scale, q_out,
                       sf_out, False, "fused decode")


def nvfp4_direct_decode_prepare(
    x: Tensor,
    topk_ids: Tensor,
    topk_weights: Tensor,
    gather: Tensor,
    slots: Tensor,
    route_ids: Tensor,
    probs: Tensor,
    padded_offsets: Tensor,
    scale: Tensor,
    q_out: Tensor,
    sf_out: Tensor,
    *,
    use_pdl: bool = True,
) -> None:
    """Quantize one token and emit direct route metadata
    (``lightmoe/kernels/quantize/decode.py:1027-1105``): ``slots[r] = r``, ``route_ids[r]`` = the
    expert of route r, ``probs[r]`` its weight; the row is quantized once into row 0 of ``q_out``
    (scale factors in atom row 0), which a ``GroupedNvfp4Gemm(direct_routes=top_k,
    broadcast_a=True)`` reads for every route.  ``padded_offsets`` only tells the expert count.
    """
    if x.ndim != 2 or topk_ids.ndim != 2:
        raise ValueError("direct decode tensors do not match the configured shape")
    _one_token_prepare(x, topk_ids, topk_weights, gather, slots, route_ids, probs, padded_offsets, scale,
                       q_out, sf_out, True, "direct decode")


__all__ = ["nvfp4_decode_prepare", "nvfp4_direct_decode_prepare", "nvfp4_dispatch_quantize_decode",
           "nvfp4_quantize_decode"]
