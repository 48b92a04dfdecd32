"""Host side of the row-wise NVFP4 quantizer.

Mirrors ``lightmoe/kernels/quantize/runtime.py:107-156`` of the reference:
same function name, positional order and argument meaning.  The launch goes
through the C-ABI entry ``lm_quantize_rowwise``.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ... import _lib
from ...tracing import traced


def _prep(pts) -> Tensor:
    """Device-resident FP32 ``[pts, 1 / pts]`` without a host sync.

    Same contract as ``lightmoe/kernels/quantize/runtime.py:82-91``.
    """
    if torch.is_tensor(pts):
        if pts.numel() == 2:
            return pts
        p32 = pts.detach().to(device="cuda", dtype=torch.float32).reshape(1)
    else:
        if not pts > 0:
            raise ValueError("per_tensor_scale must be positive")
        p32 = torch.tensor([float(pts)], dtype=torch.float32, device="cuda")
    return torch.cat([p32, 1.0 / p32])


def _check_padded_offsets(padded_offsets, cu: Tensor, experts: int) -> None:
    if padded_offsets is None:
        return
    if (
        padded_offsets.dtype != torch.int32
        or padded_offsets.numel() != experts
        or not padded_offsets.is_cuda
        or not padded_offsets.is_contiguous()
        or padded_offsets.device != cu.device
    ):
        raise ValueError("padded_offsets must be contiguous CUDA int32 with one value per expert")


def _dtype_code(t: Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise ValueError("quantizer input must use BF16 or FP32")


@traced("lightmoe.quantize")
def nvfp4_quantize_rowwise(
    z: Tensor,
    cu: Tensor,
    pts,
    q_out: Tensor,
    sf_out: Tensor,
    gather_idx: Tensor | None = None,
    rounding: str = "rn",
    seed: int = 0,
    sf_layout: str = "blocked",
    padded_offsets: Tensor | None = None,
    te_math: bool = False,
) -> None:
    """Quantize expert-ordered rows, optionally gathering source rows from ``z``.

    ``padded_offsets`` is accepted for signature parity; this implementation
    finds the expert of a scale-factor atom row from ``cu`` alone, so the
    result does not depend on it.
    """
    if rounding != "rn":
        raise NotImplementedError("stochastic rounding belongs to the training path")
    if sf_layout not in ("blocked", "linear"):
        raise ValueError("sf_layout must be 'blocked' or 'linear'")
    if not z.is_cuda or z.ndim != 2 or z.stride(-1) != 1 or z.stride(0) != z.shape[1]:
        raise ValueError("z must be a contiguous CUDA matrix")
    features = z.shape[1]
    if features % 64:
        raise ValueError("feature count must be aligned to 64")
    experts = cu.numel() - 1
    _check_padded_offsets(padded_offsets, cu, experts)
    if cu.dtype != torch.int32 or not cu.is_cuda or not cu.is_contiguous():
        raise ValueError("cu must be contiguous CUDA int32")
    rows = int(gather_idx.numel()) if gather_idx is not None else z.shape[0]
    if gather_idx is not None and (gather_idx.dtype != torch.int32 or not gather_idx.is_contiguous()):
        raise ValueError("gather indices must be contiguous int32")
    pair = _prep(pts)
    mode = _lib.SF_VARLEN if sf_layout == "blocked" else _lib.SF_LINEAR
    _lib.check(
        _lib.lib().lm_quantize_rowwise(
            z.data_ptr(), _dtype_code(z), rows, features, cu.data_ptr(), experts, 0,
            pair.data_ptr(), _lib.ptr(gather_idx), q_out.data_ptr(), sf_out.data_ptr(),
            mode, int(bool(te_math)), _lib.stream_handle(),
        )
    )


@traced("lightmoe.quantize_weights")
def nvfp4_quantize_batched(w: Tensor, pts, q_out: Tensor, sf_out: Tensor) -> None:
    """Quantize an (E, N, K) weight stack in one launch.

    Replaces the per-expert loop of ``lightmoe/_quantization.py:82-99`` and
    ``lightmoe/gemm.py:109-117``; ``sf_out`` is ``(E, ceil(N/128), K/64, 32, 4, 4)``.
    """
    if not w.is_cuda or w.ndim != 3 or not w.is_contiguous():
        raise ValueError("weights must be contiguous CUDA [E, N, K]")
    experts, n, k = w.shape
    if k % 64:
        raise ValueError("K must be aligned to 64")
    pair = _prep(pts)
    _lib.check(
        _lib.lib().lm_quantize_rowwise(
            w.data_ptr(), _dtype_code(w), experts * n, k, None, experts, n, pair.data_ptr(),
            None, q_out.data_ptr(), sf_out.data_ptr(), _lib.SF_BATCHED, 0, _lib.stream_handle(),
        )
    )


__all__ = ["nvfp4_quantize_rowwise", "nvfp4_quantize_batched"]
