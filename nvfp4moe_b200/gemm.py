"""Public NVFP4 GEMM plans and packing helpers.

Drop-in for ``lightmoe/gemm.py`` of the reference: ``quantize``,
``quantize_grouped``, ``DenseGemm`` and ``GroupedGemm`` keep their names,
argument order, return values and error messages.
"""

from __future__ import annotations

import torch

from ._quantization import _DEN
from .kernels.dense.runtime import DenseNvfp4Gemm
from .kernels.grouped.runtime import GroupedNvfp4Gemm
from .kernels.quantize.runtime import nvfp4_quantize_batched, nvfp4_quantize_rowwise

DenseGemm = DenseNvfp4Gemm
GroupedGemm = GroupedNvfp4Gemm


def _tensor_scale(x: torch.Tensor, scale: torch.Tensor | None) -> torch.Tensor:
    if scale is None:
        return (x.abs().amax().float() / _DEN).clamp_min(1e-30).reshape(1)
    return scale.detach().to(device=x.device, dtype=torch.float32).reshape(1)


def _check_matrix(x: torch.Tensor, name: str) -> None:
    if not x.is_cuda or x.ndim != 2 or not x.is_contiguous():
        raise ValueError(f"{name} must be a contiguous CUDA matrix")
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"{name} must use BF16 or FP32")
    if x.shape[1] % 64:
        raise ValueError(f"{name} K must be aligned to 64")


def _quantize_matrix(x: torch.Tensor, scale: torch.Tensor):
    rows, features = x.shape
    q = torch.empty(rows, features // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(-(-rows // 128), features // 64, 32, 4, 4,
                     dtype=torch.float8_e4m3fn, device=x.device)
    pair = torch.cat((scale, scale.reciprocal()))
    nvfp4_quantize_batched(x.unsqueeze(0), pair, q, sf)
    return q.view(torch.float4_e2m1fn_x2), sf


def quantize(x: torch.Tensor, scale: torch.Tensor | None = None):
    """Pack one BF16 or FP32 matrix into the NVFP4 layout: (q, sf, scale)."""
    _check_matrix(x, "x")
    scale = _tensor_scale(x, scale)
    q, sf = _quantize_matrix(x, scale)
    return q, sf, scale


def quantize_grouped(a, b, m_indptr, a_scale=None, b_scale=None):
    """Pack expert-major activations and weights for grouped GEMM.

    Returns ``(qa, qb, sfa, sfb, alpha)`` with ``alpha = a_scale * b_scale``.
    """
    _check_matrix(a, "a")
    if not b.is_cuda or b.ndim != 3 or not b.is_contiguous():
        raise ValueError("b must be contiguous CUDA expert weights [E, N, K]")
    if b.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("b must use BF16 or FP32")
    if b.device != a.device or b.shape[2] != a.shape[1]:
        raise ValueError("a and b must share device and K")
    experts, n, k = b.shape
    if m_indptr.dtype != torch.int32 or tuple(m_indptr.shape) != (experts + 1,):
        raise ValueError("m_indptr must be contiguous int32 with E + 1 offsets")
    if not m_indptr.is_cuda or not m_indptr.is_contiguous() or m_indptr.device != a.device:
        raise ValueError("m_indptr must be contiguous and share the input device")

    a_scale = _tensor_scale(a, a_scale)
    b_scale = _tensor_scale(b, b_scale)
    pair_a = torch.cat((a_scale, a_scale.reciprocal()))
    pair_b = torch.cat((b_scale, b_scale.reciprocal()))
    qa = torch.empty(a.shape[0], k // 2, dtype=torch.uint8, device=a.device)
    sfa = torch.zeros(1, -(-a.shape[0] // 128) + experts, k // 64, 32, 4, 4,
                      dtype=torch.float8_e4m3fn, device=a.device)
    nvfp4_quantize_rowwise(a, m_indptr, pair_a, qa, sfa)
    qb = torch.empty(experts, n, k // 2, dtype=torch.uint8, device=a.device)
    sfb = torch.empty(experts, -(-n // 128), k // 64, 32, 4, 4,
                      dtype=torch.float8_e4m3fn, device=a.device)
    nvfp4_quantize_batched(b, pair_b, qb, sfb)
    return (
        qa.view(torch.float4_e2m1fn_x2),
        qb.view(torch.float4_e2m1fn_x2),
        sfa,
        sfb,
        (a_scale * b_scale).reshape(1),
    )


__all__ = ["DenseGemm", "GroupedGemm", "quantize", "quantize_grouped"]
