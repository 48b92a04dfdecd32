"""Public NVFP4 GEMM plans and packing helpers.

Drop-in for ``lightmoe/gemm.py`` of the reference: ``quantize``, ``quantize_grouped``,
``DenseGemm`` and ``GroupedGemm`` keep their names, argument order, return values and error
messages (``tests/test_gemm_api.py`` of the reference pins them).  Packing is one launch per
operand: the activations through the row quantizer with the varlen scale-factor layout, all
expert weights through one batched launch instead of one per expert.
"""

from __future__ import annotations

import torch

from ._quantization import _DEN
from .kernels.dense.runtime import DenseNvfp4Gemm
from .kernels.grouped.runtime import GroupedNvfp4Gemm
from .kernels.quantize.runtime import nvfp4_quantize_batched, nvfp4_quantize_rowwise

DenseGemm = DenseNvfp4Gemm
GroupedGemm = GroupedNvfp4Gemm

_SF = torch.float8_e4m3fn
_FP4 = torch.float4_e2m1fn_x2


def _tensor_scale(x: torch.Tensor, scale: torch.Tensor | None) -> torch.Tensor:
    """The per-tensor scale as a (1,) FP32 device tensor: given, or amax / 2688 (floor 1e-30)."""
    if scale is not None:
        return scale.detach().to(device=x.device, dtype=torch.float32).reshape(1)
    return (x.abs().amax().float() / _DEN).clamp_min(1e-30).reshape(1)


def _pair(scale: torch.Tensor) -> torch.Tensor:
    return torch.cat((scale, scale.reciprocal()))


def _check_matrix(x: torch.Tensor, name: str) -> None:
    for broken, message in (
        (not x.is_cuda or x.ndim != 2 or not x.is_contiguous(), f"{name} must be a contiguous CUDA matrix"),
        (x.dtype not in (torch.bfloat16, torch.float32), f"{name} must use BF16 or FP32"),
        (x.ndim == 2 and x.shape[1] % 64, f"{name} K must be aligned to 64"),
    ):
        if broken:
            raise ValueError(message)


def _pack_stack(stack: torch.Tensor, scale: torch.Tensor):
    """(groups, rows, K) -> packed codes and per-group blocked scale factors, one launch."""
    groups, rows, features = stack.shape
    q = torch.empty(groups, rows, features // 2, dtype=torch.uint8, device=stack.device)
    sf = torch.empty(groups, -(-rows // 128), features // 64, 32, 4, 4, dtype=_SF, device=stack.device)
    nvfp4_quantize_batched(stack, _pair(scale), q, sf)
    return q.view(_FP4), sf


def quantize(x: torch.Tensor, scale: torch.Tensor | None = None):
    """Pack one BF16 or FP32 matrix into the NVFP4 layout: (q, sf, scale)."""
    _check_matrix(x, "x")
    scale = _tensor_scale(x, scale)
    q, sf = _pack_stack(x.unsqueeze(0), scale)
    return q[0], sf[0], scale


def quantize_grouped(a, b, m_indptr, a_scale=None, b_scale=None):
    """Pack expert-major activations and weights for grouped GEMM.

    Returns ``(qa, qb, sfa, sfb, alpha)`` with ``alpha = a_scale * b_scale``.
    """
    _check_matrix(a, "a")
    for broken, message in (
        (not b.is_cuda or b.ndim != 3 or not b.is_contiguous(),
         "b must be contiguous CUDA expert weights [E, N, K]"),
        (b.dtype not in (torch.bfloat16, torch.float32), "b must use BF16 or FP32"),
        (b.device != a.device or (b.ndim == 3 and b.shape[2] != a.shape[1]), "a and b must share device and K"),
    ):
        if broken:
            raise ValueError(message)
    experts, _, k = b.shape
    if m_indptr.dtype != torch.int32 or tuple(m_indptr.shape) != (experts + 1,):
        raise ValueError("m_indptr must be contiguous int32 with E + 1 offsets")
    if not m_indptr.is_cuda or not m_indptr.is_contiguous() or m_indptr.device != a.device:
        raise ValueError("m_indptr must be contiguous and share the input device")

    a_scale, b_scale = _tensor_scale(a, a_scale), _tensor_scale(b, b_scale)
    rows = a.shape[0]
    qa = torch.empty(rows, k // 2, dtype=torch.uint8, device=a.device)
    # every expert starts a new 128-row atom row; atoms no row reaches stay zero
    sfa = torch.zeros(1, -(-rows // 128) + experts, k // 64, 32, 4, 4, dtype=_SF, device=a.device)
    nvfp4_quantize_rowwise(a, m_indptr, _pair(a_scale), qa, sfa)
    qb, sfb = _pack_stack(b, b_scale)
    return qa.view(_FP4), qb, sfa, sfb, (a_scale * b_scale).reshape(1)


__all__ = ["DenseGemm", "GroupedGemm", "quantize", "quantize_grouped"]
