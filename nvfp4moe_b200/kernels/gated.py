"""Gated activation policies of the fused fc1 epilogue.

Same public surface as ``lightmoe/kernels/gated.py:40-126`` of the reference
(``GatedEpilogue``, defaults and validation messages); the device math lives in
``csrc/gemm.cu``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

_ACTIVATIONS = ("swiglu", "swiglu_oai", "geglu", "reglu")
FLT_MAX = 3.4028234663852886e38


def gated_output_n(accumulator_n: int) -> int:
    """Half-width output extent of an interleaved gate/up accumulator."""
    if accumulator_n <= 0 or accumulator_n % 2:
        raise ValueError("gated accumulator N must be a positive even value")
    return accumulator_n // 2


def validate_gated_tile_n(tile_n: int) -> int:
    if tile_n <= 0 or tile_n % 128:
        raise ValueError("gated NVFP4 tile_N must be a positive multiple of 128")
    return tile_n


def validate_gated_activation(activation: str) -> str:
    if activation not in _ACTIVATIONS:
        raise ValueError("activation must be one of: " + ", ".join(_ACTIVATIONS))
    return activation


def _finite_positive(value, message: str) -> float:
    value = float(value)
    if not math.isfinite(value) or value <= 0:
        raise ValueError(message)
    return value


@dataclass(frozen=True, slots=True)
class GatedEpilogue:
    """Forward gated activation fused into the GEMM epilogue."""

    activation: str = "swiglu"
    save_preact: bool = False
    clamp_limit: float | None = None
    sigmoid_alpha: float | None = None
    up_bias: float | None = None

    def __post_init__(self):
        set_ = object.__setattr__
        set_(self, "activation", validate_gated_activation(self.activation))
        oai = self.activation == "swiglu_oai"
        if oai and self.clamp_limit is None:
            set_(self, "clamp_limit", 7.0)
        if self.sigmoid_alpha is None:
            set_(self, "sigmoid_alpha", 1.702 if oai else 1.0)
        if self.up_bias is None:
            set_(self, "up_bias", 1.0 if oai else 0.0)
        if self.clamp_limit is not None:
            limit = _finite_positive(self.clamp_limit, "clamp_limit must be finite and positive")
            if self.activation not in ("swiglu", "swiglu_oai"):
                raise ValueError("clamp_limit is supported only for SwiGLU activations")
            set_(self, "clamp_limit", limit)
        alpha = _finite_positive(self.sigmoid_alpha, "sigmoid_alpha must be finite and positive")
        bias = float(self.up_bias)
        if not math.isfinite(bias):
            raise ValueError("up_bias must be finite")
        if not oai and (alpha != 1.0 or bias != 0.0):
            raise ValueError("sigmoid_alpha and up_bias require swiglu_oai")
        set_(self, "sigmoid_alpha", alpha)
        set_(self, "up_bias", bias)


@dataclass(frozen=True, slots=True)
class GatedBackwardEpilogue:
    """Training-only policy; kept so callers can name it, rejected by the GEMM."""

    activation: str = "swiglu"
    clamp_limit: float | None = None
    sigmoid_alpha: float | None = None
    up_bias: float | None = None

    def __post_init__(self):
        forward = GatedEpilogue(self.activation, clamp_limit=self.clamp_limit,
                                sigmoid_alpha=self.sigmoid_alpha, up_bias=self.up_bias)
        object.__setattr__(self, "clamp_limit", forward.clamp_limit)
        object.__setattr__(self, "sigmoid_alpha", forward.sigmoid_alpha)
        object.__setattr__(self, "up_bias", forward.up_bias)


def resolve_gemm_epilogue(epilogue, activation, dactivation):
    """Map an epilogue policy object to (activation, dactivation) names."""
    from .unary import UnaryBackwardEpilogue, UnaryEpilogue

    if epilogue is not None and (activation is not None or dactivation is not None):
        raise ValueError("epilogue cannot be combined with activation or dactivation")
    if isinstance(epilogue, (GatedEpilogue, UnaryEpilogue)):
        return epilogue.activation, None
    if isinstance(epilogue, (GatedBackwardEpilogue, UnaryBackwardEpilogue)):
        return None, epilogue.activation
    if epilogue is not None:
        raise TypeError("unsupported grouped GEMM epilogue")
    return activation, dactivation


__all__ = [
    "GatedBackwardEpilogue",
    "GatedEpilogue",
    "gated_output_n",
    "resolve_gemm_epilogue",
    "validate_gated_activation",
    "validate_gated_tile_n",
]
