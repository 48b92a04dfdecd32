"""Unary activation policy (ReLU squared) of the fused fc1 epilogue.

Same public surface as ``lightmoe/kernels/unary.py:21-40`` of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

_ACTIVATIONS = ("relu2",)


def validate_unary_activation(activation: str) -> str:
    if activation not in _ACTIVATIONS:
        raise ValueError("unary activation must be relu2")
    return activation


@dataclass(frozen=True, slots=True)
class UnaryEpilogue:
    """Forward unary activation fused into the GEMM epilogue."""

    activation: str = "relu2"
    save_preact: bool = False

    def __post_init__(self):
        object.__setattr__(self, "activation", validate_unary_activation(self.activation))


@dataclass(frozen=True, slots=True)
class UnaryBackwardEpilogue:
    """Training-only policy; kept so callers can name it, rejected by the GEMM."""

    activation: str = "relu2"

    def __post_init__(self):
        object.__setattr__(self, "activation", validate_unary_activation(self.activation))


__all__ = ["UnaryBackwardEpilogue", "UnaryEpilogue", "validate_unary_activation"]
