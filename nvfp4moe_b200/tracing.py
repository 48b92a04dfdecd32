"""NVTX ranges around the stages of a step.

The reference marks only its benchmark harness (one ``torch.cuda.nvtx`` range in
``benchmarks/moe.py:648-659``, behind a hidden flag).  Here every host wrapper that launches a
kernel of the path can open a range named after its stage (``lightmoe.dispatch``,
``lightmoe.quantize``, ``lightmoe.fc1`` ...), so that a timeline capture shows which launches
belong to which stage.  Off by default: a disabled range costs one global lookup per call, and
nothing is pushed while a CUDA graph is replayed (the wrappers do not run then).
"""

from __future__ import annotations

import functools

import torch

_enabled = False


def enable(on: bool = True) -> None:
    """Turn the ranges on or off for this process."""
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


def push(name: str) -> bool:
    """Open a range if tracing is on; returns whether ``pop`` has something to close."""
    if not _enabled:
        return False
    torch.cuda.nvtx.range_push(name)
    return True


def pop(opened: bool) -> None:
    if opened:
        torch.cuda.nvtx.range_pop()


def traced(name: str):
    """Decorator: the call runs inside a range called ``name`` while tracing is on."""

    def wrap(fn):
        @functools.wraps(fn)
        def inner(*args, **kwargs):
            if not _enabled:
                return fn(*args, **kwargs)
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()

        return inner

    return wrap


__all__ = ["enable", "enabled", "pop", "push", "traced"]
