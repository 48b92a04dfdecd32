"""The byte arena an inference plan runs in.

Same members and aliasing as ``InferenceWorkspace`` of the reference
(``lightmoe/inference.py:71-213``), which its tests pin (``_qx_u8`` shares its address with
``_routed_out``, ``_qh_u8`` with ``_out``): one ``uint8`` allocation in which the quantized
input and its scale factors alias the fc2 result rows, the quantized hidden rows alias the layer
output, and the int32 / float32 routing metadata follows.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .kernels.routing.dispatch import scratch_elems

_ALIGN = 256


def _round_up(value: int, to: int = _ALIGN) -> int:
    return -(-value // to) * to


class _Carver:
    """Hands out views of one byte tensor.  ``overlay`` places several members at the same
    offset (the region is as large as the largest of them); ``take`` appends a member."""

    def __init__(self):
        self.cursor = 0
        self._members: list[tuple[str, int, torch.dtype, tuple[int, ...]]] = []

    def overlay(self, *members):
        """members: (name, dtype, shape[, offset inside the region])."""
        base = self.cursor
        extent = 0
        for name, dtype, shape, *rest in members:
            inner = rest[0] if rest else 0
            self._members.append((name, base + inner, dtype, tuple(shape)))
            extent = max(extent, inner + math.prod(shape) * torch.empty((), dtype=dtype).element_size())
        self.cursor = base + _round_up(extent)

    def take(self, name, dtype, elements: int):
        self._members.append((name, self.cursor, dtype, (elements,)))
        self.cursor += elements * torch.empty((), dtype=dtype).element_size()

    def views(self, storage: torch.Tensor) -> dict[str, torch.Tensor]:
        out = {}
        for name, offset, dtype, shape in self._members:
            nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
            out[name] = storage[offset : offset + nbytes].view(dtype).view(shape)
        return out


@dataclass(slots=True)
class InferenceWorkspace:
    """Reusable buffers for plans that execute serially on one stream."""

    hidden_size: int
    intermediate_size: int
    experts: int
    topk: int
    max_tokens: int
    device: torch.device
    storage: torch.Tensor
    qx_u8: torch.Tensor
    qh_u8: torch.Tensor
    sfx: torch.Tensor
    sfh: torch.Tensor
    routed_out: torch.Tensor
    out: torch.Tensor
    gather: torch.Tensor
    m_indptr: torch.Tensor
    probs: torch.Tensor
    slots: torch.Tensor
    parts: torch.Tensor
    padded_offsets: torch.Tensor

    @classmethod
    def allocate(cls, hidden_size, intermediate_size, experts, topk, max_tokens, device):
        rows = max_tokens * topk
        atom_rows = -(-rows // 128) + experts  # every expert starts a new 128-row atom row
        qx_bytes = rows * hidden_size // 2
        qh_bytes = rows * intermediate_size // 2
        fp8, u8, bf16 = torch.float8_e4m3fn, torch.uint8, torch.bfloat16
        carve = _Carver()
        # fc1 reads qx + sfx and fc2 writes routed_out afterwards: one region
        carve.overlay(("qx_u8", u8, (rows, hidden_size // 2)),
                      ("sfx", fp8, (1, atom_rows, hidden_size // 64, 32, 4, 4), qx_bytes),
                      ("routed_out", bf16, (rows, hidden_size)))
        # fc2 reads qh + sfh and the combine writes out afterwards: one region
        carve.overlay(("qh_u8", u8, (rows, intermediate_size // 2)),
                      ("sfh", fp8, (1, atom_rows, intermediate_size // 64, 32, 4, 4), qh_bytes),
                      ("out", bf16, (max_tokens, hidden_size)))
        carve.take("gather", torch.int32, rows)
        carve.take("m_indptr", torch.int32, experts + 1)
        carve.take("probs", torch.float32, rows)
        carve.take("slots", torch.int32, rows)
        carve.take("parts", torch.int32, scratch_elems(rows, experts))
        carve.take("padded_offsets", torch.int32, experts)
        with torch.cuda.device(device):
            storage = torch.empty(carve.cursor, dtype=torch.uint8, device=device)
        return cls(hidden_size, intermediate_size, experts, topk, max_tokens, device, storage,
                   **carve.views(storage))

    @property
    def nbytes(self) -> int:
        return self.storage.numel()

    def matches(self, hidden_size, intermediate_size, experts, topk, max_tokens, device) -> bool:
        mine = (self.hidden_size, self.intermediate_size, self.experts, self.topk, self.max_tokens, self.device)
        return mine == (hidden_size, intermediate_size, experts, topk, max_tokens, device)


__all__ = ["InferenceWorkspace"]
