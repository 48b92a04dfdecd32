"""Host side of the stable expert-major dispatch.

Mirrors ``lightmoe/kernels/routing/dispatch.py:368-440`` of the reference
(``moe_dispatch`` and the ``MoEDispatch`` buffer holder).
"""

from __future__ import annotations

import torch
from torch import Tensor

from ... import _lib
from ...tracing import traced

CHUNK = 1024
B_MAX = 128  # scratch rows the reference always allocates; larger inputs get more
MAX_ASSIGNMENTS = 1 << 22


def scratch_elems(rows: int, experts: int) -> int:
    """int32 scratch elements ``moe_dispatch`` needs for ``rows`` assignments."""
    return max(B_MAX, -(-rows // CHUNK)) * experts


@traced("lightmoe.dispatch")
def moe_dispatch(
    topi: Tensor,
    topv: Tensor,
    E: int,
    gi: Tensor,
    cu: Tensor,
    ps: Tensor,
    slots: Tensor,
    part: Tensor,
    off_pad: Tensor,
    *,
    use_pdl: bool = True,
    gather_experts: bool = False,
    plan_tile_rows: int = 128,
) -> None:
    """Build a stable expert-major permutation from preselected routes."""
    if gather_experts:
        raise NotImplementedError("gather_experts belongs to the training path")
    assert topi.dtype == torch.int32 and topi.is_contiguous()
    assert topv.dtype == torch.float32 and topv.is_contiguous()
    assert topi.dim() == 2 and topv.shape == topi.shape
    tokens, k = topi.shape
    rows = tokens * k
    assert rows <= MAX_ASSIGNMENTS, f"M={rows} exceeds the {MAX_ASSIGNMENTS} dispatch bound"
    assert plan_tile_rows > 0 and 128 % plan_tile_rows == 0
    assert gi.numel() == rows and slots.numel() == rows and ps.numel() == rows
    assert cu.numel() == E + 1 and part.numel() >= -(-rows // CHUNK) * E
    assert off_pad.numel() == E and off_pad.dtype == torch.int32
    _lib.check(
        _lib.lib().lm_dispatch(
            topi.data_ptr(), topv.data_ptr(), tokens, k, E, gi.data_ptr(), cu.data_ptr(),
            ps.data_ptr(), slots.data_ptr(), off_pad.data_ptr(), part.data_ptr(), part.numel(),
            plan_tile_rows, _lib.stream_handle(),
        )
    )


class MoEDispatch:
    """Preallocated expert-major dispatch buffers."""

    def __init__(self, num_tokens: int, num_experts: int, top_k: int, device="cuda"):
        rows = num_tokens * top_k
        self.num_tokens = num_tokens
        self.num_experts = num_experts
        self.top_k = top_k
        self.gi = torch.empty(rows, dtype=torch.int32, device=device)
        self.cu = torch.empty(num_experts + 1, dtype=torch.int32, device=device)
        self.ps = torch.empty(rows, dtype=torch.float32, device=device)
        self.slots = torch.empty(rows, dtype=torch.int32, device=device)
        self.part = torch.empty(scratch_elems(rows, num_experts), dtype=torch.int32, device=device)
        self.off_pad = torch.empty(num_experts, dtype=torch.int32, device=device)

    def __call__(self, topi: Tensor, topv: Tensor):
        assert topi.shape == (self.num_tokens, self.top_k)
        probs = topv.float() if topv.dtype != torch.float32 else topv
        moe_dispatch(topi, probs, self.num_experts, self.gi, self.cu, self.ps, self.slots,
                     self.part, self.off_pad)
        return self.gi, self.cu, self.ps, self.slots

    def differentiable_probs(self, topv: Tensor) -> Tensor:
        """Expert-major probabilities that keep router gradients."""
        assert topv.shape == (self.num_tokens, self.top_k)
        return torch.zeros_like(self.ps).index_put((self.slots.long(),), topv.reshape(-1).float())


__all__ = ["B_MAX", "CHUNK", "MoEDispatch", "moe_dispatch", "scratch_elems"]
