"""NVFP4 scale state and expert-weight packing.

Mirrors ``lightmoe/_quantization.py`` of the reference: ``TensorScale`` keeps an
amax on the device and exposes ``[pts, 1/pts]`` without a host sync;
``quantize_expert_stack`` packs a list (or stack) of expert matrices -- here in
one batched launch instead of one launch per expert.
"""

from __future__ import annotations

import torch

from .kernels.quantize.runtime import nvfp4_quantize_batched

F4_MAX = 6.0
E4M3_MAX = 448.0
_DEN = E4M3_MAX * F4_MAX  # 2688


class TensorScale:
    """Track amax and expose quantization / dequantization scale pairs."""

    def __init__(self, device="cuda", te_rht=False):
        if te_rht:
            raise NotImplementedError("the RHT scale convention belongs to the training path")
        self._amax = torch.zeros(1, dtype=torch.float32, device=device)
        self._pair = torch.empty(2, dtype=torch.float32, device=device)
        self._ready = False
        self.te_rht = False

    @torch.no_grad()
    def update(self, t: torch.Tensor):
        """Update amax without a host synchronization."""
        mn, mx = torch.aminmax(t.detach())
        self._amax.copy_(torch.maximum(mn.neg_(), mx).reshape(1).float())
        self._refresh()

    @torch.no_grad()
    def set_amax(self, amax: torch.Tensor):
        self._amax.copy_(amax.reshape(1))
        self._refresh()

    @torch.no_grad()
    def _refresh(self):
        p = (self._amax / _DEN).clamp_(min=torch.finfo(torch.float32).tiny)
        self._pair[0:1].copy_(p)
        self._pair[1:2].copy_(1.0 / p)
        self._ready = True

    @property
    def pair(self) -> torch.Tensor:
        """``[pts, 1/pts]``."""
        assert self._ready, "TensorScale used before calibration: call update(t) once"
        return self._pair

    @property
    def pts(self) -> torch.Tensor:
        return self.pair[0:1]

    @property
    def inv_pts(self) -> torch.Tensor:
        return self.pair[1:2]


@torch.no_grad()
def quantize_expert_stack(matrices, scale):
    """Pack equally shaped expert matrices: returns (q [E,N,K/2] fp4x2, sf [E,N/128,K/64,32,4,4])."""
    if torch.is_tensor(matrices):
        stack = matrices.contiguous()
    else:
        stack = torch.stack([m.contiguous() for m in matrices])
    experts, rows, features = stack.shape
    scale = scale.detach().to(device=stack.device, dtype=torch.float32).reshape(1)
    pair = torch.cat((scale, scale.reciprocal()))
    q = torch.empty(experts, rows, features // 2, dtype=torch.uint8, device=stack.device)
    sf = torch.empty(experts, -(-rows // 128), features // 64, 32, 4, 4,
                     dtype=torch.float8_e4m3fn, device=stack.device)
    if rows % 128:
        sf.view(torch.uint8).zero_()
    nvfp4_quantize_batched(stack, pair, q, sf)
    return q.view(torch.float4_e2m1fn_x2), sf


__all__ = ["TensorScale", "quantize_expert_stack"]
