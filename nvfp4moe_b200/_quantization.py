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
    """An amax kept on the device and the quantization scale pair derived from it.

    Mirrors ``TensorScale`` of the reference (``lightmoe/_quantization.py:14-67``): ``update``
    and ``set_amax`` never read the device, ``pair`` is ``[pts, 1 / pts]`` with
    ``pts = amax / 2688`` floored at the smallest normal FP32 (an all-zero tensor must not
    produce an infinite reciprocal).  ``pts`` and ``inv_pts`` are views of ``pair``: a later
    update shows through views taken earlier.
    """

    def __init__(self, device="cuda", te_rht=False):
        if te_rht:
            raise NotImplementedError("the RHT scale convention belongs to the training path")
        self.te_rht = False
        self._ready = False
        self._amax = torch.zeros(1, dtype=torch.float32, device=device)
        self._pair = torch.empty(2, dtype=torch.float32, device=device)

    @torch.no_grad()
    def _publish(self, amax: torch.Tensor) -> None:
        self._amax.copy_(amax.reshape(1))
        torch.div(self._amax, _DEN, out=self._pair[:1])
        self._pair[:1].clamp_(min=torch.finfo(torch.float32).tiny)
        torch.reciprocal(self._pair[:1], out=self._pair[1:])
        self._ready = True

    @torch.no_grad()
    def update(self, t: torch.Tensor):
        """Update amax without a host synchronization."""
        low, high = torch.aminmax(t.detach())
        self._publish(torch.maximum(low.neg(), high).float())

    @torch.no_grad()
    def set_amax(self, amax: torch.Tensor):
        self._publish(amax.to(device=self._amax.device, dtype=torch.float32))

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
