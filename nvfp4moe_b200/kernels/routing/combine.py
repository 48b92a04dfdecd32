"""Host side of the deterministic top-k combine.

Mirrors ``moe_finalize`` of the reference
(``lightmoe/kernels/routing/combine.py:231-281``).
"""

from __future__ import annotations

import torch
from torch import Tensor

from ... import _lib
from ...tracing import traced


@traced("lightmoe.combine")
def moe_finalize(
    yw: Tensor,
    slots: Tensor,
    out: Tensor,
    topk: int,
    tile_t: int = 8,
    n_frag: int = 1,
    weights: Tensor | None = None,
    use_pdl: bool = False,
    direct: bool = False,
    num_threads: int = 256,
    broadcast_slots: bool = False,
    valid: Tensor | None = None,
) -> None:
    """out[t] = sum over this token's non-negative slots of yw rows (times weights).

    ``tile_t``, ``n_frag``, ``num_threads`` and ``broadcast_slots`` are scheduling knobs of the
    reference's kernel; the result does not depend on them and this kernel has no use for
    them.  ``use_pdl`` launches the kernel as a programmatic dependent of the previous one.
    ``valid`` (not in the reference): an int32 device flag; when it holds 0 the rows were not
    computed this step and ``out`` is written as zeros.
    """
    assert yw.stride(-1) == 1 and out.stride(-1) == 1
    if yw.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise ValueError("moe_finalize supports BF16 rows")
    if num_threads not in (128, 256, 512, 768):
        raise ValueError("num_threads must be 128, 256, 512, or 768")
    tokens, hidden = out.shape
    if direct:
        assert tokens == 1 and yw.shape[0] == topk
        assert weights is not None and n_frag == 2
        slots = torch.arange(topk, dtype=torch.int32, device=yw.device)
    assert slots.dtype == torch.int32 and slots.numel() == tokens * topk
    if weights is not None:
        assert weights.dtype == torch.float32 and weights.numel() == yw.shape[0]
        assert weights.is_contiguous()
    assert hidden % 8 == 0, "d must be a multiple of 8"
    assert yw.stride(0) % 8 == 0 and out.stride(0) % 8 == 0, (
        "row strides must keep 128-bit vector alignment"
    )
    _lib.check(
        _lib.lib().lm_finalize(
            yw.data_ptr(), slots.data_ptr(), _lib.ptr(weights), out.data_ptr(), tokens, topk,
            hidden, yw.stride(0), out.stride(0), _lib.ptr(valid), int(bool(use_pdl)), _lib.stream_handle(),
        )
    )


__all__ = ["moe_finalize"]
