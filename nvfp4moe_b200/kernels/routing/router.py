"""Router step in front of the dispatch: softmax over the experts, top-k, renormalise.

The reference leaves this step to the host framework (its tests and benchmarks build
``topk_ids`` / ``topk_weights`` with torch: ``tests/test_training_gpu.py:23-27``) and keeps
it out of its timings (``BENCHMARKS.md:15``).  ``route_topk`` is that recipe in one launch;
its outputs are exactly what ``moe_dispatch`` and ``InferenceMoE.run`` take.
"""

from __future__ import annotations

import torch

from ... import _lib


def route_topk(logits: torch.Tensor, top_k: int, *, topk_ids: torch.Tensor | None = None,
               topk_weights: torch.Tensor | None = None):
    """``softmax(logits, -1)`` -> ``topk`` -> weights divided by their sum.

    ``logits`` (tokens, experts) BF16 or FP32 on CUDA, at most 256 experts.  Returns
    ``(topk_ids int32 (tokens, top_k), topk_weights float32 (tokens, top_k))``, the larger
    probability first and the lower expert id on a tie; pass preallocated outputs to keep a
    serving loop allocation-free.
    """
    if not logits.is_cuda or logits.ndim != 2 or not logits.is_contiguous():
        raise ValueError("logits must be a contiguous CUDA matrix (tokens, experts)")
    if logits.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("logits must be BF16 or FP32")
    tokens, experts = logits.shape
    if experts > 256:
        raise ValueError("route_topk supports at most 256 experts")
    if not 0 < top_k <= min(32, experts):
        raise ValueError("top_k must be in 1..min(32, experts)")
    if topk_ids is None:
        topk_ids = torch.empty(tokens, top_k, dtype=torch.int32, device=logits.device)
    if topk_weights is None:
        topk_weights = torch.empty(tokens, top_k, dtype=torch.float32, device=logits.device)
    for name, tensor, dtype in (("topk_ids", topk_ids, torch.int32), ("topk_weights", topk_weights, torch.float32)):
        if (tensor.dtype != dtype or tuple(tensor.shape) != (tokens, top_k) or not tensor.is_contiguous()
                or tensor.device != logits.device):
            raise ValueError(f"{name} must be contiguous {dtype} with shape ({tokens}, {top_k}) on {logits.device}")
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().lm_route_topk(logits.data_ptr(), 0 if logits.dtype == torch.bfloat16 else 1,
                                            tokens, experts, top_k, topk_ids.data_ptr(),
                                            topk_weights.data_ptr(), _lib.stream_handle()))
    return topk_ids, topk_weights


__all__ = ["route_topk"]
