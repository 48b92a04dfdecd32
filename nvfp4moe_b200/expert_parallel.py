"""Expert-parallel execution of the NVFP4 MoE layer over one NVLink domain.

The reference has no communication code ("expert-parallel communication ...
remain the host framework's responsibility", README.md:227-228 of the
reference); this module is the host framework side for one 8xB200 box.

Rank r of G owns the contiguous experts [r*E/G, (r+1)*E/G) and brings its own
batch of tokens.  One step:

1. stable dispatch of the local (token, route) pairs by *global* expert id --
   expert-major order is also destination-rank-major order;
2. all-to-all of the per-expert row counts (a [G, E/G] int32 matrix);
3. all-to-all-v of the gathered BF16 rows to the ranks that own their experts;
4. on the owner: a second stable dispatch keyed by local expert puts the
   received rows (ordered by source rank) into expert-major order; the gather
   is fused into the quantizer; fc1 and fc2 run as on a single GPU;
5. all-to-all-v of the BF16 fc2 rows back to their source ranks;
6. deterministic weighted combine on the source rank, in route order.

Because every exchanged row is computed by exactly one expert and the combine
order is fixed, the result does not depend on G beyond the single-GPU
tolerance and is bit-identical from run to run.  Collectives are NCCL over
NVLink/NVSwitch when the process group is NCCL; the same code runs on gloo for
host-side tests.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def owner_splits(m_indptr: torch.Tensor, world: int) -> torch.Tensor:
    """Rows this rank sends to each owner rank, from the global-expert prefix."""
    experts = m_indptr.numel() - 1
    local = experts // world
    bounds = m_indptr[::local]
    return bounds[1:] - bounds[:-1]


def received_expert_ids(recv_counts: torch.Tensor) -> torch.Tensor:
    """Local expert id of every received row; rows arrive ordered by (source, expert)."""
    world, local = recv_counts.shape
    ids = torch.arange(local, dtype=torch.int32, device=recv_counts.device).repeat(world)
    return torch.repeat_interleave(ids, recv_counts.reshape(-1).long())


class ExpertParallelExchange:
    """The two all-to-all-v exchanges of one step and their bookkeeping."""

    def __init__(self, experts: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if experts % self.world:
            raise ValueError("the expert count must be divisible by the number of ranks")
        self.experts = experts
        self.local_experts = experts // self.world

    def exchange_counts(self, m_indptr: torch.Tensor) -> torch.Tensor:
        """[G, E/G] rows per (source rank, local expert) that this rank will receive."""
        counts = (m_indptr[1:] - m_indptr[:-1]).reshape(self.world, self.local_experts).contiguous()
        if self.world == 1:
            return counts
        received = torch.empty_like(counts)
        dist.all_to_all_single(received, counts, group=self.group)
        return received

    def forward_rows(self, rows: torch.Tensor, send_splits: list[int], recv_splits: list[int]):
        if self.world == 1:
            return rows
        out = torch.empty(sum(recv_splits), rows.shape[1], dtype=rows.dtype, device=rows.device)
        dist.all_to_all_single(out, rows, recv_splits, send_splits, group=self.group)
        return out

    def return_rows(self, rows: torch.Tensor, send_splits: list[int], recv_splits: list[int]):
        """Inverse of :meth:`forward_rows` (the split lists swap roles)."""
        if self.world == 1:
            return rows
        out = torch.empty(sum(send_splits), rows.shape[1], dtype=rows.dtype, device=rows.device)
        dist.all_to_all_single(out, rows, send_splits, recv_splits, group=self.group)
        return out


class ExpertParallelMoE:
    """``InferenceMoE`` sharded expert-parallel across the ranks of ``group``.

    ``max_tokens`` bounds the tokens per rank; ``max_recv_rows`` bounds the rows
    a rank may receive in one step (default: ``world * max_tokens * top_k``, the
    worst case of every pair in the box landing on one rank, capped at the
    dispatch limit).
    """

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top_k: int,
                 max_tokens: int, *, group=None, max_recv_rows: int | None = None,
                 device: torch.device | str = "cuda", **plan_kwargs):
        from .inference import InferenceMoE
        from .kernels.routing.dispatch import MAX_ASSIGNMENTS, MoEDispatch

        self.exchange = ExpertParallelExchange(num_experts, group)
        world = self.exchange.world
        self.hidden_size = hidden_size
        self.experts = num_experts
        self.topk = top_k
        self.max_tokens = max_tokens
        self.device = torch.device(device)
        rows = max_tokens * top_k
        if max_recv_rows is None:
            max_recv_rows = min(world * rows, MAX_ASSIGNMENTS)
        self.max_recv_rows = max_recv_rows
        # source side: sort local pairs by global expert
        self.source = MoEDispatch(max_tokens, num_experts, top_k, device=self.device)
        # owner side: a plan over the local experts whose "tokens" are received rows
        self.local = InferenceMoE(hidden_size, intermediate_size, self.exchange.local_experts, 1,
                                  max_recv_rows, device=self.device, **plan_kwargs)
        self._out = torch.empty(max_tokens, hidden_size, dtype=torch.bfloat16, device=self.device)
        self._ones = torch.ones(max_recv_rows, 1, dtype=torch.float32, device=self.device)
        self.last_recv_rows = 0

    # weights and scales of the local expert shard: same calls as InferenceMoE
    def load_weights(self, *args):
        self.local.load_weights(*args)
        return self

    def load_packed_weights(self, *args):
        self.local.load_packed_weights(*args)
        return self

    def set_activation_scales(self, input_scale, hidden_scale):
        self.local.set_activation_scales(input_scale, hidden_scale)
        return self

    @property
    def output(self) -> torch.Tensor:
        return self._out

    @torch.no_grad()
    def run(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
            *, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [T, H] BF16, topk_ids [T, k] int32 global expert ids, topk_weights [T, k] FP32."""
        from .kernels.quantize.runtime import nvfp4_quantize_rowwise
        from .kernels.routing.combine import moe_finalize
        from .kernels.routing.dispatch import moe_dispatch

        ex = self.exchange
        tokens = x.shape[0]
        rows = tokens * self.topk
        src = self.source
        if tokens != src.num_tokens:
            raise ValueError("the token count must match the configured per-rank batch")
        gather, m_indptr, probs, slots = src(topk_ids, topk_weights)

        recv_counts = ex.exchange_counts(m_indptr)
        send_splits = owner_splits(m_indptr, ex.world)
        # one host read per step sizes the exchange (the split lists of all_to_all_single)
        host = torch.cat((send_splits, recv_counts.sum(1))).tolist()
        send_list, recv_list = host[: ex.world], host[ex.world :]
        received = sum(recv_list)
        self.last_recv_rows = received
        if received > self.max_recv_rows:
            raise RuntimeError(f"received {received} rows, workspace holds {self.max_recv_rows}")

        send_rows = x.index_select(0, gather.long())
        recv_rows = ex.forward_rows(send_rows, send_list, recv_list)

        plan = self.local
        if received > 0:
            ids = received_expert_ids(recv_counts).reshape(received, 1)
            moe_dispatch(ids, self._ones[:received], plan.experts, plan._gather[:received],
                         plan._m_indptr, plan._probs[:received], plan._slots[:received],
                         plan._parts, plan._padded_offsets)
            # one prepared plan over the whole receive arena: the GEMMs take the real row
            # bounds from m_indptr on the device, so the row count may change every step
            execution = plan._full_execution(plan.max_tokens, decode=False)
            nvfp4_quantize_rowwise(recv_rows, plan._m_indptr, plan._x_scale,
                                   execution.qx[:received],
                                   execution.sfx, gather_idx=plan._gather[:received],
                                   padded_offsets=plan._padded_offsets, te_math=True)
            execution.fc1.launch()
            execution.fc2.launch()
            # expert-major rows back into arrival order
            back = execution.routed_out[:received].index_select(0, plan._slots[:received].long())
        else:
            back = recv_rows
        returned = ex.return_rows(back, send_list, recv_list)

        output = self._out[:tokens] if out is None else out
        moe_finalize(returned, slots, output, self.topk, weights=probs)
        return output

    __call__ = run


def reference_step(x, topk_ids, topk_weights, compute_rows: Callable, exchange: ExpertParallelExchange):
    """The same exchange pattern on plain torch ops, for host-side (gloo) tests.

    ``compute_rows(rows, local_expert_ids)`` stands in for the expert GEMMs.
    """
    tokens, k = topk_ids.shape
    flat = topk_ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=exchange.experts)
    m_indptr = torch.zeros(exchange.experts + 1, dtype=torch.int32)
    m_indptr[1:] = counts.cumsum(0)
    recv_counts = exchange.exchange_counts(m_indptr)
    send_list = owner_splits(m_indptr, exchange.world).tolist()
    recv_list = recv_counts.sum(1).tolist()
    recv_rows = exchange.forward_rows(x[(order // k)].contiguous(), send_list, recv_list)
    ids = received_expert_ids(recv_counts)
    back = compute_rows(recv_rows, ids)
    returned = exchange.return_rows(back.contiguous(), send_list, recv_list)
    out = torch.zeros(tokens, x.shape[1], dtype=torch.float32)
    weights = topk_weights.reshape(-1)[order]
    out.index_add_(0, order // k, returned.float() * weights.unsqueeze(1))
    return out


__all__ = ["ExpertParallelExchange", "ExpertParallelMoE", "owner_splits", "received_expert_ids",
           "reference_step"]
