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

from .tracing import traced


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

    def verify_splits(self, send_splits: list[int], recv_splits: list[int]) -> None:
        """Host-side check before an all-to-all-v: what this rank is about to send to rank o
        must be what o expects from it.  A mismatch (ranks built with different expert counts,
        a count table that was overwritten) would otherwise surface as a hang or as rows in the
        wrong place.  Every rank learns of a mismatch anywhere and raises ``RuntimeError``, so
        no rank enters the exchange alone.  Costs two small collectives: a debugging aid, off
        by default."""
        if self.world == 1:
            return
        backend = dist.get_backend(self.group)
        device = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
        mine = torch.tensor(send_splits, dtype=torch.int64, device=device)
        theirs = torch.empty_like(mine)
        dist.all_to_all_single(theirs, mine, group=self.group)  # theirs[o] = rows o will send here
        expected = torch.tensor(recv_splits, dtype=torch.int64, device=device)
        flag = (theirs != expected).any().to(torch.int32).reshape(1)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        if int(flag.item()):
            raise RuntimeError(
                f"rank {self.rank}: all-to-all split sizes disagree between ranks "
                f"(peers send {theirs.tolist()}, this rank expects {list(recv_splits)})")

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


def _align(value: int, to: int = 256) -> int:
    return -(-value // to) * to


class ExpertParallelMoE:
    """``InferenceMoE`` sharded expert-parallel across the ranks of ``group``.

    ``max_tokens`` bounds the tokens per rank; ``max_recv_rows`` bounds the rows
    a rank may receive in one step (default: ``world * max_tokens * top_k``, the
    worst case of every pair in the box landing on one rank, capped at the
    dispatch limit).

    ``transport``:

    * ``"peer"`` (default on CUDA with more than one rank): no row ever passes through a
      collective.  The ranks gather each other's per-expert counts (1 KB), every rank derives
      the whole route plan on its device, the quantizer stores packed rows and scale factors
      straight into the owners' GEMM operand buffers and the fc2 GEMM stores its BF16 rows
      straight into the source ranks' buffers, both through peer pointers over NVLink.  The
      counts and the two fences between the phases travel through signal pads in the same
      peer memory (``signals="peer"``, one single-CTA kernel each, bounded waits) or through
      NCCL (``signals="nccl"``).  The host never reads a count: a step is a fixed sequence of
      launches.
    * ``"collective"``: BF16 rows travel through ``all_to_all_single`` both ways; one host
      read per step sizes the exchange.  Works on any backend.

    ``rank`` / ``world`` build a *virtual* rank that makes no ``torch.distributed`` call:
    several of them in one process, joined by :func:`connect_virtual_ranks`, run the
    peer transport on one GPU (tests, debugging).
    """

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top_k: int,
                 max_tokens: int, *, group=None, max_recv_rows: int | None = None,
                 device: torch.device | str = "cuda", transport: str | None = None,
                 rank: int | None = None, world: int | None = None, signals: str = "peer",
                 signal_timeout_ms: int = 0, **plan_kwargs):
        from .inference import InferenceMoE
        from .kernels.routing.dispatch import MAX_ASSIGNMENTS, MoEDispatch

        self.virtual = rank is not None
        if self.virtual:
            if world is None or not 0 <= rank < world or num_experts % world:
                raise ValueError("a virtual rank needs 0 <= rank < world and experts divisible by world")
            self.exchange = None
            self.world, self.rank = world, rank
        else:
            self.exchange = ExpertParallelExchange(num_experts, group)
            self.world, self.rank = self.exchange.world, self.exchange.rank
        self.group = group
        self.hidden_size = hidden_size
        self.experts = num_experts
        self.local_experts = num_experts // self.world
        self.topk = top_k
        self.max_tokens = max_tokens
        self.device = torch.device(device)
        if transport is None:
            transport = "peer" if (self.virtual or (self.world > 1 and self.device.type == "cuda")) else "collective"
        if transport not in ("peer", "collective"):
            raise ValueError("transport must be 'peer' or 'collective'")
        if transport == "peer" and self.world > 8:
            raise ValueError("the peer transport serves one NVLink domain of at most 8 ranks")
        self.transport = transport
        if signals not in ("peer", "nccl"):
            raise ValueError("signals must be 'peer' or 'nccl'")
        self.signals = signals
        self.signal_timeout_ms = int(signal_timeout_ms)
        rows = max_tokens * top_k
        if max_recv_rows is None:
            max_recv_rows = min(self.world * rows, MAX_ASSIGNMENTS)
        self.max_recv_rows = max_recv_rows
        # source side: sort local pairs by global expert
        self.source = MoEDispatch(max_tokens, num_experts, top_k, device=self.device)
        # owner side: a plan over the local experts whose "tokens" are received rows
        self.local = InferenceMoE(hidden_size, intermediate_size, self.local_experts, 1,
                                  max_recv_rows, device=self.device, **plan_kwargs)
        self._out = torch.empty(max_tokens, hidden_size, dtype=torch.bfloat16, device=self.device)
        self._ones = torch.ones(max_recv_rows, 1, dtype=torch.float32, device=self.device)
        self.last_recv_rows = 0
        self.verify_splits = False  # collective transport: check the split lists across ranks first
        self._peer = None
        if transport == "peer":
            self._build_peer_buffers()

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

    # ------------------------------------------------------------ peer transport
    def _build_peer_buffers(self):
        """One arena per rank, at the same offsets on every rank: the packed rows and row-major
        scale factors of the rows this rank computes (written by the sources) and the BF16 rows
        this rank combines (written by the owners)."""
        hidden, m, rows = self.hidden_size, self.max_recv_rows, self.max_tokens * self.topk
        sf_rows = -(-m // 128) + self.local_experts
        off_q = 0
        off_sf = _align(m * (hidden // 2))
        off_ret = off_sf + _align(m * (hidden // 16))
        off_cnt = off_ret + _align(rows * hidden * 2)
        off_sig = off_cnt + _align(self.world * self.experts * 4)
        nbytes = off_sig + 256
        if self.virtual or self.world == 1:
            arena = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            bases = [arena.data_ptr()] * self.world  # rewritten by connect_virtual_ranks
            handle = None
        else:
            import os

            # plain peer mappings are all this path needs: no NVLink multicast binding
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm

            group = self.group if self.group is not None else dist.group.WORLD
            arena = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
            handle = symm.rendezvous(arena, group.group_name)
            bases = [int(ptr) for ptr in handle.buffer_ptrs]
            arena.zero_()
            # no rank may signal into a pad that its owner has yet to clear
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        dev = self.device
        peer = {
            "arena": arena, "handle": handle, "offsets": (off_q, off_sf, off_ret, off_cnt, off_sig),
            "qx": arena[off_q : off_q + m * (hidden // 2)].view(m, hidden // 2).view(torch.float4_e2m1fn_x2),
            # scale factors arrive row-major; the local swizzle kernel turns them into atoms
            "sf_rows": arena[off_sf : off_sf + m * (hidden // 16)].view(m, hidden // 16),
            "sfx": torch.zeros(1, sf_rows, hidden // 64, 32, 4, 4, dtype=torch.uint8, device=dev)
            .view(torch.float8_e4m3fn),
            "ret": arena[off_ret : off_ret + rows * hidden * 2].view(torch.bfloat16).view(rows, hidden),
            "counts": torch.zeros(self.experts, dtype=torch.int32, device=dev),
            "counts_all": arena[off_cnt : off_cnt + self.world * self.experts * 4].view(torch.int32)
            .view(self.world, self.experts),
            "dest_base": torch.zeros(self.experts, dtype=torch.int32, device=dev),
            "owner_start": torch.zeros(self.experts, dtype=torch.int32, device=dev),
            "row_ptrs": torch.zeros(m, dtype=torch.int64, device=dev),
            # per 32-row block of every row tile: the rank and row its result block returns to
            "out_blocks": torch.full(((m // 128 + self.local_experts) * 4, 2), -1, dtype=torch.int32, device=dev),
            "valid": torch.ones(1, dtype=torch.int32, device=dev),
            "token": torch.zeros(1, dtype=torch.int32, device=dev),
            "gemms": None,
        }
        self._peer = peer
        self._set_peer_bases(bases)

    def _set_peer_bases(self, bases):
        import ctypes

        off_q, off_sf, off_ret, off_cnt, off_sig = self._peer["offsets"]
        array = ctypes.c_uint64 * self.world
        self._peer["cnt_base"] = array(*[b + off_cnt for b in bases])
        self._peer["sig_base"] = array(*[b + off_sig for b in bases])
        self._peer["q_base"] = array(*[b + off_q for b in bases])
        self._peer["sf_base"] = array(*[b + off_sf for b in bases])
        self._peer["ret_base"] = array(*[b + off_ret for b in bases])

    def _peer_gemms(self):
        """fc1 reads the arena the sources fill; fc2 writes through the row-pointer table."""
        peer, plan = self._peer, self.local
        if peer["gemms"] is None:
            m = self.max_recv_rows
            _, qh, _, sfh = plan._views(m)
            with torch.cuda.device(self.device):
                fc1 = plan._new_gemm("fc1", m, torch.float4_e2m1fn_x2)
                fc2 = plan._new_gemm("fc2", m)
            fc1.prepare(peer["qx"], plan.qb1, qh, plan._m_indptr, peer["sfx"], plan.sfb1, plan._alpha1,
                        output_sf=sfh, output_scale=plan._h_scale)
            # result rows go back from inside the fc2 epilogue: whole 32-row blocks of one source as
            # bulk stores into that rank's return buffer, the rest row by row
            fc2.output_row_ptrs = peer["row_ptrs"]
            fc2.output_blocks = peer["out_blocks"]
            fc2.return_bases = peer["ret_base"]
            fc2.return_rows = self.max_tokens * self.topk
            fc2.prepare(qh, plan.qb2, plan._routed_out[:m], plan._m_indptr, sfh, plan.sfb2, plan._alpha2)
            peer["gemms"] = (fc1, fc2)
        return peer["gemms"]

    def _phase_dispatch(self, topk_ids, topk_weights):
        """Sort this rank's routes by global expert; returns the per-expert counts to gather."""
        _, m_indptr, _, _ = self.source(topk_ids, topk_weights)
        torch.sub(m_indptr[1:], m_indptr[:-1], out=self._peer["counts"])
        return self._peer["counts"]

    @traced("lightmoe.ep_plan_quantize_send")
    def _phase_send(self, x):
        """Route plan from the gathered counts, then quantize once and store to the owners."""
        from . import _lib

        peer, plan, src = self._peer, self.local, self.source
        plan._require_ready()
        lib = _lib.lib()
        stream = _lib.stream_handle()
        with torch.cuda.device(self.device):
            _lib.check(lib.lm_ep_plan(peer["counts_all"].data_ptr(), self.world, self.rank, self.experts,
                                      self.max_recv_rows, self.hidden_size * 2, peer["ret_base"],
                                      plan._m_indptr.data_ptr(), peer["dest_base"].data_ptr(),
                                      peer["owner_start"].data_ptr(), peer["row_ptrs"].data_ptr(),
                                      peer["out_blocks"].data_ptr(), peer["valid"].data_ptr(), stream))
            _lib.check(lib.lm_ep_quantize_send(x.data_ptr(), x.shape[0], self.hidden_size, self.topk,
                                               self.world, self.experts, src.slots.data_ptr(),
                                               self._ids.data_ptr(), src.cu.data_ptr(),
                                               peer["dest_base"].data_ptr(), peer["owner_start"].data_ptr(),
                                               peer["valid"].data_ptr(), plan._x_scale.data_ptr(),
                                               peer["q_base"], peer["sf_base"], stream))

    @traced("lightmoe.ep_compute_and_return")
    def _phase_compute(self, mark=None):
        from . import _lib

        fc1, fc2 = self._peer_gemms()
        peer, plan = self._peer, self.local
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lm_ep_sf_swizzle(peer["sf_rows"].data_ptr(), self.max_recv_rows,
                                                   self.hidden_size, plan._m_indptr.data_ptr(),
                                                   self.local_experts, peer["sfx"].data_ptr(),
                                                   _lib.stream_handle()))
        if mark is not None:
            mark("swizzle")
        fc1.launch()
        if mark is not None:
            mark("fc1")
        fc2.launch()
        if mark is not None:
            mark("fc2_and_return")

    def _phase_combine(self, out):
        from .kernels.routing.combine import moe_finalize

        tokens = self._ids.shape[0]
        output = self._out[:tokens] if out is None else out
        # a step the route plan skipped (a rank would have overflowed) combines to zeros
        moe_finalize(self._peer["ret"][: tokens * self.topk], self.source.slots, output, self.topk,
                     weights=self.source.ps, valid=self._peer["valid"])
        return output

    def _signal(self, m_indptr=None):
        """Every rank has finished the launches before this point; with ``m_indptr`` the ranks
        also leave their per-expert counts in each other's tables.  One small kernel per rank
        over the signal pads in peer memory (``signals="nccl"``: collectives instead)."""
        if self.virtual or self.world == 1:
            return
        peer = self._peer
        if self.signals == "nccl":
            if m_indptr is not None:
                torch.sub(m_indptr[1:], m_indptr[:-1], out=peer["counts"])
                dist.all_gather_into_tensor(peer["counts_all"].view(-1), peer["counts"], group=self.group)
            else:
                dist.all_reduce(peer["token"], group=self.group)
            return
        from . import _lib

        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lm_ep_signal(None if m_indptr is None else m_indptr.data_ptr(),
                                               self.experts, self.world, self.rank, peer["cnt_base"],
                                               peer["sig_base"], self.signal_timeout_ms,
                                               _lib.stream_handle()))

    def _check_inputs(self, x, topk_ids, topk_weights):
        tokens = x.shape[0]
        if tokens != self.source.num_tokens:
            raise ValueError("the token count must match the configured per-rank batch")
        if x.dtype != torch.bfloat16 or x.shape[1] != self.hidden_size or not x.is_contiguous():
            raise ValueError(f"x must be contiguous BF16 with shape (tokens, {self.hidden_size})")
        if topk_ids.dtype != torch.int32 or tuple(topk_ids.shape) != (tokens, self.topk):
            raise ValueError(f"topk_ids must be int32 with shape ({tokens}, {self.topk})")
        self._ids = topk_ids

    @torch.no_grad()
    def _run_peer(self, x, topk_ids, topk_weights, out):
        self._check_inputs(x, topk_ids, topk_weights)
        if self.world == 1:
            self._peer["counts_all"].copy_(self._phase_dispatch(topk_ids, topk_weights).view(1, -1))
        else:
            _, m_indptr, _, _ = self.source(topk_ids, topk_weights)
            self._signal(m_indptr)  # every rank's counts are in every rank's table
        self._phase_send(x)
        self._signal()  # all packed rows have landed on their owners
        self._phase_compute()
        self._signal()  # all result rows have landed on their sources
        return self._phase_combine(out)

    @torch.no_grad()
    def run_phases(self, x, topk_ids, topk_weights, *, out=None):
        """One peer-transport step with a CUDA event after every phase.  Returns
        ``({phase: milliseconds}, output)``; the time a rank spends waiting for the others inside
        a signal kernel counts towards the phase that the signal closes.  Synchronises the
        stream (a measuring aid, not part of the serving path)."""
        if self.transport != "peer" or self.virtual:
            raise RuntimeError("run_phases times the peer transport of a real rank")
        marks = [("start", torch.cuda.Event(enable_timing=True))]
        marks[0][1].record()

        def mark(name):
            event = torch.cuda.Event(enable_timing=True)
            event.record()
            marks.append((name, event))

        self._check_inputs(x, topk_ids, topk_weights)
        if self.world == 1:
            self._peer["counts_all"].copy_(self._phase_dispatch(topk_ids, topk_weights).view(1, -1))
            mark("dispatch")
        else:
            _, m_indptr, _, _ = self.source(topk_ids, topk_weights)
            mark("dispatch")
            self._signal(m_indptr)
            mark("exchange_counts")
        self._phase_send(x)
        mark("plan_quantize_send")
        self._signal()
        mark("fence_rows_landed")
        self._phase_compute(mark)
        self._signal()
        mark("fence_results_landed")
        output = self._phase_combine(out)
        mark("combine")
        torch.cuda.synchronize(self.device)
        times = {name: marks[i][1].elapsed_time(event) for i, (name, event) in enumerate(marks[1:])}
        return times, output

    def step_is_valid(self) -> bool:
        """False when the last step was skipped because a rank would have received more than
        ``max_recv_rows`` rows (reads one flag from the device: a synchronisation)."""
        return self._peer is None or bool(self._peer["valid"].item())

    @torch.no_grad()
    def run(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
            *, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [T, H] BF16, topk_ids [T, k] int32 global expert ids, topk_weights [T, k] FP32."""
        if self.transport == "peer":
            if self.virtual:
                raise RuntimeError("virtual ranks are stepped together by run_virtual_ranks")
            return self._run_peer(x, topk_ids, topk_weights, out)
        return self._run_collective(x, topk_ids, topk_weights, out)

    # ------------------------------------------------------ collective transport
    @torch.no_grad()
    def _run_collective(self, x, topk_ids, topk_weights, out):
        from .kernels.quantize.runtime import nvfp4_quantize_rowwise
        from .kernels.routing.combine import moe_finalize
        from .kernels.routing.dispatch import moe_dispatch

        ex = self.exchange
        tokens = x.shape[0]
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
        if self.verify_splits:
            ex.verify_splits(send_list, recv_list)
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


def connect_virtual_ranks(layers) -> None:
    """Join virtual ranks that live in one process (one GPU): each one's peer table points at
    the others' arenas."""
    layers = list(layers)
    world = layers[0].world
    if sorted(layer.rank for layer in layers) != list(range(world)) or any(not l.virtual for l in layers):
        raise ValueError("connect_virtual_ranks needs one virtual rank per rank of the world")
    ordered = sorted(layers, key=lambda layer: layer.rank)
    bases = [layer._peer["arena"].data_ptr() for layer in ordered]
    for layer in ordered:
        layer._set_peer_bases(bases)


@torch.no_grad()
def run_virtual_ranks(layers, batches, outs=None):
    """One expert-parallel step of all virtual ranks on the current stream, phase by phase;
    stream order stands in for the cross-rank fences.  ``batches[r] = (x, topk_ids, topk_weights)``."""
    ordered = sorted(layers, key=lambda layer: layer.rank)
    counts = []
    for layer, (x, ids, w) in zip(ordered, batches):
        layer._check_inputs(x, ids, w)
        counts.append(layer._phase_dispatch(ids, w))
    gathered = torch.stack(counts)
    for layer, (x, _, _) in zip(ordered, batches):
        layer._peer["counts_all"].copy_(gathered)
        layer._phase_send(x)
    for layer in ordered:
        layer._phase_compute()
    return [layer._phase_combine(None if outs is None else outs[layer.rank]) for layer in ordered]


def reference_step(x, topk_ids, topk_weights, compute_rows: Callable, exchange: ExpertParallelExchange,
                   *, verify: bool = False, tamper: Callable | None = None):
    """The same exchange pattern on plain torch ops, for host-side (gloo) tests.

    ``compute_rows(rows, local_expert_ids)`` stands in for the expert GEMMs.  ``verify`` runs
    :meth:`ExpertParallelExchange.verify_splits` before rows move; ``tamper(send, recv)`` lets a
    test corrupt the split lists of one rank first.
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
    if tamper is not None:
        send_list, recv_list = tamper(send_list, recv_list)
    if verify:
        exchange.verify_splits(send_list, recv_list)
    recv_rows = exchange.forward_rows(x[(order // k)].contiguous(), send_list, recv_list)
    ids = received_expert_ids(recv_counts)
    back = compute_rows(recv_rows, ids)
    returned = exchange.return_rows(back.contiguous(), send_list, recv_list)
    out = torch.zeros(tokens, x.shape[1], dtype=torch.float32)
    weights = topk_weights.reshape(-1)[order]
    out.index_add_(0, order // k, returned.float() * weights.unsqueeze(1))
    return out


__all__ = ["ExpertParallelExchange", "ExpertParallelMoE", "connect_virtual_ranks", "owner_splits",
           "received_expert_ids", "reference_step", "run_virtual_ranks"]
