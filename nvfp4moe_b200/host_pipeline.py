"""Host-resident batches through a device layer: copy in, step, copy out, overlapped.

A serving loop that holds its activations in pinned host memory pays one
host-to-device copy of ``x`` / ``topk_ids`` / ``topk_weights`` and one device-to-host
copy of the output per step; on a PCIe-attached B200 both copies take longer than
the layer itself.  :class:`HostPipeline` keeps ``depth`` device buffer sets and three
streams (copy-in, compute, copy-out) so that the copy-in of batch ``i + 1`` and the
copy-out of batch ``i - 1`` run while batch ``i`` computes.  Every wait between the
streams is a device-side event wait: ``submit`` never blocks the host.

The layer is anything with ``run(x, topk_ids, topk_weights, out=...)`` on device
tensors: :class:`nvfp4moe_b200.InferenceMoE` or
:class:`nvfp4moe_b200.expert_parallel.ExpertParallelMoE`.
"""

from __future__ import annotations

import torch


class HostPipeline:
    def __init__(self, layer, tokens: int, hidden_size: int, top_k: int, *, depth: int = 2,
                 device=None):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        if not torch.cuda.is_available():
            raise RuntimeError("HostPipeline needs a CUDA device")
        self.layer = layer
        self.tokens = int(tokens)
        self.hidden_size = int(hidden_size)
        self.top_k = int(top_k)
        self.depth = int(depth)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with torch.cuda.device(self.device):
            self._copy_in = torch.cuda.Stream()
            self._compute = torch.cuda.Stream()
            self._copy_out = torch.cuda.Stream()
        dev = self.device
        self._x = [torch.empty(tokens, hidden_size, dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self._ids = [torch.empty(tokens, top_k, dtype=torch.int32, device=dev) for _ in range(depth)]
        self._w = [torch.empty(tokens, top_k, dtype=torch.float32, device=dev) for _ in range(depth)]
        self._out = [torch.empty(tokens, hidden_size, dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self._loaded = [torch.cuda.Event() for _ in range(depth)]    # inputs of the slot are on the device
        self._computed = [torch.cuda.Event() for _ in range(depth)]  # the slot's inputs may be overwritten
        self._stored = [torch.cuda.Event() for _ in range(depth)]    # the slot's output is on the host
        self._submitted = 0
        # the layer's workspace was filled on another stream: order it before the first step
        torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ checks
    def _check_host(self, name, tensor, shape, dtype):
        if tensor.device.type != "cpu" or not tensor.is_pinned():
            raise ValueError(f"{name} must be a pinned host tensor")
        if tuple(tensor.shape) != shape or tensor.dtype != dtype or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous {dtype} with shape {shape}")

    # ------------------------------------------------------------------- steps
    @torch.no_grad()
    def submit(self, x_host, ids_host, w_host, out_host) -> int:
        """Enqueue one batch; returns its ticket.  The host buffers belong to the pipeline
        until ``wait(ticket)`` returns."""
        t, h, k = self.tokens, self.hidden_size, self.top_k
        self._check_host("x", x_host, (t, h), torch.bfloat16)
        self._check_host("topk_ids", ids_host, (t, k), torch.int32)
        self._check_host("topk_weights", w_host, (t, k), torch.float32)
        self._check_host("out", out_host, (t, h), torch.bfloat16)
        ticket = self._submitted
        slot = ticket % self.depth
        reused = ticket >= self.depth
        with torch.cuda.device(self.device):
            with torch.cuda.stream(self._copy_in):
                if reused:  # the step that last read this slot's inputs has finished
                    self._copy_in.wait_event(self._computed[slot])
                self._x[slot].copy_(x_host, non_blocking=True)
                self._ids[slot].copy_(ids_host, non_blocking=True)
                self._w[slot].copy_(w_host, non_blocking=True)
                self._loaded[slot].record(self._copy_in)
            with torch.cuda.stream(self._compute):
                self._compute.wait_event(self._loaded[slot])
                if reused:  # the slot's previous output has left the device
                    self._compute.wait_event(self._stored[slot])
                self.layer.run(self._x[slot], self._ids[slot], self._w[slot], out=self._out[slot])
                self._computed[slot].record(self._compute)
            with torch.cuda.stream(self._copy_out):
                self._copy_out.wait_event(self._computed[slot])
                out_host.copy_(self._out[slot], non_blocking=True)
                self._stored[slot].record(self._copy_out)
        self._submitted += 1
        return ticket

    def wait(self, ticket: int | None = None) -> None:
        """Block the host until the batch's output is in its host buffer (default: all batches)."""
        if ticket is None:
            for slot in range(min(self.depth, self._submitted)):
                self._stored[slot].synchronize()
            return
        if ticket < 0 or ticket >= self._submitted:
            raise ValueError("unknown ticket")
        # a slot's event is re-recorded by later batches on the same stream, so waiting on it
        # also covers every earlier batch of the slot
        self._stored[ticket % self.depth].synchronize()

    @property
    def streams(self):
        """(copy-in, compute, copy-out) streams, for callers that record their own events."""
        return self._copy_in, self._compute, self._copy_out


__all__ = ["HostPipeline"]
