"""Allocation-free NVFP4 MoE inference plan for B200.

Drop-in for ``lightmoe/inference.py`` of the reference: ``InferenceWorkspace``
and ``InferenceMoE`` keep their constructor arguments, methods, private buffer
names and error messages.  Steady-state ``run`` allocates nothing, never
synchronises and launches on the current stream, so a step can be captured in
a CUDA Graph.

Stage order of one step (``lightmoe/inference.py:883-1001``):
dispatch -> quantize gathered rows -> fc1 (activation + requantization fused)
-> fc2 -> weighted combine.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ._quantization import _DEN, quantize_expert_stack
from .kernels.gated import GatedEpilogue
from .kernels.grouped.runtime import GroupedNvfp4Gemm
from .kernels.quantize.decode import (nvfp4_direct_decode_prepare, nvfp4_dispatch_quantize_decode,
                                      nvfp4_quantize_decode)
from .kernels.quantize.runtime import nvfp4_quantize_rowwise
from .kernels.routing.combine import moe_finalize
from .kernels.routing.dispatch import MAX_ASSIGNMENTS, moe_dispatch, scratch_elems
from .kernels.unary import UnaryEpilogue

DECODE_ROWS_PER_EXPERT = 16
FAST_DECODE_ROWS = 64


def _use_swapped_fc2(tokens: int) -> bool:
    return tokens <= 8


def _decode_tile_rows(tokens: int, hidden: int, intermediate: int, experts: int) -> int:
    """Decode tile policy table of the reference (``inference.py:30-36``)."""
    if hidden >= 4096 and intermediate >= 2048 and experts >= 48:
        if tokens >= 64:
            return 32
        if tokens >= 16:
            return 16
    return 8


def _tile_n(n: int, k: int, decode: bool) -> int:
    """Column-tile width of a grouped GEMM.

    128 x 256 tiles pull a quarter less data into the SM per FLOP than 128 x 128 tiles and
    were 1.25x to 1.7x faster on every prefill shape measured (K from 512 to 4096); decode
    steps have few row tiles and keep the narrow tile so that more CTAs share the weight
    traffic.
    """
    return 128 if decode or n % 256 else 256


def _expected_padded_rows(mean_rows: float, tile: int) -> float:
    """Rows an expert occupies once padded to whole ``tile``-row tiles, averaged over a
    per-expert row count drawn from N(mean, mean) (uniform routing)."""
    sigma = max(math.sqrt(mean_rows), 1.0)

    def cdf(v: float) -> float:
        return 0.5 * (1.0 + math.erf((v - mean_rows) / (sigma * math.sqrt(2.0))))

    first = max(0, int((mean_rows - 5.0 * sigma) // tile))
    last = int((mean_rows + 5.0 * sigma) // tile) + 1
    total = 0.0
    for t in range(first, last + 1):
        total += (cdf((t + 1) * tile) - cdf(t * tile)) * (t + 1) * tile
    return total


def _row_tile(policy_tile_m: int, rows: int, experts: int, n: int, k: int, decode: bool, nvfp4_out: bool) -> int:
    """Row-tile height handed to a grouped GEMM: 256 runs 256 x 256 tiles on CTA pairs.

    A pair moves 30 % fewer bytes through each SM's shared memory per FLOP and issues half as
    many MMAs.  Measured per padded row it is about 1.25x faster than 128 x 256 tiles on a
    first projection with K >= 4096 and about 1.1x elsewhere (short contractions and BF16
    output are bound by the epilogue, which a pair does not change).  It pads every expert to
    256 rows, though, so it is chosen when that padding costs less than the pair wins: the
    expected padded rows of both tile heights are compared for the plan's mean rows per
    expert (with about 256 rows per expert the taller tile pads 20 % more and loses; with
    192, or with 512 and more, it wins).  The reference's own table (``_tile_m``) is not
    consulted.
    """
    if decode or n % 256 or rows < 128 * experts:
        return 128
    mean_rows = rows / experts
    gain = 1.22 if (nvfp4_out and k >= 4096) else 1.10
    return 256 if _expected_padded_rows(mean_rows, 256) <= gain * _expected_padded_rows(mean_rows, 128) else 128


def _tile_m(token_expert_assignments: int, experts: int, hidden: int, intermediate: int):
    """Row-tile policy table of the reference (``inference.py:39-50``)."""
    large = token_expert_assignments >= 256 * experts
    fc1 = 256 if large else 128
    fc2 = 256 if large and hidden > 2048 and intermediate > 1024 else 128
    if intermediate <= 1024:
        fc2 = 128
    return fc1, fc2


def _check_positive(name: str, value: int) -> int:
    value = int(value)
    if value <= 0:
        raise ValueError(f"{name} must be positive")
    return value


@dataclass(slots=True)
class _FullExecution:
    fc1: GroupedNvfp4Gemm
    fc2: GroupedNvfp4Gemm
    qx: torch.Tensor
    qh: torch.Tensor
    sfx: torch.Tensor
    sfh: torch.Tensor
    routed_out: torch.Tensor


@dataclass(slots=True)
class InferenceWorkspace:
    """Reusable buffers for plans that execute serially on one stream.

    One byte arena: the quantized input and its scale factors alias the fc2
    output rows, the quantized hidden rows alias the layer output; routing
    metadata follows (``lightmoe/inference.py:95-191``).
    """

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
        sf_rows = -(-rows // 128) + experts
        sfx_shape = (1, sf_rows, hidden_size // 64, 32, 4, 4)
        sfh_shape = (1, sf_rows, intermediate_size // 64, 32, 4, 4)
        qx_bytes = rows * hidden_size // 2
        qh_bytes = rows * intermediate_size // 2
        sfx_bytes = math.prod(sfx_shape)
        sfh_bytes = math.prod(sfh_shape)
        routed_bytes = rows * hidden_size * 2
        out_bytes = max_tokens * hidden_size * 2
        first_bytes = max(qx_bytes + sfx_bytes, routed_bytes)
        second_bytes = max(qh_bytes + sfh_bytes, out_bytes)
        first_bytes = -(-first_bytes // 256) * 256
        second_bytes = -(-second_bytes // 256) * 256
        parts_elems = scratch_elems(rows, experts)
        metadata_bytes = 4 * (rows * 3 + experts + 1 + parts_elems + experts)
        storage_bytes = first_bytes + second_bytes + metadata_bytes
        with torch.cuda.device(device):
            storage = torch.empty(storage_bytes, dtype=torch.uint8, device=device)

        def view(offset, byte_count, dtype, shape):
            return storage[offset : offset + byte_count].view(dtype).view(shape)

        qx_u8 = view(0, qx_bytes, torch.uint8, (rows, hidden_size // 2))
        sfx = view(qx_bytes, sfx_bytes, torch.float8_e4m3fn, sfx_shape)
        routed_out = view(0, routed_bytes, torch.bfloat16, (rows, hidden_size))
        qh_u8 = view(first_bytes, qh_bytes, torch.uint8, (rows, intermediate_size // 2))
        sfh = view(first_bytes + qh_bytes, sfh_bytes, torch.float8_e4m3fn, sfh_shape)
        out = view(first_bytes, out_bytes, torch.bfloat16, (max_tokens, hidden_size))
        cursor = first_bytes + second_bytes

        def take(elements, dtype):
            nonlocal cursor
            result = view(cursor, elements * 4, dtype, (elements,))
            cursor += elements * 4
            return result

        gather = take(rows, torch.int32)
        m_indptr = take(experts + 1, torch.int32)
        probs = take(rows, torch.float32)
        slots = take(rows, torch.int32)
        parts = take(parts_elems, torch.int32)
        padded_offsets = take(experts, torch.int32)
        assert cursor == storage_bytes
        return cls(hidden_size, intermediate_size, experts, topk, max_tokens, device, storage,
                   qx_u8, qh_u8, sfx, sfh, routed_out, out, gather, m_indptr, probs, slots,
                   parts, padded_offsets)

    @property
    def nbytes(self) -> int:
        return self.storage.numel()

    def matches(self, hidden_size, intermediate_size, experts, topk, max_tokens, device) -> bool:
        return (self.hidden_size, self.intermediate_size, self.experts, self.topk,
                self.max_tokens, self.device) == (hidden_size, intermediate_size, experts, topk,
                                                  max_tokens, device)


class InferenceMoE:
    """Static-scale expert plan with caller-selected router assignments."""

    def __init__(
        self,
        hidden_size: int,
        intermediate_size: int,
        num_experts: int,
        top_k: int,
        max_tokens: int,
        *,
        activation: str = "swiglu",
        activation_clamp: float | None = None,
        activation_sigmoid_alpha: float | None = None,
        activation_up_bias: float | None = None,
        use_dynamic_sched: bool | None = None,
        device: torch.device | str = "cuda",
        workspace: InferenceWorkspace | None = None,
    ):
        self.hidden_size = _check_positive("hidden_size", hidden_size)
        self.intermediate_size = _check_positive("intermediate_size", intermediate_size)
        self.experts = _check_positive("num_experts", num_experts)
        self.topk = _check_positive("top_k", top_k)
        self.max_tokens = _check_positive("max_tokens", max_tokens)
        if self.hidden_size % 128 or self.intermediate_size % 128:
            raise ValueError("hidden_size and intermediate_size must align to 128")
        if self.experts > 256:
            raise ValueError("at most 256 local experts are supported")
        if self.topk > self.experts:
            raise ValueError("top_k cannot exceed the local expert count")
        if self.max_tokens * self.topk > MAX_ASSIGNMENTS:
            raise ValueError(f"max_tokens * top_k cannot exceed {MAX_ASSIGNMENTS}")
        if activation not in ("swiglu", "swiglu_oai", "geglu", "reglu", "relu2"):
            raise ValueError("unsupported expert activation")
        oai = activation == "swiglu_oai"
        if oai and activation_clamp is None:
            activation_clamp = 7.0
        if activation_sigmoid_alpha is None:
            activation_sigmoid_alpha = 1.702 if oai else 1.0
        if activation_up_bias is None:
            activation_up_bias = 1.0 if oai else 0.0
        if activation_clamp is not None:
            activation_clamp = float(activation_clamp)
            if not math.isfinite(activation_clamp) or activation_clamp <= 0:
                raise ValueError("activation_clamp must be finite and positive")
            if activation not in ("swiglu", "swiglu_oai"):
                raise ValueError("activation_clamp is supported only for SwiGLU activations")
        activation_sigmoid_alpha = float(activation_sigmoid_alpha)
        activation_up_bias = float(activation_up_bias)
        if not math.isfinite(activation_sigmoid_alpha) or activation_sigmoid_alpha <= 0:
            raise ValueError("activation_sigmoid_alpha must be finite and positive")
        if not math.isfinite(activation_up_bias):
            raise ValueError("activation_up_bias must be finite")
        if not oai and (activation_sigmoid_alpha != 1.0 or activation_up_bias != 0.0):
            raise ValueError("activation sigmoid alpha and up bias require swiglu_oai")

        self.activation = activation
        self.activation_clamp = activation_clamp
        self.activation_sigmoid_alpha = activation_sigmoid_alpha
        self.activation_up_bias = activation_up_bias
        self.use_dynamic_sched = use_dynamic_sched
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("InferenceMoE requires a CUDA device")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())

        geometry = (self.hidden_size, self.intermediate_size, self.experts, self.topk,
                    self.max_tokens, self.device)
        if workspace is None:
            workspace = InferenceWorkspace.allocate(*geometry)
        elif not workspace.matches(*geometry):
            raise ValueError("workspace configuration must match the inference plan")
        self.workspace = workspace
        self._qx_u8 = workspace.qx_u8
        self._qh_u8 = workspace.qh_u8
        self._sfx = workspace.sfx
        self._sfh = workspace.sfh
        self._routed_out = workspace.routed_out
        self._out = workspace.out
        self._gather = workspace.gather
        self._m_indptr = workspace.m_indptr
        self._probs = workspace.probs
        self._slots = workspace.slots
        self._parts = workspace.parts
        self._padded_offsets = workspace.padded_offsets
        with torch.cuda.device(self.device):
            self._x_scale = torch.empty(2, dtype=torch.float32, device=self.device)
            self._h_scale = torch.empty(2, dtype=torch.float32, device=self.device)
            self._alpha1 = torch.empty(1, dtype=torch.float32, device=self.device)
            self._alpha2 = torch.empty(1, dtype=torch.float32, device=self.device)

        # (tile_m, tile_n) forced on every GEMM this plan builds from now on, or None for the
        # policy above; tests use it to compare tilings bit for bit
        self.tile_override: tuple[int, int] | None = None
        self._weights_ready = False
        self._scales_ready = False
        self._full_executions: dict[tuple[int, bool], _FullExecution] = {}
        self._routed_gemms: dict[tuple[str, int], GroupedNvfp4Gemm] = {}
        self._calibration_gemms: dict[int, GroupedNvfp4Gemm] = {}
        self._direct_execution_plan: _FullExecution | None = None

    # ------------------------------------------------------------------ state
    @property
    def output(self) -> torch.Tensor:
        """The reusable full-MoE output workspace."""
        return self._out

    @property
    def workspace_bytes(self) -> int:
        private = (self._x_scale, self._h_scale, self._alpha1, self._alpha2)
        return self.workspace.nbytes + sum(t.numel() * t.element_size() for t in private)

    def _check_tensor(self, tensor, name, shape, dtype) -> None:
        if (
            tuple(tensor.shape) != shape
            or tensor.dtype != dtype
            or tensor.device != self.device
            or not tensor.is_contiguous()
        ):
            raise ValueError(
                f"{name} must be contiguous {dtype} on {self.device} with shape {shape}"
            )

    # ---------------------------------------------------------------- weights
    @torch.no_grad()
    def load_weights(self, gate, up, down=None) -> "InferenceMoE":
        e, d, i = self.experts, self.hidden_size, self.intermediate_size
        if self.activation == "relu2":
            if down is not None:
                raise ValueError("ReLU squared experts use load_weights(up, down)")
            down, up = up, gate
            self._check_tensor(up, "up", (e, i, d), torch.bfloat16)
            self._check_tensor(down, "down", (e, d, i), torch.bfloat16)
            first = up
            amax1 = up.abs().amax()
        else:
            if down is None:
                raise ValueError("gated experts use load_weights(gate, up, down)")
            self._check_tensor(gate, "gate", (e, i, d), torch.bfloat16)
            self._check_tensor(up, "up", (e, i, d), torch.bfloat16)
            self._check_tensor(down, "down", (e, d, i), torch.bfloat16)
            # row 2j = gate_j, row 2j+1 = up_j
            first = torch.stack((gate, up), dim=2).reshape(e, 2 * i, d)
            amax1 = torch.stack((gate.abs().amax(), up.abs().amax())).amax()
        amax2 = down.abs().amax()
        p1 = (amax1.float() / _DEN).clamp_min(1e-30).reshape(1)
        p2 = (amax2.float() / _DEN).clamp_min(1e-30).reshape(1)
        q1, sf1 = quantize_expert_stack(first, p1)
        q2, sf2 = quantize_expert_stack(down, p2)
        return self.load_packed_weights(q1, sf1, p1, q2, sf2, p2)

    @torch.no_grad()
    def load_packed_weights(self, gate_up, gate_up_sf, gate_up_scale, down, down_sf,
                            down_scale) -> "InferenceMoE":
        e, d, i = self.experts, self.hidden_size, self.intermediate_size
        first_projection = i if self.activation == "relu2" else 2 * i
        self._check_tensor(gate_up, "up" if self.activation == "relu2" else "gate_up",
                           (e, first_projection, d // 2), torch.float4_e2m1fn_x2)
        self._check_tensor(gate_up_sf, "gate_up_sf",
                           (e, -(-first_projection // 128), d // 64, 32, 4, 4), torch.float8_e4m3fn)
        self._check_tensor(down, "down", (e, d, i // 2), torch.float4_e2m1fn_x2)
        self._check_tensor(down_sf, "down_sf", (e, -(-d // 128), i // 64, 32, 4, 4),
                           torch.float8_e4m3fn)
        self._check_weight_scale(gate_up_scale, "gate_up_scale")
        self._check_weight_scale(down_scale, "down_scale")
        if self._alpha1.shape != gate_up_scale.shape:
            self._alpha1 = torch.empty_like(gate_up_scale)
        if self._alpha2.shape != down_scale.shape:
            self._alpha2 = torch.empty_like(down_scale)
        self.qb1, self.sfb1, self.p_w1 = gate_up, gate_up_sf, gate_up_scale
        self.qb2, self.sfb2, self.p_w2 = down, down_sf, down_scale
        self._weights_ready = True
        self._full_executions.clear()
        self._routed_gemms.clear()
        self._calibration_gemms.clear()
        self._direct_execution_plan = None
        if self._scales_ready:
            self._refresh_alphas()
        return self

    def _check_weight_scale(self, scale, name) -> None:
        if (
            scale.dtype != torch.float32
            or tuple(scale.shape) not in ((1,), (self.experts,))
            or scale.device != self.device
            or not scale.is_contiguous()
        ):
            raise ValueError(
                f"{name} must be contiguous float32 on {self.device} "
                f"with shape (1,) or ({self.experts},)"
            )

    # ----------------------------------------------------------------- scales
    @torch.no_grad()
    def set_activation_scales(self, input_scale, hidden_scale) -> "InferenceMoE":
        self._set_scale(self._x_scale, input_scale, "input_scale")
        self._set_scale(self._h_scale, hidden_scale, "hidden_scale")
        self._scales_ready = True
        if self._weights_ready:
            self._refresh_alphas()
        return self

    @torch.no_grad()
    def _set_scale(self, target, value, name) -> None:
        if torch.is_tensor(value):
            if value.numel() != 1:
                raise ValueError(f"{name} must contain one value")
            target[:1].copy_(value.detach().to(device=self.device, dtype=torch.float32).reshape(1))
        else:
            value = float(value)
            if not math.isfinite(value) or value <= 0:
                raise ValueError(f"{name} must be finite and positive")
            target[0] = value
        torch.reciprocal(target[:1], out=target[1:])

    @torch.no_grad()
    def _refresh_alphas(self) -> None:
        torch.mul(self._x_scale[:1], self.p_w1, out=self._alpha1)
        torch.mul(self._h_scale[:1], self.p_w2, out=self._alpha2)

    def _require_weights(self) -> None:
        if not self._weights_ready:
            raise RuntimeError("load_weights or load_packed_weights must run first")

    def _require_ready(self) -> None:
        self._require_weights()
        if not self._scales_ready:
            raise RuntimeError("calibrate or set_activation_scales must run first")

    # ------------------------------------------------------------------ plans
    def _views(self, rows: int, *, sf_tile_rows: int = 128):
        sf_rows = -(-rows // 128) + self.experts
        qx = self._qx_u8[:rows].view(torch.float4_e2m1fn_x2)
        qh = self._qh_u8[:rows].view(torch.float4_e2m1fn_x2)
        return qx, qh, self._sfx[:, :sf_rows], self._sfh[:, :sf_rows]

    def _epilogue(self):
        if self.activation == "relu2":
            return UnaryEpilogue(self.activation)
        return GatedEpilogue(self.activation, save_preact=False, clamp_limit=self.activation_clamp,
                             sigmoid_alpha=self.activation_sigmoid_alpha,
                             up_bias=self.activation_up_bias)

    def _new_gemm(self, projection: str, rows: int, output_dtype=torch.bfloat16, *,
                  decode: bool = False):
        schedule = False if decode and self.use_dynamic_sched is None else self.use_dynamic_sched
        fc1_m, fc2_m = _tile_m(rows, self.experts, self.hidden_size, self.intermediate_size)
        if projection == "fc1":
            unary = self.activation == "relu2"
            n1 = self.intermediate_size if unary else 2 * self.intermediate_size
            tile_m, tile_n = self.tile_override or (
                _row_tile(fc1_m, rows, self.experts, n1, self.hidden_size, decode,
                          output_dtype == torch.float4_e2m1fn_x2),
                _tile_n(n1, self.hidden_size, decode))
            if decode and self.tile_override is None:
                # the decode-shaped kernel: weights on the 128-row side of the MMA
                tile_m, tile_n = 128, _decode_tile_rows(rows // self.topk, self.hidden_size,
                                                        self.intermediate_size, self.experts)
            return GroupedNvfp4Gemm(
                self.experts,
                n1,
                self.hidden_size,
                tile_m,
                tile_n,
                output_dtype=output_dtype,
                epilogue=self._epilogue() if output_dtype == torch.float4_e2m1fn_x2 else None,
                use_dynamic_sched=schedule,
                use_pdl=True,
                swap_ab=decode and self.tile_override is None,
                fast_decode_sched=(decode and not schedule and self.hidden_size >= 2048),
            )
        tile_m, tile_n = self.tile_override or (
            _row_tile(fc2_m, rows, self.experts, self.hidden_size, self.intermediate_size, decode, False),
            _tile_n(self.hidden_size, self.intermediate_size, decode))
        if decode and self.tile_override is None:
            tile_m, tile_n = 128, _decode_tile_rows(rows // self.topk, self.hidden_size,
                                                    self.intermediate_size, self.experts)
        return GroupedNvfp4Gemm(
            self.experts,
            self.hidden_size,
            self.intermediate_size,
            tile_m,
            tile_n,
            use_dynamic_sched=schedule,
            use_pdl=True,
            swap_ab=decode and self.tile_override is None,
        )

    def _full_execution(self, tokens: int, *, decode: bool) -> _FullExecution:
        key = (tokens, decode)
        execution = self._full_executions.get(key)
        if execution is not None:
            return execution
        rows = tokens * self.topk
        qx, qh, sfx, sfh = self._views(rows)
        routed_out = self._routed_out[:rows]
        with torch.cuda.device(self.device):
            fc1 = self._new_gemm("fc1", rows, torch.float4_e2m1fn_x2, decode=decode)
            if decode:
                fc1.fast_decode_sched = not fc1.use_dynamic_sched
            fc2 = self._new_gemm("fc2", rows, decode=decode)
            # fc2 follows fc1 directly and its routing table is older than fc1: its weight
            # stream may start while fc1 drains
            fc2.weights_ahead = decode and fc2.swap_ab
        fc1.prepare(qx, self.qb1, qh, self._m_indptr, sfx, self.sfb1, self._alpha1,
                    output_sf=sfh, output_scale=self._h_scale)
        fc2.prepare(qh, self.qb2, routed_out, self._m_indptr, sfh, self.sfb2, self._alpha2)
        execution = _FullExecution(fc1, fc2, qx, qh, sfx, sfh, routed_out)
        self._full_executions[key] = execution
        return execution

    def _direct_execution(self) -> _FullExecution:
        """The one-token step without a dispatch (``lightmoe/inference.py:656-721``): the token is
        quantized once, both GEMMs walk the ``top_k`` routes in route order with the expert ids
        in the first ``top_k`` words of ``_m_indptr``; fc1 reads row 0 for every route."""
        execution = self._direct_execution_plan
        if execution is not None:
            return execution
        rows = self.topk
        qx, qh, sfx, sfh = self._views(rows)
        routed_out = self._routed_out[:rows]
        route_ids = self._m_indptr[: self.topk]
        unary = self.activation == "relu2"
        with torch.cuda.device(self.device):
            fc1 = GroupedNvfp4Gemm(
                self.experts, self.intermediate_size if unary else 2 * self.intermediate_size,
                self.hidden_size, 128, 128, output_dtype=torch.float4_e2m1fn_x2, epilogue=self._epilogue(),
                use_dynamic_sched=False, use_pdl=True, direct_routes=self.topk, broadcast_a=True)
            fc2 = GroupedNvfp4Gemm(self.experts, self.hidden_size, self.intermediate_size, 128, 128,
                                   use_dynamic_sched=False, use_pdl=True, direct_routes=self.topk)
            fc2.weights_ahead = True
        fc1.prepare(qx, self.qb1, qh, route_ids, sfx, self.sfb1, self._alpha1, output_sf=sfh,
                    output_scale=self._h_scale)
        fc2.prepare(qh, self.qb2, routed_out, route_ids, sfh, self.sfb2, self._alpha2)
        execution = _FullExecution(fc1, fc2, qx, qh, sfx, sfh, routed_out)
        self._direct_execution_plan = execution
        return execution

    # ------------------------------------------------------------ calibration
    @torch.no_grad()
    def calibrate_routed(self, x, m_indptr, padded_offsets) -> "InferenceMoE":
        self._require_weights()
        rows = x.shape[0]
        self._validate_routed(x, m_indptr, padded_offsets)
        input_scale = (x.abs().amax().float() / _DEN).clamp_min(1e-30).reshape(1)
        self._set_scale(self._x_scale, input_scale, "input_scale")
        qx, _, sfx, _ = self._views(rows)
        nvfp4_quantize_rowwise(x, m_indptr, self._x_scale, qx, sfx,
                               padded_offsets=padded_offsets, te_math=True)
        preact_cols = (self.intermediate_size if self.activation == "relu2"
                       else 2 * self.intermediate_size)
        preact = torch.empty(rows, preact_cols, dtype=torch.bfloat16, device=self.device)
        fc1 = self._calibration_gemms.get(rows)
        if fc1 is None:
            with torch.cuda.device(self.device):
                fc1 = self._new_gemm("fc1", rows)
            self._calibration_gemms[rows] = fc1
        torch.mul(self._x_scale[:1], self.p_w1, out=self._alpha1)
        fc1(qx, self.qb1, preact, m_indptr, sfx, self.sfb1, self._alpha1)
        if self.activation == "relu2":
            hidden = torch.relu(preact.float()).square_()
        else:
            gate = preact[:, 0::2].float()
            up = preact[:, 1::2].float()
            if self.activation_clamp is not None:
                gate.clamp_(max=self.activation_clamp)
                up.clamp_(min=-self.activation_clamp, max=self.activation_clamp)
            if self.activation == "swiglu":
                hidden = torch.nn.functional.silu(gate).mul_(up)
            elif self.activation == "swiglu_oai":
                hidden = gate.mul(torch.sigmoid(self.activation_sigmoid_alpha * gate)).mul_(
                    up.add(self.activation_up_bias))
            elif self.activation == "geglu":
                hidden = torch.nn.functional.gelu(gate, approximate="tanh").mul_(up)
            else:
                hidden = torch.nn.functional.relu(gate).mul_(up)
        hidden_scale = (hidden.abs().amax().float() / _DEN).clamp_min(1e-30).reshape(1)
        self._set_scale(self._h_scale, hidden_scale, "hidden_scale")
        self._scales_ready = True
        self._refresh_alphas()
        return self

    @torch.no_grad()
    def calibrate(self, x, topk_ids, topk_weights) -> "InferenceMoE":
        tokens = self._validate_full(x, topk_ids, topk_weights)
        rows = tokens * self.topk
        self._dispatch(topk_ids, topk_weights, rows)
        gathered = x.index_select(0, self._gather[:rows].long())
        return self.calibrate_routed(gathered, self._m_indptr, self._padded_offsets)

    # ------------------------------------------------------------- validation
    def _validate_routed(self, x, m_indptr, padded_offsets) -> int:
        rows = int(x.shape[0])
        if rows <= 0 or rows > self.max_tokens * self.topk:
            raise ValueError("token-expert assignment rows must be within the configured workspace")
        self._check_tensor(x, "x", (rows, self.hidden_size), torch.bfloat16)
        self._check_tensor(m_indptr, "m_indptr", (self.experts + 1,), torch.int32)
        self._check_tensor(padded_offsets, "padded_offsets", (self.experts,), torch.int32)
        return rows

    def _validate_full(self, x, topk_ids, topk_weights) -> int:
        tokens = int(x.shape[0])
        if tokens <= 0 or tokens > self.max_tokens:
            raise ValueError("token count must be within the configured workspace")
        self._check_tensor(x, "x", (tokens, self.hidden_size), torch.bfloat16)
        self._check_tensor(topk_ids, "topk_ids", (tokens, self.topk), torch.int32)
        self._check_tensor(topk_weights, "topk_weights", (tokens, self.topk), torch.float32)
        return tokens

    def _output_view(self, output, rows: int, name: str):
        if output is None:
            source = self._routed_out if name == "routed_out" else self._out
            return source[:rows]
        self._check_tensor(output, name, (rows, self.hidden_size), torch.bfloat16)
        return output

    def _dispatch(self, topk_ids, topk_weights, rows: int) -> None:
        moe_dispatch(topk_ids, topk_weights, self.experts, self._gather[:rows], self._m_indptr,
                     self._probs[:rows], self._slots[:rows], self._parts, self._padded_offsets)

    # -------------------------------------------------------------- execution
    @torch.no_grad()
    def run_routed(self, x, m_indptr, padded_offsets, *, out=None) -> torch.Tensor:
        """Expert-major entry point: rows already grouped by expert."""
        self._require_ready()
        rows = self._validate_routed(x, m_indptr, padded_offsets)
        qx, qh, sfx, sfh = self._views(rows)
        routed_out = self._output_view(out, rows, "routed_out")
        nvfp4_quantize_rowwise(x, m_indptr, self._x_scale, qx, sfx,
                               padded_offsets=padded_offsets, te_math=True)
        fc1_m, fc2_m = _tile_m(rows, self.experts, self.hidden_size, self.intermediate_size)
        with torch.cuda.device(self.device):
            fc1 = self._routed_gemms.get(("fc1", fc1_m))
            if fc1 is None:
                fc1 = self._new_gemm("fc1", rows, torch.float4_e2m1fn_x2)
                self._routed_gemms[("fc1", fc1_m)] = fc1
            fc2 = self._routed_gemms.get(("fc2", fc2_m))
            if fc2 is None:
                fc2 = self._new_gemm("fc2", rows)
                self._routed_gemms[("fc2", fc2_m)] = fc2
        fc1(qx, self.qb1, qh, m_indptr, sfx, self.sfb1, self._alpha1, output_sf=sfh,
            output_scale=self._h_scale)
        fc2(qh, self.qb2, routed_out, m_indptr, sfh, self.sfb2, self._alpha2)
        return routed_out

    @torch.no_grad()
    def run_prefill(self, x, topk_ids, topk_weights, *, out=None) -> torch.Tensor:
        self._require_ready()
        tokens = self._validate_full(x, topk_ids, topk_weights)
        rows = tokens * self.topk
        output = self._output_view(out, tokens, "out")
        execution = self._full_execution(tokens, decode=False)
        self._dispatch(topk_ids, topk_weights, rows)
        # each token is quantized once and its codes and scale factors are written to all of
        # its expert-major rows: same bits as quantizing the gathered rows, 1/top_k of the math
        nvfp4_quantize_decode(x, topk_ids, self._slots[:rows], self._m_indptr,
                              self._padded_offsets, self._x_scale, execution.qx, execution.sfx)
        execution.fc1.launch()
        execution.fc2.launch()
        moe_finalize(execution.routed_out, self._slots[:rows], output, self.topk, tile_t=1,
                     n_frag=2, weights=self._probs[:rows], use_pdl=True)
        return output

    @torch.no_grad()
    def run_decode(self, x, topk_ids, topk_weights, *, out=None) -> torch.Tensor:
        """Small-batch step: each token is quantized once and scattered to its slots."""
        self._require_ready()
        tokens = self._validate_full(x, topk_ids, topk_weights)
        rows = tokens * self.topk
        output = self._output_view(out, tokens, "out")
        if tokens == 1 and self.topk <= 32 and self.tile_override is None:
            # one token: no dispatch, the routes keep their order
            execution = self._direct_execution()
            nvfp4_direct_decode_prepare(x, topk_ids, topk_weights, self._gather[:rows], self._slots[:rows],
                                        self._m_indptr[: self.topk], self._probs[:rows],
                                        self._padded_offsets, self._x_scale, execution.qx, execution.sfx)
            execution.fc1.launch()
            execution.fc2.launch()
            moe_finalize(execution.routed_out, self._slots[:rows], output, self.topk, tile_t=1,
                         n_frag=2, weights=self._probs[:rows], use_pdl=True)
            return output
        execution = self._full_execution(tokens, decode=True)
        if rows <= 1024:
            # one launch: dispatch + decode plan + quantize-once-and-scatter
            nvfp4_dispatch_quantize_decode(x, topk_ids, topk_weights, self._parts,
                                           self._gather[:rows], self._m_indptr, self._probs[:rows],
                                           self._slots[:rows], self._padded_offsets, self._x_scale,
                                           execution.qx, execution.sfx)
        else:
            self._dispatch(topk_ids, topk_weights, rows)
            nvfp4_quantize_decode(x, topk_ids, self._slots[:rows], self._m_indptr,
                                  self._padded_offsets, self._x_scale, execution.qx, execution.sfx)
        execution.fc1.launch()
        execution.fc2.launch()
        moe_finalize(execution.routed_out, self._slots[:rows], output, self.topk, tile_t=1,
                     n_frag=2, weights=self._probs[:rows], use_pdl=True,
                     num_threads=768 if self.hidden_size >= 2048 else 256)
        return output

    @torch.no_grad()
    def run(self, x, topk_ids, topk_weights, *, out=None) -> torch.Tensor:
        rows = x.shape[0] * self.topk
        if rows <= DECODE_ROWS_PER_EXPERT * self.experts:
            return self.run_decode(x, topk_ids, topk_weights, out=out)
        return self.run_prefill(x, topk_ids, topk_weights, out=out)

    __call__ = run

    @torch.no_grad()
    def warmup(self, x, topk_ids, topk_weights, *, iterations: int = 2) -> None:
        if iterations <= 0:
            raise ValueError("iterations must be positive")
        for _ in range(iterations):
            self.run(x, topk_ids, topk_weights)
        torch.cuda.synchronize(self.device)


__all__ = ["InferenceMoE", "InferenceWorkspace"]
