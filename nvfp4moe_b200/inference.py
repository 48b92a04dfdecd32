"""Allocation-free NVFP4 MoE inference plan for B200.

Drop-in for ``lightmoe/inference.py`` of the reference: ``InferenceWorkspace`` and
``InferenceMoE`` keep their constructor arguments, methods, private buffer names and error
messages (the reference's tests pin them).  Steady-state ``run`` allocates nothing, never
synchronises and launches on the current stream, so a step can be captured in a CUDA Graph.

One step (``lightmoe/inference.py:883-1001``): dispatch -> quantize each token once into its
expert-major rows -> fc1 (activation + requantization in the epilogue) -> fc2 -> weighted
combine.  Which kernels carry a step:

    prefill            two-launch dispatch, quantize-once-scatter, 128 x 256 tiles or CTA pairs
    decode (rows <= 16 per expert on average)
                       fused dispatch + quantize (up to 1024 routes); up to 128 routes the
                       decode-shaped GEMM (weights on the 128-row side of the MMA) as programmatic
                       dependents, beyond that 128 x 256 tiles
    one token          no dispatch at all: direct routes
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib
from ._quantization import _DEN, quantize_expert_stack
from .kernels.gated import GatedEpilogue
from .kernels.grouped.runtime import GroupedNvfp4Gemm
from .kernels.quantize.decode import (nvfp4_direct_decode_prepare, nvfp4_dispatch_quantize_decode,
                                      nvfp4_quantize_decode)
from .kernels.quantize.runtime import nvfp4_quantize_rowwise
from .kernels.routing.combine import moe_finalize
from .kernels.routing.dispatch import MAX_ASSIGNMENTS, moe_dispatch
from .kernels.unary import UnaryEpilogue
from .policy import (DECODE_ROWS_PER_EXPERT, FAST_DECODE_ROWS, FUSED_PREPARE_MAX_ROWS, SWAPPED_MAX_ROWS,  # noqa: F401
                     _decode_tile_rows, _tile_m, _use_swapped_fc2, pick_tiles)
from .workspace import InferenceWorkspace

_ACTIVATIONS = ("swiglu", "swiglu_oai", "geglu", "reglu", "relu2")
_FP4 = torch.float4_e2m1fn_x2


def _positive(name: str, value) -> int:
    value = int(value)
    if value <= 0:
        raise ValueError(f"{name} must be positive")
    return value


def _activation_settings(activation, clamp, sigmoid_alpha, up_bias):
    """Defaults and checks of the activation arguments (``lightmoe/inference.py:250-277``)."""
    if activation not in _ACTIVATIONS:
        raise ValueError("unsupported expert activation")
    oai = activation == "swiglu_oai"
    clamp = 7.0 if (oai and clamp is None) else clamp
    sigmoid_alpha = (1.702 if oai else 1.0) if sigmoid_alpha is None else sigmoid_alpha
    up_bias = (1.0 if oai else 0.0) if up_bias is None else up_bias
    if clamp is not None:
        clamp = float(clamp)
        if not math.isfinite(clamp) or clamp <= 0:
            raise ValueError("activation_clamp must be finite and positive")
        if activation not in ("swiglu", "swiglu_oai"):
            raise ValueError("activation_clamp is supported only for SwiGLU activations")
    sigmoid_alpha, up_bias = float(sigmoid_alpha), float(up_bias)
    if not math.isfinite(sigmoid_alpha) or sigmoid_alpha <= 0:
        raise ValueError("activation_sigmoid_alpha must be finite and positive")
    if not math.isfinite(up_bias):
        raise ValueError("activation_up_bias must be finite")
    if not oai and (sigmoid_alpha != 1.0 or up_bias != 0.0):
        raise ValueError("activation sigmoid alpha and up bias require swiglu_oai")
    return clamp, sigmoid_alpha, up_bias


@dataclass(slots=True)
class _FullExecution:
    fc1: GroupedNvfp4Gemm
    fc2: GroupedNvfp4Gemm
    qx: torch.Tensor
    qh: torch.Tensor
    sfx: torch.Tensor
    sfh: torch.Tensor
    routed_out: torch.Tensor


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
        self.hidden_size = _positive("hidden_size", hidden_size)
        self.intermediate_size = _positive("intermediate_size", intermediate_size)
        self.experts = _positive("num_experts", num_experts)
        self.topk = _positive("top_k", top_k)
        self.max_tokens = _positive("max_tokens", max_tokens)
        for broken, message in (
            (self.hidden_size % 128 or self.intermediate_size % 128,
             "hidden_size and intermediate_size must align to 128"),
            (self.experts > 256, "at most 256 local experts are supported"),
            (self.topk > self.experts, "top_k cannot exceed the local expert count"),
            (self.max_tokens * self.topk > MAX_ASSIGNMENTS, f"max_tokens * top_k cannot exceed {MAX_ASSIGNMENTS}"),
        ):
            if broken:
                raise ValueError(message)
        self.activation = activation
        (self.activation_clamp, self.activation_sigmoid_alpha,
         self.activation_up_bias) = _activation_settings(activation, activation_clamp, activation_sigmoid_alpha,
                                                         activation_up_bias)
        self.use_dynamic_sched = use_dynamic_sched
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("InferenceMoE requires a CUDA device")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())

        geometry = (self.hidden_size, self.intermediate_size, self.experts, self.topk, self.max_tokens,
                    self.device)
        if workspace is None:
            workspace = InferenceWorkspace.allocate(*geometry)
        elif not workspace.matches(*geometry):
            raise ValueError("workspace configuration must match the inference plan")
        self.workspace = workspace
        # the private names of the reference's plan (its tests read them)
        for private, member in (("_qx_u8", "qx_u8"), ("_qh_u8", "qh_u8"), ("_sfx", "sfx"), ("_sfh", "sfh"),
                                ("_routed_out", "routed_out"), ("_out", "out"), ("_gather", "gather"),
                                ("_m_indptr", "m_indptr"), ("_probs", "probs"), ("_slots", "slots"),
                                ("_parts", "parts"), ("_padded_offsets", "padded_offsets")):
            setattr(self, private, getattr(workspace, member))
        with torch.cuda.device(self.device):
            # [scale, 1 / scale] pairs, the GEMM alphas (activation scale x weight scale) and the
            # device word the calibration kernel reduces into
            self._x_scale = torch.empty(2, dtype=torch.float32, device=self.device)
            self._h_scale = torch.empty(2, dtype=torch.float32, device=self.device)
            self._alpha1 = torch.empty(1, dtype=torch.float32, device=self.device)
            self._alpha2 = torch.empty(1, dtype=torch.float32, device=self.device)
            self._amax = torch.zeros(1, dtype=torch.float32, device=self.device)

        # (tile_m, tile_n) forced on every GEMM this plan builds from now on, or None for the
        # measured policy; tests use it to compare tilings bit for bit
        self.tile_override: tuple[int, int] | None = None
        self._weights_ready = False
        self._scales_ready = False
        self._full_executions: dict[tuple[int, bool], _FullExecution] = {}
        self._routed_gemms: dict[tuple[str, int], GroupedNvfp4Gemm] = {}
        self._calibration_gemms: dict[int, GroupedNvfp4Gemm] = {}
        self._direct_execution_plan: _FullExecution | None = None  # the one used last
        self._direct_plans: dict[int | None, _FullExecution] = {}
        self._direct_seen: set[int] = set()

    # ------------------------------------------------------------------ state
    @property
    def output(self) -> torch.Tensor:
        """The reusable full-MoE output workspace."""
        return self._out

    @property
    def workspace_bytes(self) -> int:
        private = (self._x_scale, self._h_scale, self._alpha1, self._alpha2)
        return self.workspace.nbytes + sum(t.numel() * t.element_size() for t in private)

    @property
    def _first_projection_rows(self) -> int:
        return self.intermediate_size if self.activation == "relu2" else 2 * self.intermediate_size

    def _check_tensor(self, tensor, name, shape, dtype) -> None:
        fine = (tuple(tensor.shape) == shape and tensor.dtype == dtype and tensor.device == self.device
                and tensor.is_contiguous())
        if not fine:
            raise ValueError(f"{name} must be contiguous {dtype} on {self.device} with shape {shape}")

    def _forget_plans(self) -> None:
        self._full_executions.clear()
        self._routed_gemms.clear()
        self._calibration_gemms.clear()
        self._direct_execution_plan = None
        self._direct_plans.clear()
        self._direct_seen.clear()

    # ---------------------------------------------------------------- weights
    @torch.no_grad()
    def load_weights(self, gate, up, down=None) -> "InferenceMoE":
        """BF16 master weights -> NVFP4, one scale per projection.  Gated experts pass
        ``(gate, up, down)``, ReLU squared experts ``(up, down)``."""
        e, d, i = self.experts, self.hidden_size, self.intermediate_size
        if self.activation == "relu2":
            if down is not None:
                raise ValueError("ReLU squared experts use load_weights(up, down)")
            first, down = gate, up
            self._check_tensor(first, "up", (e, i, d), torch.bfloat16)
            self._check_tensor(down, "down", (e, d, i), torch.bfloat16)
            amax_first = first.abs().amax()
        else:
            if down is None:
                raise ValueError("gated experts use load_weights(gate, up, down)")
            for tensor, name in ((gate, "gate"), (up, "up")):
                self._check_tensor(tensor, name, (e, i, d), torch.bfloat16)
            self._check_tensor(down, "down", (e, d, i), torch.bfloat16)
            amax_first = torch.maximum(gate.abs().amax(), up.abs().amax())
            # fc1 rows alternate: row 2j = gate_j, row 2j + 1 = up_j, so that an accumulator's
            # neighbouring columns are the pair one output needs
            first = torch.empty(e, i, 2, d, dtype=torch.bfloat16, device=self.device)
            first[:, :, 0].copy_(gate)
            first[:, :, 1].copy_(up)
            first = first.view(e, 2 * i, d)
        scale_first = (amax_first.float() / _DEN).clamp_min(1e-30).reshape(1)
        scale_down = (down.abs().amax().float() / _DEN).clamp_min(1e-30).reshape(1)
        packed_first = quantize_expert_stack(first, scale_first)
        del first
        packed_down = quantize_expert_stack(down, scale_down)
        return self.load_packed_weights(*packed_first, scale_first, *packed_down, scale_down)

    @torch.no_grad()
    def load_packed_weights(self, gate_up, gate_up_sf, gate_up_scale, down, down_sf,
                            down_scale) -> "InferenceMoE":
        """Checkpoint tensors as they are: packed codes, blocked scale factors and a scale of
        shape (1,) or (experts,) per projection (``lightmoe/inference.py:398-456``)."""
        e, d, i = self.experts, self.hidden_size, self.intermediate_size
        n1 = self._first_projection_rows
        self._check_tensor(gate_up, "up" if self.activation == "relu2" else "gate_up", (e, n1, d // 2), _FP4)
        self._check_tensor(gate_up_sf, "gate_up_sf", (e, -(-n1 // 128), d // 64, 32, 4, 4), torch.float8_e4m3fn)
        self._check_tensor(down, "down", (e, d, i // 2), _FP4)
        self._check_tensor(down_sf, "down_sf", (e, -(-d // 128), i // 64, 32, 4, 4), torch.float8_e4m3fn)
        self._check_weight_scale(gate_up_scale, "gate_up_scale")
        self._check_weight_scale(down_scale, "down_scale")
        # the alphas take the shape of the weight scales (one value, or one per expert)
        if self._alpha1.shape != gate_up_scale.shape:
            self._alpha1 = torch.empty_like(gate_up_scale)
        if self._alpha2.shape != down_scale.shape:
            self._alpha2 = torch.empty_like(down_scale)
        self.qb1, self.sfb1, self.p_w1 = gate_up, gate_up_sf, gate_up_scale
        self.qb2, self.sfb2, self.p_w2 = down, down_sf, down_scale
        self._weights_ready = True
        self._forget_plans()  # prepared GEMMs hold the old operands
        if self._scales_ready:
            self._refresh_alphas()
        return self

    def _check_weight_scale(self, scale, name) -> None:
        fine = (scale.dtype == torch.float32 and tuple(scale.shape) in ((1,), (self.experts,))
                and scale.device == self.device and scale.is_contiguous())
        if not fine:
            raise ValueError(f"{name} must be contiguous float32 on {self.device} "
                             f"with shape (1,) or ({self.experts},)")

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
    def _set_scale(self, pair, value, name) -> None:
        """``pair`` <- [value, 1 / value]; a tensor value never passes through the host."""
        if torch.is_tensor(value):
            if value.numel() != 1:
                raise ValueError(f"{name} must contain one value")
            pair[:1].copy_(value.detach().to(device=self.device, dtype=torch.float32).reshape(1))
        else:
            number = float(value)
            if not math.isfinite(number) or number <= 0:
                raise ValueError(f"{name} must be finite and positive")
            pair[0] = number
        torch.reciprocal(pair[:1], out=pair[1:])

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
        """Operand views of a step with ``rows`` rows: packed input, packed hidden rows and the
        leading atom rows of both scale-factor buffers."""
        atom_rows = -(-rows // 128) + self.experts
        return (self._qx_u8[:rows].view(_FP4), self._qh_u8[:rows].view(_FP4),
                self._sfx[:, :atom_rows], self._sfh[:, :atom_rows])

    def _epilogue(self):
        if self.activation == "relu2":
            return UnaryEpilogue(self.activation)
        return GatedEpilogue(self.activation, save_preact=False, clamp_limit=self.activation_clamp,
                             sigmoid_alpha=self.activation_sigmoid_alpha, up_bias=self.activation_up_bias)

    def _new_gemm(self, projection: str, rows: int, output_dtype=torch.bfloat16, *, decode: bool = False):
        """A grouped GEMM of this layer for a step of ``rows`` rows: ``"fc1"`` (output BF16 for
        calibration, NVFP4 with the fused epilogue otherwise) or ``"fc2"``."""
        first = projection == "fc1"
        n, k = ((self._first_projection_rows, self.hidden_size) if first
                else (self.hidden_size, self.intermediate_size))
        fused = first and output_dtype == _FP4
        # decode steps keep the static schedule unless the caller asked otherwise
        schedule = False if (decode and self.use_dynamic_sched is None) else self.use_dynamic_sched
        swapped = decode and self.tile_override is None and rows <= SWAPPED_MAX_ROWS
        if self.tile_override is not None:
            tile_m, tile_n = self.tile_override
        elif swapped:
            # the decode-shaped kernel: weights on the 128-row side of the MMA
            tile_m, tile_n = 128, _decode_tile_rows(max(rows // self.topk, 1), self.hidden_size,
                                                    self.intermediate_size, self.experts)
        else:
            tile_m, tile_n = pick_tiles(rows, self.experts, n, k, nvfp4_out=fused)
        return GroupedNvfp4Gemm(
            self.experts, n, k, tile_m, tile_n,
            output_dtype=output_dtype if first else torch.bfloat16,
            epilogue=self._epilogue() if fused else None,
            use_dynamic_sched=schedule,
            # decode-shaped launches always chain; prefill launches only in short steps, where
            # a kernel's set-up beside its predecessor is a tenth of the step (a long prefill
            # chain measured 5 % slower with it)
            use_pdl=swapped or rows <= FUSED_PREPARE_MAX_ROWS,
            swap_ab=swapped,
            fast_decode_sched=first and decode and not schedule and self.hidden_size >= 2048,
        )

    def _pair_of_gemms(self, fc1, fc2, rows, cu, *, first_cu=None) -> _FullExecution:
        """Prepare fc1 -> fc2 over the plan's own buffers for ``rows`` rows routed by ``cu``
        (``first_cu``: fc1 reads the same routing from another tensor)."""
        qx, qh, sfx, sfh = self._views(rows)
        routed_out = self._routed_out[:rows]
        fc1.prepare(qx, self.qb1, qh, cu if first_cu is None else first_cu, sfx, self.sfb1, self._alpha1,
                    output_sf=sfh, output_scale=self._h_scale)
        fc2.prepare(qh, self.qb2, routed_out, cu, sfh, self.sfb2, self._alpha2)
        fc1.trace_name, fc2.trace_name = "lightmoe.fc1", "lightmoe.fc2"
        return _FullExecution(fc1, fc2, qx, qh, sfx, sfh, routed_out)

    def _full_execution(self, tokens: int, *, decode: bool) -> _FullExecution:
        key = (tokens, decode)
        execution = self._full_executions.get(key)
        if execution is None:
            rows = tokens * self.topk
            with torch.cuda.device(self.device):
                fc1 = self._new_gemm("fc1", rows, _FP4, decode=decode)
                fc2 = self._new_gemm("fc2", rows, decode=decode)
            if decode:
                fc1.fast_decode_sched = not fc1.use_dynamic_sched
                # fc2 follows fc1 directly and its routing table is older than fc1: its weight
                # stream may start while fc1 drains
                fc2.weights_ahead = fc2.swap_ab
            execution = self._full_executions[key] = self._pair_of_gemms(fc1, fc2, rows, self._m_indptr)
        return execution

    def _direct_execution(self, topk_ids=None) -> _FullExecution:
        """The one-token step without a dispatch (``lightmoe/inference.py:656-721``): the token is
        quantized once, both GEMMs walk the ``top_k`` routes in route order with the expert ids
        in the first ``top_k`` words of ``_m_indptr``; fc1 reads row 0 for every route.

        With ``topk_ids`` fc1 reads the expert ids from the caller's tensor instead, which the
        prepare launch only copies: the ids are older than that launch, so fc1 may read them and
        start its weight stream while the prepare launch still quantizes.  The prepared GEMM holds
        the tensor's address, hence one plan per address (a handful: a serving loop or a captured
        graph passes the same buffers every step)."""
        key = None if topk_ids is None else topk_ids.data_ptr()
        if key is not None and key not in self._direct_plans and key not in self._direct_seen:
            # an address met for the first time runs on the shared plan: only one that comes
            # back (a serving loop's buffer, a captured graph) is worth a plan of its own
            if len(self._direct_seen) >= 64:
                self._direct_seen.clear()
            self._direct_seen.add(key)
            key, topk_ids = None, None
        execution = self._direct_plans.get(key)
        if execution is None:
            common = dict(use_dynamic_sched=False, use_pdl=True, direct_routes=self.topk)
            with torch.cuda.device(self.device):
                fc1 = GroupedNvfp4Gemm(self.experts, self._first_projection_rows, self.hidden_size, 128, 128,
                                       output_dtype=_FP4, epilogue=self._epilogue(), broadcast_a=True, **common)
                fc2 = GroupedNvfp4Gemm(self.experts, self.hidden_size, self.intermediate_size, 128, 128, **common)
            fc2.weights_ahead = True
            fc1.weights_ahead = topk_ids is not None
            execution = self._pair_of_gemms(fc1, fc2, self.topk, self._m_indptr[: self.topk],
                                            first_cu=None if topk_ids is None else topk_ids.view(-1))
            while len(self._direct_plans) >= 16:
                self._direct_plans.pop(next(k for k in self._direct_plans if k is not None))
            self._direct_plans[key] = execution
        self._direct_execution_plan = execution
        return execution

    # ------------------------------------------------------------ calibration
    @torch.no_grad()
    def calibrate_routed(self, x, m_indptr, padded_offsets) -> "InferenceMoE":
        """Static scales from one expert-major batch: the input scale from amax(x); the hidden
        scale from amax of the activation applied to a BF16 fc1 result, reduced on the device
        (``lm_activation_amax``) so that nothing larger than that result is allocated."""
        self._require_weights()
        rows = self._validate_routed(x, m_indptr, padded_offsets)
        self._set_scale(self._x_scale, (x.abs().amax().float() / _DEN).clamp_min(1e-30).reshape(1), "input_scale")
        qx, _, sfx, _ = self._views(rows)
        nvfp4_quantize_rowwise(x, m_indptr, self._x_scale, qx, sfx, padded_offsets=padded_offsets, te_math=True)
        n1 = self._first_projection_rows
        preact = torch.empty(rows, n1, dtype=torch.bfloat16, device=self.device)
        fc1 = self._calibration_gemms.get(rows)
        if fc1 is None:
            with torch.cuda.device(self.device):
                fc1 = self._calibration_gemms[rows] = self._new_gemm("fc1", rows)
        torch.mul(self._x_scale[:1], self.p_w1, out=self._alpha1)
        fc1(qx, self.qb1, preact, m_indptr, sfx, self.sfb1, self._alpha1)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lm_activation_amax(
                preact.data_ptr(), rows, n1, _lib.ACTIVATIONS[self.activation], self.activation_clamp or 0.0,
                self.activation_sigmoid_alpha, self.activation_up_bias, self._amax.data_ptr(),
                _lib.stream_handle()))
        self._set_scale(self._h_scale, (self._amax / _DEN).clamp_min(1e-30), "hidden_scale")
        self._scales_ready = True
        self._refresh_alphas()
        return self

    @torch.no_grad()
    def calibrate(self, x, topk_ids, topk_weights) -> "InferenceMoE":
        tokens = self._validate_full(x, topk_ids, topk_weights)
        rows = tokens * self.topk
        self._dispatch(topk_ids, topk_weights, rows)
        return self.calibrate_routed(x.index_select(0, self._gather[:rows].long()), self._m_indptr,
                                     self._padded_offsets)

    # ------------------------------------------------------------- validation
    def _validate_routed(self, x, m_indptr, padded_offsets) -> int:
        rows = int(x.shape[0])
        if not 0 < rows <= self.max_tokens * self.topk:
            raise ValueError("token-expert assignment rows must be within the configured workspace")
        self._check_tensor(x, "x", (rows, self.hidden_size), torch.bfloat16)
        self._check_tensor(m_indptr, "m_indptr", (self.experts + 1,), torch.int32)
        self._check_tensor(padded_offsets, "padded_offsets", (self.experts,), torch.int32)
        return rows

    def _validate_full(self, x, topk_ids, topk_weights) -> int:
        tokens = int(x.shape[0])
        if not 0 < tokens <= self.max_tokens:
            raise ValueError("token count must be within the configured workspace")
        self._check_tensor(x, "x", (tokens, self.hidden_size), torch.bfloat16)
        self._check_tensor(topk_ids, "topk_ids", (tokens, self.topk), torch.int32)
        self._check_tensor(topk_weights, "topk_weights", (tokens, self.topk), torch.float32)
        return tokens

    def _output_view(self, output, rows: int, name: str):
        if output is None:
            return (self._routed_out if name == "routed_out" else self._out)[:rows]
        self._check_tensor(output, name, (rows, self.hidden_size), torch.bfloat16)
        return output

    def _dispatch(self, topk_ids, topk_weights, rows: int) -> None:
        moe_dispatch(topk_ids, topk_weights, self.experts, self._gather[:rows], self._m_indptr,
                     self._probs[:rows], self._slots[:rows], self._parts, self._padded_offsets)

    # -------------------------------------------------------------- execution
    def _finish(self, execution: _FullExecution, rows: int, output, *, threads: int = 256):
        """fc1 -> fc2 -> weighted combine of a prepared step."""
        execution.fc1.launch()
        execution.fc2.launch()
        # the combine chains to fc2 where fc2 itself chains (short steps); behind a long prefill
        # GEMM an early-launched combine measured 14 us slower on the 8192-token layer
        moe_finalize(execution.routed_out, self._slots[:rows], output, self.topk, tile_t=1, n_frag=2,
                     weights=self._probs[:rows], use_pdl=execution.fc2.use_pdl, num_threads=threads)
        return output

    @torch.no_grad()
    def run_routed(self, x, m_indptr, padded_offsets, *, out=None) -> torch.Tensor:
        """Expert-major entry point: rows already grouped by expert; returns the fc2 rows."""
        self._require_ready()
        rows = self._validate_routed(x, m_indptr, padded_offsets)
        qx, qh, sfx, sfh = self._views(rows)
        routed_out = self._output_view(out, rows, "routed_out")
        nvfp4_quantize_rowwise(x, m_indptr, self._x_scale, qx, sfx, padded_offsets=padded_offsets, te_math=True)
        # the GEMMs are cached per row-tile class of the reference's table; they are prepared
        # on every call because the caller's m_indptr and output may change
        tile_class = _tile_m(rows, self.experts, self.hidden_size, self.intermediate_size)
        gemms = []
        with torch.cuda.device(self.device):
            for projection, tile, dtype in (("fc1", tile_class[0], _FP4), ("fc2", tile_class[1], torch.bfloat16)):
                gemm = self._routed_gemms.get((projection, tile))
                if gemm is None:
                    gemm = self._routed_gemms[(projection, tile)] = self._new_gemm(projection, rows, dtype)
                gemms.append(gemm)
        gemms[0](qx, self.qb1, qh, m_indptr, sfx, self.sfb1, self._alpha1, output_sf=sfh,
                 output_scale=self._h_scale)
        gemms[1](qh, self.qb2, routed_out, m_indptr, sfh, self.sfb2, self._alpha2)
        return routed_out

    @torch.no_grad()
    def run_prefill(self, x, topk_ids, topk_weights, *, out=None) -> torch.Tensor:
        self._require_ready()
        tokens = self._validate_full(x, topk_ids, topk_weights)
        rows = tokens * self.topk
        output = self._output_view(out, tokens, "out")
        execution = self._full_execution(tokens, decode=False)
        if rows <= FUSED_PREPARE_MAX_ROWS:
            # a short prefill step (a few rows on few experts) is a handful of launches of a few
            # microseconds each: dispatch and quantization in one
            nvfp4_dispatch_quantize_decode(x, topk_ids, topk_weights, self._parts, self._gather[:rows],
                                           self._m_indptr, self._probs[:rows], self._slots[:rows],
                                           self._padded_offsets, self._x_scale, execution.qx, execution.sfx)
            return self._finish(execution, rows, output)
        self._dispatch(topk_ids, topk_weights, rows)
        # each token is quantized once and its codes and scale factors are written to all of
        # its expert-major rows: same bits as quantizing the gathered rows, 1/top_k of the math
        nvfp4_quantize_decode(x, topk_ids, self._slots[:rows], self._m_indptr, self._padded_offsets,
                              self._x_scale, execution.qx, execution.sfx)
        return self._finish(execution, rows, output)

    @torch.no_grad()
    def run_decode(self, x, topk_ids, topk_weights, *, out=None) -> torch.Tensor:
        """Small-batch step on the decode-shaped kernels."""
        self._require_ready()
        tokens = self._validate_full(x, topk_ids, topk_weights)
        rows = tokens * self.topk
        output = self._output_view(out, tokens, "out")
        if tokens == 1 and self.topk <= 32 and self.tile_override is None:
            # one token: no dispatch, the routes keep their order
            execution = self._direct_execution(topk_ids)
            nvfp4_direct_decode_prepare(x, topk_ids, topk_weights, self._gather[:rows], self._slots[:rows],
                                        self._m_indptr[: self.topk], self._probs[:rows],
                                        self._padded_offsets, self._x_scale, execution.qx, execution.sfx)
            return self._finish(execution, rows, output)
        execution = self._full_execution(tokens, decode=True)
        if rows <= FUSED_PREPARE_MAX_ROWS:
            # one launch: dispatch + decode plan + quantize-once-and-scatter
            nvfp4_dispatch_quantize_decode(x, topk_ids, topk_weights, self._parts, self._gather[:rows],
                                           self._m_indptr, self._probs[:rows], self._slots[:rows],
                                           self._padded_offsets, self._x_scale, execution.qx, execution.sfx)
        else:
            self._dispatch(topk_ids, topk_weights, rows)
            nvfp4_quantize_decode(x, topk_ids, self._slots[:rows], self._m_indptr, self._padded_offsets,
                                  self._x_scale, execution.qx, execution.sfx)
        return self._finish(execution, rows, output, threads=768 if self.hidden_size >= 2048 else 256)

    @torch.no_grad()
    def run(self, x, topk_ids, topk_weights, *, out=None) -> torch.Tensor:
        if x.shape[0] * self.topk <= DECODE_ROWS_PER_EXPERT * self.experts:
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
