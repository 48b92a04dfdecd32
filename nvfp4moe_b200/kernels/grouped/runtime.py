"""Host runtime of the grouped NVFP4 GEMM.

Mirrors ``GroupedNvfp4Gemm`` of the reference
(``lightmoe/kernels/grouped/runtime.py:178-624``): same constructor and
``prepare`` / ``launch`` / ``run`` signatures, same validation rules and
messages.  ``prepare`` encodes the TMA descriptors once through
``lm_gemm_prepare``; ``launch`` is a single ``lm_gemm_launch`` call on the
current stream and is safe inside CUDA Graph capture.
"""

from __future__ import annotations

import ctypes

import torch

from ... import _lib, tracing
from ..gated import GatedBackwardEpilogue, GatedEpilogue, resolve_gemm_epilogue
from ..unary import UnaryBackwardEpilogue, UnaryEpilogue

DECODE_GRID_PERSISTENT = 0
DECODE_GRID_DOUBLE = 1


def _resolve_dynamic_schedule(use_dynamic_sched: bool | None, k: int) -> bool:
    """Scheduling policy flag of the reference (``runtime.py:22-25``): a performance hint.

    The kernels here deal their units statically (round-robin, or equal contiguous shares in
    the decode-shaped kernel); the flag is resolved and kept because callers read it back and
    because ``fast_decode_sched`` is validated against it.
    """
    if use_dynamic_sched is None:
        return k > 2048
    return bool(use_dynamic_sched)


def _decode_grid_mode(gather_b: bool, k: int, n: int, rows: int, experts: int) -> int:
    """Grid policy table of the reference (``runtime.py:28-35``)."""
    if not gather_b or rows <= 1:
        return DECODE_GRID_PERSISTENT
    if k >= 4096 and n >= 4096 and rows <= (64 if experts >= 48 else 16):
        return DECODE_GRID_DOUBLE
    if k >= 3072 and n == 3072 and rows <= 32:
        return DECODE_GRID_DOUBLE
    return DECODE_GRID_PERSISTENT


def _out_kind(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return _lib.OUT_BF16
    if dtype == torch.float32:
        return _lib.OUT_F32
    return _lib.OUT_NVFP4


class GroupedNvfp4Gemm:
    """Grouped NVFP4 GEMM for contiguous expert-major assignments.

    What the decode options of the reference's constructor select here:

    ``swap_ab``            the decode-shaped kernel: the expert's weights take the 128-row side
                           of the MMA and its few rows the 8..64-column side; ``tile_m`` /
                           ``tile_n`` then only pass validation.  Results are bit-identical to
                           the other tilings.
    ``direct_routes``      (with or without ``swap_ab``) the routes of one token without a
                           dispatch, on the same kernel: ``cu`` holds the expert id of each
                           route, route r reads row r of A (row 0 with ``broadcast_a``) and
                           writes row r of the output.
    ``use_pdl``            the launch is a programmatic dependent of the previous kernel: its
                           set-up runs beside that kernel and it waits for it before reading
                           operands.  Pays in steps of a few short launches; on a long prefill
                           chain it measured slower (``InferenceMoE`` asks for it accordingly).  ``weights_ahead`` (attribute, set before ``prepare``)
                           lets it start its weight stream before the previous kernel ends.
    ``fast_decode_sched``  a scheduling hint of the reference (tiles read from the dispatch
                           plan); every kernel here derives its tiles from ``cu`` on the device,
                           so the flag changes nothing and is only validated.
    ``gather_b``           refused: the quantizers of this build write rows expert-major, there
                           is no token-major buffer to gather from.
    """

    def __init__(
        self,
        experts: int,
        n: int,
        k: int,
        tile_m: int,
        tile_n: int,
        output_dtype: torch.dtype = torch.bfloat16,
        activation: str | None = None,
        dactivation: str | None = None,
        epilogue=None,
        use_dynamic_sched: bool | None = None,
        use_pdl: bool = False,
        swap_ab: bool = False,
        fast_decode_sched: bool = False,
        direct_routes: int = 0,
        broadcast_a: bool = False,
        gather_b: bool = False,
    ):
        activation, dactivation = resolve_gemm_epilogue(epilogue, activation, dactivation)
        if epilogue is None and activation is not None:
            epilogue = UnaryEpilogue(activation) if activation == "relu2" else GatedEpilogue(activation)
        gated_policy = isinstance(epilogue, (GatedEpilogue, GatedBackwardEpilogue))
        save_preact = isinstance(epilogue, (GatedEpilogue, UnaryEpilogue)) and epilogue.save_preact
        self.gated_clamp_limit = float(epilogue.clamp_limit or 0.0) if gated_policy else 0.0
        self.activation_sigmoid_alpha = epilogue.sigmoid_alpha if gated_policy else 1.0
        self.activation_up_bias = epilogue.up_bias if gated_policy else 0.0

        fp4 = torch.float4_e2m1fn_x2
        known = (None, "swiglu", "swiglu_oai", "geglu", "reglu", "relu2")
        gated = activation is not None and activation != "relu2"
        # (failed, exception, message) in the order the reference checks them
        # (lightmoe/kernels/grouped/runtime.py:226-290): its callers and tests meet the first
        # message that applies
        rules = (
            (experts <= 0 or n <= 0 or k <= 0, ValueError, "experts, N, and K must be positive"),
            (experts > 256, ValueError, "grouped GEMM supports at most 256 local experts"),
            (k % 64, ValueError, "grouped GEMM requires K aligned to 64"),
            (tile_m not in (128, 256) or not 8 <= tile_n <= 256 or tile_n % 8, ValueError,
             "grouped GEMM supports M=128/256 and N=8..256 aligned to 8"),
            (output_dtype not in (torch.bfloat16, torch.float32, torch.int32, fp4), ValueError,
             "grouped GEMM output must be BF16, FP32, Int32, or NVFP4"),
            (activation not in known, ValueError, "unsupported grouped GEMM activation"),
            (dactivation not in known, ValueError, "unsupported grouped GEMM derivative"),
            (activation is not None and dactivation is not None, ValueError,
             "activation and dactivation are mutually exclusive"),
            (dactivation is not None or save_preact or output_dtype == torch.int32, NotImplementedError,
             "backward epilogues belong to the training path"),
            (output_dtype == fp4 and activation is None, ValueError, "NVFP4 output requires an activation epilogue"),
            (output_dtype == fp4 and n % 128, ValueError, "gated NVFP4 output requires N aligned to 128"),
            (activation is not None and output_dtype != fp4, NotImplementedError,
             "activation epilogues write NVFP4 in the inference path"),
            (gated and (n % 2 or (tile_m if swap_ab else tile_n) % 128), ValueError,
             f"gated GEMM requires even N and {'tile_M' if swap_ab else 'tile_N'} aligned to 128"),
            (swap_ab and activation is not None and tile_n > 64, ValueError,
             "operand-swapped activation GEMM requires tile_N at most 64"),
        )
        for failed, error, message in rules:
            if failed:
                raise error(message)
        self.experts, self.n, self.k = experts, n, k
        self.tile_m, self.tile_n = tile_m, tile_n
        self.output_dtype = output_dtype
        self.activation, self.dactivation = activation, dactivation
        self.save_preact = save_preact
        self.epilogue = epilogue
        self.use_dynamic_sched = _resolve_dynamic_schedule(use_dynamic_sched, k)
        self.use_pdl = bool(use_pdl)
        self.swap_ab = bool(swap_ab)
        self.fast_decode_sched = bool(fast_decode_sched)
        self.direct_routes = int(direct_routes)
        self.broadcast_a = bool(broadcast_a)
        self.gather_b = bool(gather_b)
        self._direct_c_store = False
        if self.fast_decode_sched and self.use_dynamic_sched:
            raise ValueError("fast decode scheduling requires a static GEMM")
        if self.direct_routes < 0 or self.direct_routes > 32:
            raise ValueError("direct route count must be between 0 and 32")
        if self.broadcast_a and not self.direct_routes:
            raise ValueError("broadcast A requires direct routing")
        if self.gather_b and not (self.swap_ab and self.fast_decode_sched):
            raise ValueError("gather B requires swapped fast decode")
        if self.gather_b:
            raise NotImplementedError(
                "gather_b: the quantizers of this build write rows expert-major, there is no "
                "token-major buffer to gather from")
        self.output_n = n
        if gated:
            self.output_n = n // 2
        self.device = torch.cuda.current_device()
        self.max_ctas = 0  # 0 = one CTA per SM; tests lower it to run many tiles per CTA
        # decode-shaped kernel with use_pdl: start the weight stream before the previous kernel
        # in the stream has finished.  Only for a second projection that directly follows its
        # first projection (cu, B, SFB and alpha are older than that kernel).
        self.weights_ahead = False
        self.trace_name = "lightmoe.grouped_gemm"  # NVTX range of a launch (nvfp4moe_b200.tracing)
        # Set before ``prepare``: int64 CUDA tensor with one 16-byte aligned address per row.
        # Every BF16 output row is then written to its own address (which may lie in a peer
        # GPU's memory) instead of ``out``; the expert-parallel layer returns rows to their
        # source ranks this way.
        self.output_row_ptrs = None
        # With ``output_row_ptrs``: whole 32-row blocks that the route plan's block table
        # (``lm_ep_plan``) assigns to one rank leave as one bulk store into that rank's return
        # buffer.  ``output_blocks`` = the int32 table, ``return_bases`` = a ctypes uint64 array of
        # the ranks' return buffers, ``return_rows`` = rows of each of them.
        self.output_blocks = None
        self.return_bases = None
        self.return_rows = 0
        self._plan = None

    def prepare(
        self,
        a,
        b,
        out,
        cu,
        sfa,
        sfb,
        alpha,
        output_sf=None,
        output_scale=None,
        preact=None,
        aux=None,
        decode_plan=None,
        gather_idx=None,
    ):
        tensors = {"A": a, "B": b, "output": out, "cu": cu, "SFA": sfa, "SFB": sfb, "alpha": alpha}
        for name, tensor in tensors.items():
            if not tensor.is_cuda or tensor.device.index != self.device:
                raise ValueError(f"{name} must be on CUDA device {self.device}")
            if not tensor.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        if a.dtype != torch.float4_e2m1fn_x2 or a.ndim != 2 or a.shape[1] * 2 != self.k:
            raise ValueError(f"A must have packed shape (M, {self.k // 2})")
        if b.dtype != torch.float4_e2m1fn_x2 or tuple(b.shape) != (self.experts, self.n, self.k // 2):
            raise ValueError("B does not match the compiled expert geometry")
        rows = a.shape[0]
        nvfp4_out = self.output_dtype == torch.float4_e2m1fn_x2
        output_cols = self.output_n // 2 if nvfp4_out else self.output_n
        if tuple(out.shape) != (rows, output_cols) or out.dtype != self.output_dtype:
            raise ValueError(
                f"output must use {self.output_dtype} with shape ({rows}, {output_cols})"
            )
        cu_shape = (self.direct_routes,) if self.direct_routes else (self.experts + 1,)
        if cu.dtype != torch.int32 or tuple(cu.shape) != cu_shape:
            raise ValueError(f"routing metadata must be contiguous int32 with shape {cu_shape}")
        if self.direct_routes and rows != self.direct_routes:
            raise ValueError("direct routing takes one row per route")
        expected_sfa = (1, -(-rows // 128) + self.experts, self.k // 64, 32, 4, 4)
        expected_sfb = (self.experts, -(-self.n // 128), self.k // 64, 32, 4, 4)
        if sfa.dtype != torch.float8_e4m3fn or tuple(sfa.shape) != expected_sfa:
            raise ValueError(f"SFA must have shape {expected_sfa}")
        if sfb.dtype != torch.float8_e4m3fn or tuple(sfb.shape) != expected_sfb:
            raise ValueError(f"SFB must have shape {expected_sfb}")
        if alpha.dtype != torch.float32 or tuple(alpha.shape) not in ((1,), (self.experts,)):
            raise ValueError(
                f"alpha must be contiguous float32 with shape (1,) or ({self.experts},)"
            )
        if nvfp4_out:
            expected_output_sf = (1, -(-rows // 128) + self.experts, self.output_n // 64, 32, 4, 4)
            if (
                output_sf is None
                or not output_sf.is_cuda
                or output_sf.dtype != torch.float8_e4m3fn
                or tuple(output_sf.shape) != expected_output_sf
                or not output_sf.is_contiguous()
                or output_sf.device.index != self.device
            ):
                raise ValueError(f"output_sf must have shape {expected_output_sf}")
            if (
                output_scale is None
                or not output_scale.is_cuda
                or output_scale.dtype != torch.float32
                or tuple(output_scale.shape) != (2,)
                or not output_scale.is_contiguous()
                or output_scale.device.index != self.device
            ):
                raise ValueError("output_scale must be contiguous float32 [pts, inv_pts]")
        args = _lib.GemmArgs()
        args.experts = self.experts
        args.n = self.n
        args.k = self.k
        args.tile_m = self.tile_m
        args.tile_n = self.tile_n
        args.out_kind = _out_kind(self.output_dtype)
        args.activation = _lib.ACTIVATIONS[self.activation]
        args.clamp_limit = self.gated_clamp_limit
        args.sigmoid_alpha = self.activation_sigmoid_alpha
        args.up_bias = self.activation_up_bias
        args.alpha_per_expert = int(alpha.shape[0] == self.experts and self.experts > 1)
        args.dense = 0
        args.sf_tile_rows = 128
        args.max_ctas = int(self.max_ctas)
        args.rows = rows
        args.a = a.data_ptr()
        args.b = b.data_ptr()
        args.out = out.data_ptr()
        args.m_indptr = cu.data_ptr()
        args.sfa = sfa.data_ptr()
        args.sfb = sfb.data_ptr()
        args.alpha = alpha.data_ptr()
        args.out_sf = output_sf.data_ptr() if nvfp4_out else None
        args.out_scale = output_scale.data_ptr() if nvfp4_out else None
        output_row_ptrs = self.output_row_ptrs
        if output_row_ptrs is not None:
            if self.output_dtype != torch.bfloat16:
                raise ValueError("output_row_ptrs requires BF16 output")
            if (not output_row_ptrs.is_cuda or output_row_ptrs.dtype != torch.int64
                    or output_row_ptrs.ndim != 1 or output_row_ptrs.shape[0] < rows
                    or not output_row_ptrs.is_contiguous()):
                raise ValueError(f"output_row_ptrs must be a contiguous int64 CUDA tensor of {rows} addresses")
            args.out_row_ptrs = output_row_ptrs.data_ptr()
            if self.output_blocks is not None and not (self.swap_ab or self.direct_routes):
                blocks = self.output_blocks
                need = (rows // 128 + self.experts) * 4 * 2
                if (not blocks.is_cuda or blocks.dtype != torch.int32 or blocks.numel() < need
                        or not blocks.is_contiguous() or self.return_bases is None or self.return_rows <= 0):
                    raise ValueError(f"output_blocks must be a contiguous int32 CUDA tensor of {need} entries "
                                     "with return_bases and return_rows set")
                args.out_blocks = blocks.data_ptr()
                args.return_bases = ctypes.cast(self.return_bases, ctypes.POINTER(ctypes.c_uint64))
                args.return_world = len(self.return_bases)
                args.return_rows = int(self.return_rows)
        decode_shaped = self.swap_ab or self.direct_routes > 0
        args.swap_ab = int(decode_shaped)
        args.direct_routes = self.direct_routes
        args.broadcast_a = int(self.broadcast_a)
        args.use_pdl = int(self.use_pdl)
        args.weights_ahead = int(self.weights_ahead and self.use_pdl and decode_shaped)
        plan = _lib.GemmPlan()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lm_gemm_prepare(ctypes.byref(args), ctypes.byref(plan)))
        self._plan = plan
        # keep operands alive for as long as the plan may launch
        self._keepalive = (a, b, out, cu, sfa, sfb, alpha, output_sf, output_scale, output_row_ptrs,
                           self.output_blocks, self.return_bases)

    @property
    def stages(self) -> int:
        """Depth of the operand ring of the prepared plan (0 before ``prepare``)."""
        return 0 if self._plan is None else _lib.plan_info(self._plan)["stages"]

    def launch(self):
        if self._plan is None:
            raise RuntimeError("prepare must run before launch")
        opened = tracing.push(self.trace_name)
        try:
            with torch.cuda.device(self.device):  # the plan belongs to this device's context and stream
                _lib.check(_lib.lib().lm_gemm_launch(ctypes.byref(self._plan), _lib.stream_handle()))
        finally:
            tracing.pop(opened)

    def __call__(self, a, b, out, cu, sfa, sfb, alpha, output_sf=None, output_scale=None,
                 preact=None, aux=None, decode_plan=None, gather_idx=None):
        self.prepare(a, b, out, cu, sfa, sfb, alpha, output_sf, output_scale, preact, aux,
                     decode_plan, gather_idx)
        self.launch()

    run = __call__


def grouped_nvfp4_gemm(experts, n, k, tile_m, tile_n, output_dtype=torch.bfloat16, activation=None,
                       dactivation=None, epilogue=None, use_dynamic_sched=None, use_pdl=False,
                       swap_ab=False, fast_decode_sched=False, direct_routes=0, broadcast_a=False):
    return GroupedNvfp4Gemm(experts, n, k, tile_m, tile_n, output_dtype, activation, dactivation,
                            epilogue, use_dynamic_sched, use_pdl, swap_ab, fast_decode_sched,
                            direct_routes, broadcast_a)


__all__ = ["GroupedNvfp4Gemm", "grouped_nvfp4_gemm"]
