"""Host runtime of the dense NVFP4 GEMM ``C = alpha * A @ B.T``.

Mirrors ``DenseNvfp4Gemm`` of the reference
(``lightmoe/kernels/dense/runtime.py:54-143``).  The dense GEMM is the grouped
kernel with a single group, so it shares ``lm_gemm_prepare`` / ``lm_gemm_launch``.
"""

from __future__ import annotations

import ctypes

import torch

from ... import _lib, tracing


class DenseNvfp4Gemm:
    """Dense ``C = A @ B.T`` GEMM for prepacked NVFP4 operands."""

    def __init__(self, n: int, k: int, tile_m: int, tile_n: int,
                 output_dtype: torch.dtype = torch.bfloat16):
        if n <= 0 or k <= 0 or k % 64:
            raise ValueError("N and K must be positive and K must be aligned to 64")
        if tile_m not in (128, 256) or tile_n not in (64, 128, 192, 256):
            raise ValueError("dense GEMM supports M tiles 128/256 and N tiles 64/128/192/256")
        if output_dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dense GEMM output must use BF16 or FP32")
        if tile_n in (64, 192):
            raise NotImplementedError("the kernels of this build have 128- and 256-column tiles; "
                                      "tile_n 64 and 192 are not built")
        self.n = n
        self.k = k
        self.tile_m = tile_m
        self.tile_n = tile_n
        self.output_dtype = output_dtype
        self.device = torch.cuda.current_device()
        self._plan = None

    @property
    def stages(self) -> int:
        """Depth of the operand ring of the prepared plan (0 before ``prepare``)."""
        return 0 if self._plan is None else _lib.plan_info(self._plan)["stages"]

    def prepare(self, a, b, out, sfa, sfb, alpha):
        tensors = {"A": a, "B": b, "output": out, "SFA": sfa, "SFB": sfb, "alpha": alpha}
        for name, tensor in tensors.items():
            if not tensor.is_cuda or tensor.device.index != self.device:
                raise ValueError(f"{name} must be on CUDA device {self.device}")
            if not tensor.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        rows = a.shape[0]
        if a.dtype != torch.float4_e2m1fn_x2 or tuple(a.shape) != (rows, self.k // 2):
            raise ValueError(f"A must have packed shape (M, {self.k // 2})")
        if b.dtype != torch.float4_e2m1fn_x2 or tuple(b.shape) != (self.n, self.k // 2):
            raise ValueError(f"B must have packed shape ({self.n}, {self.k // 2})")
        if out.dtype != self.output_dtype or tuple(out.shape) != (rows, self.n):
            raise ValueError(f"output must have shape ({rows}, {self.n})")
        expected_sfa = (-(-rows // 128), self.k // 64, 32, 4, 4)
        expected_sfb = (-(-self.n // 128), self.k // 64, 32, 4, 4)
        if sfa.dtype != torch.float8_e4m3fn or tuple(sfa.shape) != expected_sfa:
            raise ValueError(f"SFA must have shape {expected_sfa}")
        if sfb.dtype != torch.float8_e4m3fn or tuple(sfb.shape) != expected_sfb:
            raise ValueError(f"SFB must have shape {expected_sfb}")
        if alpha.dtype != torch.float32 or tuple(alpha.shape) != (1,):
            raise ValueError("alpha must be float32 with shape (1,)")
        args = _lib.GemmArgs()
        args.experts = 1
        args.n = self.n
        args.k = self.k
        args.tile_m = self.tile_m
        args.tile_n = self.tile_n
        args.out_kind = _lib.OUT_BF16 if self.output_dtype == torch.bfloat16 else _lib.OUT_F32
        args.activation = 0
        args.sigmoid_alpha = 1.0
        args.dense = 1
        args.sf_tile_rows = 128
        args.rows = rows
        args.a = a.data_ptr()
        args.b = b.data_ptr()
        args.out = out.data_ptr()
        args.m_indptr = None
        args.sfa = sfa.data_ptr()
        args.sfb = sfb.data_ptr()
        args.alpha = alpha.data_ptr()
        plan = _lib.GemmPlan()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lm_gemm_prepare(ctypes.byref(args), ctypes.byref(plan)))
        self._plan = plan
        self._inputs = (a, b, out, sfa, sfb, alpha)

    def launch(self):
        if self._plan is None:
            raise RuntimeError("prepare must run before launch")
        opened = tracing.push("lightmoe.dense_gemm")
        try:
            with torch.cuda.device(self.device):  # the plan belongs to this device's context and stream
                _lib.check(_lib.lib().lm_gemm_launch(ctypes.byref(self._plan), _lib.stream_handle()))
        finally:
            tracing.pop(opened)

    def __call__(self, a, b, out, sfa, sfb, alpha):
        self.prepare(a, b, out, sfa, sfb, alpha)
        self.launch()

    run = __call__


__all__ = ["DenseNvfp4Gemm"]
