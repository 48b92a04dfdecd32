"""ctypes binding of ``liblightmoe_b200.so`` (the C-ABI in ``include/lightmoe_b200.h``).

There is no fallback: if the shared library is missing or fails to load, every
kernel entry point raises.
"""

from __future__ import annotations

import ctypes
import pathlib

import torch

_LIB_PATH = pathlib.Path(__file__).resolve().parent / "liblightmoe_b200.so"
_lib = None

c_i32 = ctypes.c_int32
c_i64 = ctypes.c_int64
c_ptr = ctypes.c_void_p
c_f32 = ctypes.c_float

SF_VARLEN, SF_BATCHED, SF_LINEAR = 0, 1, 2
OUT_BF16, OUT_F32, OUT_NVFP4 = 0, 1, 2
ACTIVATIONS = {None: 0, "swiglu": 1, "swiglu_oai": 2, "geglu": 3, "reglu": 4, "relu2": 5}


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("experts", c_i32),
        ("n", c_i32),
        ("k", c_i32),
        ("tile_m", c_i32),
        ("tile_n", c_i32),
        ("out_kind", c_i32),
        ("activation", c_i32),
        ("clamp_limit", c_f32),
        ("sigmoid_alpha", c_f32),
        ("up_bias", c_f32),
        ("alpha_per_expert", c_i32),
        ("dense", c_i32),
        ("sf_tile_rows", c_i32),
        ("max_ctas", c_i32),
        ("rows", c_i64),
        ("a", c_ptr),
        ("b", c_ptr),
        ("out", c_ptr),
        ("m_indptr", c_ptr),
        ("sfa", c_ptr),
        ("sfb", c_ptr),
        ("alpha", c_ptr),
        ("out_sf", c_ptr),
        ("out_scale", c_ptr),
        ("out_row_ptrs", c_ptr),
        ("swap_ab", c_i32),
        ("direct_routes", c_i32),
        ("broadcast_a", c_i32),
        ("use_pdl", c_i32),
        ("weights_ahead", c_i32),
        ("out_blocks", c_ptr),
        ("return_bases", ctypes.POINTER(ctypes.c_uint64)),
        ("return_world", c_i32),
        ("return_rows", c_i64),
    ]


class GemmPlan(ctypes.Structure):
    _fields_ = [("opaque", ctypes.c_uint64 * 320)]


_SIGNATURES = {
    "lm_version": (c_i32, []),
    "lm_last_error_string": (ctypes.c_char_p, []),
    "lm_sm_count": (c_i32, [ctypes.POINTER(c_i32)]),
    "lm_launch_count": (ctypes.c_uint64, []),
    "lm_device_status": (c_i32, [ctypes.POINTER(ctypes.c_uint32), c_ptr]),
    "lm_device_status_clear": (c_i32, [c_ptr]),
    "lm_quantize_rowwise": (
        c_i32,
        [c_ptr, c_i32, c_i64, c_i32, c_ptr, c_i32, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_i32, c_i32, c_ptr],
    ),
    "lm_quantize_decode": (
        c_i32,
        [c_ptr, c_i64, c_i32, c_i32, c_ptr, c_ptr, c_ptr, c_i32, c_ptr, c_ptr, c_ptr, c_ptr],
    ),
    "lm_activation_amax": (c_i32, [c_ptr, c_i64, c_i32, c_i32, c_f32, c_f32, c_f32, c_ptr, c_ptr]),
    "lm_route_topk": (c_i32, [c_ptr, c_i32, c_i64, c_i32, c_i32, c_ptr, c_ptr, c_ptr]),
    "lm_ep_plan": (
        c_i32,
        [c_ptr, c_i32, c_i32, c_i32, c_i64, c_i64, ctypes.POINTER(ctypes.c_uint64), c_ptr, c_ptr, c_ptr,
         c_ptr, c_ptr, c_ptr, c_ptr],
    ),
    "lm_ep_quantize_send": (
        c_i32,
        [c_ptr, c_i64, c_i32, c_i32, c_i32, c_i32, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
         ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64), c_ptr],
    ),
    "lm_ep_signal": (
        c_i32,
        [c_ptr, c_i32, c_i32, c_i32, ctypes.POINTER(ctypes.c_uint64),
         ctypes.POINTER(ctypes.c_uint64), c_i32, c_ptr],
    ),
    "lm_ep_sf_swizzle": (c_i32, [c_ptr, c_i64, c_i32, c_ptr, c_i32, c_ptr, c_ptr]),
    "lm_dispatch_scratch_elems": (c_i64, [c_i64, c_i32]),
    "lm_dispatch": (
        c_i32,
        [c_ptr, c_ptr, c_i64, c_i32, c_i32, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i32, c_ptr],
    ),
    "lm_dispatch_quantize_decode": (
        c_i32,
        [c_ptr, c_ptr, c_ptr, c_i64, c_i32, c_i32, c_i32, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
         c_i64, c_i32, c_ptr, c_ptr, c_ptr, c_ptr],
    ),
    "lm_decode_prepare": (
        c_i32,
        [c_ptr, c_ptr, c_ptr, c_i32, c_i32, c_i32, c_i32, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
         c_ptr],
    ),
    "lm_dispatch_static_max_rows": (c_i64, []),
    "lm_dispatch_static": (
        c_i32,
        [c_ptr, c_ptr, c_i64, c_i32, c_i32, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i32, c_ptr],
    ),
    "lm_finalize": (c_i32, [c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i32, c_i32, c_i64, c_i64, c_ptr, c_i32, c_ptr]),
    "lm_gemm_prepare": (c_i32, [ctypes.POINTER(GemmArgs), ctypes.POINTER(GemmPlan)]),
    "lm_gemm_launch": (c_i32, [ctypes.POINTER(GemmPlan), c_ptr]),
    "lm_gemm_plan_info": (c_i32, [ctypes.POINTER(GemmPlan), ctypes.POINTER(c_i32), ctypes.POINTER(c_i32),
                                  ctypes.POINTER(c_i32)]),
}


def exported_symbols() -> tuple[str, ...]:
    return tuple(_SIGNATURES)


def library_path() -> pathlib.Path:
    return _LIB_PATH


def lib():
    """Load the shared library once; raise if it is not built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m nvfp4moe_b200.build` "
                "(there is no CPU or PyTorch fallback)"
            )
        handle = ctypes.CDLL(str(_LIB_PATH))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        message = lib().lm_last_error_string().decode("utf-8", "replace")
        if status == 1:
            raise ValueError(message)
        raise RuntimeError(message)


def ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def stream_handle() -> int:
    return torch.cuda.current_stream().cuda_stream


def sm_count() -> int:
    out = c_i32(0)
    check(lib().lm_sm_count(ctypes.byref(out)))
    return out.value


def device_status() -> int:
    out = ctypes.c_uint32(0)
    check(lib().lm_device_status(ctypes.byref(out), stream_handle()))
    return out.value


def device_status_clear() -> None:
    check(lib().lm_device_status_clear(stream_handle()))


def launch_count() -> int:
    """Kernel launches made through the library so far in this process."""
    return int(lib().lm_launch_count())


KERNEL_NAMES = ("128x128 tiles", "128x256 tiles", "256x256 tiles on CTA pairs", "decode-shaped")


def plan_info(plan: GemmPlan) -> dict:
    """Kernel, grid and ring depth a prepared GEMM plan launches with."""
    kernel, grid, ring = c_i32(0), c_i32(0), c_i32(0)
    check(lib().lm_gemm_plan_info(ctypes.byref(plan), ctypes.byref(kernel), ctypes.byref(grid), ctypes.byref(ring)))
    return {"kernel": KERNEL_NAMES[kernel.value], "grid": grid.value, "stages": ring.value}
