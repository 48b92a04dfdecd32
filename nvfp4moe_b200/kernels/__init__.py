"""sm_100a kernels of the NVFP4 routed-expert inference path (host wrappers)."""

from importlib import import_module

_EXPORTS = {
    "DenseNvfp4Gemm": (".dense.runtime", "DenseNvfp4Gemm"),
    "GatedBackwardEpilogue": (".gated", "GatedBackwardEpilogue"),
    "GatedEpilogue": (".gated", "GatedEpilogue"),
    "GroupedNvfp4Gemm": (".grouped.runtime", "GroupedNvfp4Gemm"),
    "MoEDispatch": (".routing.dispatch", "MoEDispatch"),
    "UnaryBackwardEpilogue": (".unary", "UnaryBackwardEpilogue"),
    "UnaryEpilogue": (".unary", "UnaryEpilogue"),
    "grouped_nvfp4_gemm": (".grouped.runtime", "grouped_nvfp4_gemm"),
    "moe_dispatch": (".routing.dispatch", "moe_dispatch"),
    "moe_finalize": (".routing.combine", "moe_finalize"),
    "nvfp4_decode_prepare": (".quantize.decode", "nvfp4_decode_prepare"),
    "nvfp4_direct_decode_prepare": (".quantize.decode", "nvfp4_direct_decode_prepare"),
    "nvfp4_quantize_batched": (".quantize.runtime", "nvfp4_quantize_batched"),
    "nvfp4_quantize_decode": (".quantize.decode", "nvfp4_quantize_decode"),
    "nvfp4_quantize_rowwise": (".quantize.runtime", "nvfp4_quantize_rowwise"),
}
__all__ = sorted(_EXPORTS)


def __getattr__(name):
    try:
        module_name, attr_name = _EXPORTS[name]
    except KeyError as exc:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from exc
    value = getattr(import_module(module_name, __name__), attr_name)
    globals()[name] = value
    return value


def __dir__():
    return sorted((*globals(), *_EXPORTS))
