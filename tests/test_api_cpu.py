"""CPU checks: the C-ABI library exports what the header declares, and the
Python surface keeps the reference's names, defaults, policies and messages
(``tests/test_imports.py``, ``tests/test_gemm_api.py``,
``tests/test_gated_epilogue.py``, ``tests/test_unary_epilogue.py`` and the
policy tables of ``tests/test_inference.py:107-114,295-323`` of the reference).
"""

import ctypes
import inspect
import pathlib
import re
import subprocess
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _header_symbols():
    text = (ROOT / "include" / "lightmoe_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from nvfp4moe_b200 import _lib
    from nvfp4moe_b200.build import build

    build()
    names = _header_symbols()
    assert len(names) >= 12
    handle = ctypes.CDLL(str(_lib.library_path()))
    for name in names:
        assert getattr(handle, name) is not None, name
    assert sorted(_lib.exported_symbols()) == names
    assert _lib.lib().lm_version() >= 1


def test_host_side_argument_checks_need_no_gpu():
    from nvfp4moe_b200 import _lib

    lib = _lib.lib()
    assert lib.lm_quantize_rowwise(None, 0, 1, 64, None, 1, 0, None, None, None, None, 0, 0, None) == 1
    assert b"null pointer" in lib.lm_last_error_string()
    assert lib.lm_dispatch_scratch_elems(1000, 8) == 128 * 8
    assert lib.lm_dispatch_scratch_elems(196608, 256) == 192 * 256
    plan = _lib.GemmPlan()
    assert lib.lm_gemm_launch(ctypes.byref(plan), None) == 1
    assert b"not prepared" in lib.lm_last_error_string()
    args = _lib.GemmArgs()
    args.experts, args.n, args.k, args.rows = 1, 128, 100, 5
    assert lib.lm_gemm_prepare(ctypes.byref(args), ctypes.byref(plan)) == 1
    assert b"multiple of 64" in lib.lm_last_error_string()


def test_public_exports_and_aliases():
    import lightmoe
    import nvfp4moe_b200
    from lightmoe import gemm
    from lightmoe.gemm import DenseGemm, GroupedGemm
    from lightmoe.inference import InferenceMoE
    from lightmoe.kernels.dense.runtime import DenseNvfp4Gemm
    from lightmoe.kernels.grouped.runtime import GroupedNvfp4Gemm
    from lightmoe.kernels.routing.dispatch import MoEDispatch
    from lightmoe.training import MoEExpertLayer

    assert lightmoe is nvfp4moe_b200
    assert lightmoe.InferenceMoE is InferenceMoE
    assert lightmoe.MoEExpertLayer is MoEExpertLayer
    assert lightmoe.MoEDispatch is MoEDispatch
    assert lightmoe.__all__ == ["InferenceMoE", "MoEDispatch", "MoEExpertLayer"]
    assert gemm.__all__ == ["DenseGemm", "GroupedGemm", "quantize", "quantize_grouped"]
    assert DenseGemm is DenseNvfp4Gemm and GroupedGemm is GroupedNvfp4Gemm
    assert DenseGemm.run is DenseGemm.__call__
    assert GroupedGemm.run is GroupedGemm.__call__


def test_constructor_names():
    from lightmoe import InferenceMoE, MoEDispatch, MoEExpertLayer
    from lightmoe.gemm import GroupedGemm

    assert tuple(inspect.signature(InferenceMoE).parameters)[:5] == (
        "hidden_size", "intermediate_size", "num_experts", "top_k", "max_tokens")
    assert tuple(inspect.signature(MoEDispatch).parameters)[:3] == (
        "num_tokens", "num_experts", "top_k")
    assert tuple(inspect.signature(MoEExpertLayer).parameters)[:4] == (
        "hidden_size", "intermediate_size", "num_experts", "top_k")
    assert tuple(inspect.signature(InferenceMoE.load_packed_weights).parameters)[1:7] == (
        "gate_up", "gate_up_sf", "gate_up_scale", "down", "down_sf", "down_scale")
    assert tuple(inspect.signature(GroupedGemm).parameters) == (
        "experts", "n", "k", "tile_m", "tile_n", "output_dtype", "activation", "dactivation",
        "epilogue", "use_dynamic_sched", "use_pdl", "swap_ab", "fast_decode_sched",
        "direct_routes", "broadcast_a", "gather_b")
    assert tuple(inspect.signature(GroupedGemm.prepare).parameters)[1:] == (
        "a", "b", "out", "cu", "sfa", "sfb", "alpha", "output_sf", "output_scale", "preact",
        "aux", "decode_plan", "gather_idx")


def test_policy_tables():
    from lightmoe.inference import _decode_tile_rows, _tile_m, _use_swapped_fc2
    from lightmoe.kernels.grouped.kernel import DECODE_GRID_DOUBLE, DECODE_GRID_PERSISTENT
    from lightmoe.kernels.grouped.runtime import _decode_grid_mode, _resolve_dynamic_schedule

    assert not _resolve_dynamic_schedule(None, 2048)
    assert _resolve_dynamic_schedule(None, 4096)
    assert _resolve_dynamic_schedule(True, 2048)
    assert not _resolve_dynamic_schedule(False, 4096)
    assert _tile_m(8 * 128, 128, 2048, 768) == (128, 128)
    assert _tile_m(256 * 128, 128, 2048, 768) == (256, 128)
    assert _tile_m(256 * 32, 32, 7168, 2048) == (256, 256)
    assert _use_swapped_fc2(8) and not _use_swapped_fc2(9)
    assert _decode_tile_rows(16, 7168, 2048, 48) == 16
    assert _decode_tile_rows(64, 7168, 2048, 48) == 32
    assert _decode_tile_rows(8, 7168, 2048, 48) == 8
    assert _decode_tile_rows(32, 7168, 2048, 32) == 8
    assert _decode_tile_rows(32, 4096, 1536, 128) == 8
    assert _decode_grid_mode(True, 6144, 6144, 1, 128) == DECODE_GRID_PERSISTENT
    assert _decode_grid_mode(True, 4096, 4096, 1, 256) == DECODE_GRID_PERSISTENT
    assert _decode_grid_mode(True, 6144, 6144, 8, 128) == DECODE_GRID_DOUBLE


def test_measured_tile_policy():
    """The tiles this build launches (``policy.pick_tiles``): wide tiles whenever N is two or more
    128-column blocks, CTA pairs when padding every expert to 256 rows costs less than the pair
    wins."""
    from nvfp4moe_b200.policy import (FUSED_PREPARE_MAX_ROWS, SWAPPED_MAX_ROWS, expected_padded_rows,
                                      pick_tiles)

    # N must be two or more whole 128-column blocks for the wide tile; an odd count is fine
    # (Nemotron's 1920 / 2688: the last tile is half empty)
    assert pick_tiles(49152, 8, 136, 2688, nvfp4_out=False) == (128, 128)
    assert pick_tiles(49152, 8, 128, 2688, nvfp4_out=False) == (128, 128)
    assert pick_tiles(49152, 8, 1920, 2688, nvfp4_out=True) == (256, 256)
    assert pick_tiles(512, 8, 2688, 1920, nvfp4_out=False) == (128, 256)
    # fewer than 128 rows per expert: never the tall tile
    assert pick_tiles(1024, 16, 1024, 2048, nvfp4_out=True) == (128, 256)
    # C2: 256 rows per expert pad to 2.5 tiles of 128 or to 3 x 128 in tall tiles: stays on 128 x 256
    assert pick_tiles(65536, 256, 1024, 2048, nvfp4_out=True) == (128, 256)
    assert pick_tiles(65536, 256, 2048, 512, nvfp4_out=False) == (128, 256)
    # C3 (192 rows per expert), C5 and the published shards (thousands of rows per expert): pairs
    assert pick_tiles(49152, 256, 4096, 4096, nvfp4_out=True) == (256, 256)
    assert pick_tiles(65536, 16, 1024, 2048, nvfp4_out=True) == (256, 256)
    assert pick_tiles(49152, 8, 4096, 2048, nvfp4_out=False) == (256, 256)
    # padded rows: a tile boundary in the middle of the distribution costs half a tile on average
    assert abs(expected_padded_rows(256.0, 128) - 320.0) < 8.0
    assert abs(expected_padded_rows(256.0, 256) - 384.0) < 8.0
    assert expected_padded_rows(4096.0, 256) < 4096.0 + 256.0 + 1.0
    assert SWAPPED_MAX_ROWS == 128 and FUSED_PREPARE_MAX_ROWS == 1024


def test_epilogue_policies():
    from lightmoe.kernels.gated import (GatedBackwardEpilogue, GatedEpilogue, gated_output_n,
                                        resolve_gemm_epilogue, validate_gated_tile_n)
    from lightmoe.kernels.unary import UnaryBackwardEpilogue, UnaryEpilogue

    assert GatedEpilogue("swiglu").activation == "swiglu"
    assert GatedEpilogue("swiglu", save_preact=True).save_preact
    assert GatedBackwardEpilogue("geglu").activation == "geglu"
    with pytest.raises(ValueError, match="activation must be one of"):
        GatedEpilogue("gelu")
    assert GatedEpilogue("swiglu", clamp_limit=10).clamp_limit == 10.0
    with pytest.raises(ValueError, match="finite and positive"):
        GatedEpilogue("swiglu", clamp_limit=0)
    with pytest.raises(ValueError, match="only for SwiGLU"):
        GatedEpilogue("geglu", clamp_limit=10)
    oai = GatedEpilogue("swiglu_oai")
    assert (oai.clamp_limit, oai.sigmoid_alpha, oai.up_bias) == (7.0, 1.702, 1.0)
    back = GatedBackwardEpilogue("swiglu_oai", clamp_limit=7, sigmoid_alpha=1.702, up_bias=1)
    assert back.sigmoid_alpha == 1.702 and back.up_bias == 1.0
    with pytest.raises(ValueError, match="require swiglu_oai"):
        GatedEpilogue("swiglu", sigmoid_alpha=1.702)
    assert resolve_gemm_epilogue(GatedEpilogue("geglu"), None, None) == ("geglu", None)
    assert resolve_gemm_epilogue(GatedBackwardEpilogue("reglu"), None, None) == (None, "reglu")
    assert resolve_gemm_epilogue(UnaryEpilogue(), None, None) == ("relu2", None)
    assert resolve_gemm_epilogue(UnaryBackwardEpilogue(), None, None) == (None, "relu2")
    with pytest.raises(ValueError, match="cannot be combined"):
        resolve_gemm_epilogue(GatedEpilogue(), "swiglu", None)
    with pytest.raises(ValueError, match="must be relu2"):
        UnaryEpilogue("gelu")
    assert gated_output_n(256) == 128
    with pytest.raises(ValueError):
        gated_output_n(3)
    with pytest.raises(ValueError):
        validate_gated_tile_n(64)


def test_cpu_inputs_are_rejected_before_any_launch():
    from lightmoe.gemm import quantize, quantize_grouped

    with pytest.raises(ValueError, match="contiguous CUDA matrix"):
        quantize(torch.empty(8, 64, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="contiguous CUDA matrix"):
        quantize_grouped(torch.empty(8, 64, dtype=torch.bfloat16),
                         torch.empty(1, 8, 64, dtype=torch.bfloat16),
                         torch.zeros(2, dtype=torch.int32))


def test_inference_plan_argument_validation():
    from lightmoe import InferenceMoE

    cases = (
        (dict(hidden_size=100, intermediate_size=128), "align to 128"),
        (dict(num_experts=257), "at most 256 local experts"),
        (dict(num_experts=2, top_k=3), "top_k cannot exceed"),
        (dict(max_tokens=1 << 22), "max_tokens \\* top_k cannot exceed"),
        (dict(activation="gelu"), "unsupported expert activation"),
        (dict(activation="geglu", activation_clamp=3.0), "only for SwiGLU"),
        (dict(activation_clamp=-1.0), "finite and positive"),
        (dict(activation_sigmoid_alpha=2.0), "require swiglu_oai"),
        (dict(hidden_size=0), "hidden_size must be positive"),
        (dict(device="cpu"), "requires a CUDA device"),
    )
    base = dict(hidden_size=256, intermediate_size=128, num_experts=4, top_k=2, max_tokens=8)
    for override, message in cases:
        kwargs = {**base, **override}
        positional = [kwargs.pop(name) for name in
                      ("hidden_size", "intermediate_size", "num_experts", "top_k", "max_tokens")]
        with pytest.raises(ValueError, match=message):
            InferenceMoE(*positional, **kwargs)


def test_imports_are_self_contained():
    code = (
        "import lightmoe.kernels.grouped.runtime\n"
        "from lightmoe.kernels.gated import GatedEpilogue\n"
        "from lightmoe.kernels.grouped.runtime import GroupedNvfp4Gemm\n"
        "from lightmoe.training import MoEExpertLayer\n"
        "assert GroupedNvfp4Gemm.__name__ == 'GroupedNvfp4Gemm'\n"
        "assert GatedEpilogue('swiglu').activation == 'swiglu'\n"
    )
    subprocess.run([sys.executable, "-c", code], cwd=ROOT, check=True)


def test_product_package_never_imports_the_oracle():
    for path in (ROOT / "nvfp4moe_b200").rglob("*.py"):
        text = path.read_text()
        assert "oracle" not in text, path
    for path in (ROOT / "nvfp4moe_b200" / "csrc").glob("*.cu*"):
        assert "oracle" not in path.read_text(), path


def test_host_pipeline_needs_cuda():
    """The host-buffer pipeline has no CPU path: it refuses to build without a device."""
    import torch

    from nvfp4moe_b200 import HostPipeline

    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError, match="needs a CUDA device"):
        HostPipeline(object(), 8, 128, 2)
    with pytest.raises(ValueError, match="depth"):
        HostPipeline(object(), 8, 128, 2, depth=0)


def test_tensor_scale_tracks_amax_without_host_reads():
    """``TensorScale`` (``lightmoe/_quantization.py:14-67``): amax / 2688 with its reciprocal,
    floored at the smallest normal FP32, readable only after a first update."""
    from nvfp4moe_b200._quantization import TensorScale

    scale = TensorScale(device="cpu")
    with pytest.raises(AssertionError, match="before calibration"):
        scale.pair
    t = torch.tensor([[0.5, -5376.0], [3.0, 1.0]], dtype=torch.bfloat16)
    scale.update(t)
    assert scale.pair.dtype == torch.float32 and tuple(scale.pair.shape) == (2,)
    assert float(scale.pts) == 2.0 and float(scale.inv_pts) == 0.5  # |-5376| / 2688
    scale.update(torch.tensor([1344.0, -2.0]))
    assert float(scale.pts) == 0.5 and float(scale.inv_pts) == 2.0
    scale.set_amax(torch.tensor(2688.0))
    assert float(scale.pts) == 1.0 and float(scale.inv_pts) == 1.0
    # an all-zero tensor does not produce an infinite reciprocal
    scale.update(torch.zeros(4))
    assert float(scale.pts) == torch.finfo(torch.float32).tiny
    assert torch.isfinite(scale.inv_pts).all()
    # the views alias the pair: a later update is visible through views taken earlier
    pts_view = scale.pts
    scale.set_amax(torch.tensor(5376.0))
    assert float(pts_view) == 2.0
    with pytest.raises(NotImplementedError):
        TensorScale(device="cpu", te_rht=True)


def test_tracing_ranges_only_when_enabled(monkeypatch):
    """``tracing.traced`` opens and closes one NVTX range per call while enabled, none otherwise,
    and closes it when the call raises."""
    import torch

    from nvfp4moe_b200 import tracing

    events = []
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: events.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: events.append(("pop",)))

    @tracing.traced("lightmoe.stage")
    def stage(value, fail=False):
        if fail:
            raise ValueError("boom")
        return value + 1

    assert stage(1) == 2 and events == []
    tracing.enable()
    try:
        assert stage(2) == 3
        with pytest.raises(ValueError):
            stage(0, fail=True)
        opened = tracing.push("lightmoe.fc1")
        tracing.pop(opened)
    finally:
        tracing.enable(False)
    assert events == [("push", "lightmoe.stage"), ("pop",), ("push", "lightmoe.stage"), ("pop",),
                      ("push", "lightmoe.fc1"), ("pop",)]
    assert tracing.push("x") is False and not tracing.enabled()
    # the wrappers of the path carry their stage names
    from nvfp4moe_b200.kernels.routing.combine import moe_finalize
    from nvfp4moe_b200.kernels.routing.dispatch import moe_dispatch

    assert moe_dispatch.__name__ == "moe_dispatch" and moe_finalize.__name__ == "moe_finalize"


def test_ctypes_structs_match_the_header_layout(tmp_path):
    """The ctypes mirrors of ``lm_gemm_args`` / ``lm_gemm_plan`` have the size and the field
    offsets a C compiler gives the header's structs (the header is plain C: it compiles with gcc)."""
    import shutil

    from nvfp4moe_b200 import _lib

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    header = pathlib.Path(__file__).resolve().parents[1] / "include"
    fields = [name for name, _ in _lib.GemmArgs._fields_]
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "lightmoe_b200.h"', "int main(void) {",
             '  printf("%zu %zu\\n", sizeof(lm_gemm_args), sizeof(lm_gemm_plan));']
    lines += [f'  printf("{name} %zu\\n", offsetof(lm_gemm_args, {name}));' for name in fields]
    lines += ["  return 0;", "}"]
    source = tmp_path / "layout.c"
    source.write_text("\n".join(lines))
    binary = tmp_path / "layout"
    subprocess.run([gcc, "-std=c99", "-I", str(header), str(source), "-o", str(binary)], check=True)
    out = subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.split("\n")
    args_size, plan_size = map(int, out[0].split())
    assert args_size == ctypes.sizeof(_lib.GemmArgs)
    assert plan_size == ctypes.sizeof(_lib.GemmPlan)
    offsets = dict(line.split() for line in out[1:] if line)
    assert set(offsets) == set(fields)
    for name in fields:
        assert int(offsets[name]) == getattr(_lib.GemmArgs, name).offset, name


def test_ctypes_signatures_have_the_header_argument_counts():
    """Every prototype of the header takes as many arguments as the ctypes table passes."""
    from nvfp4moe_b200 import _lib

    text = (ROOT / "include" / "lightmoe_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = re.findall(r"\b[A-Za-z_][\w\s\*]*?\b(lm_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S)
    assert len(protos) >= 20
    for name, params in protos:
        params = params.strip()
        count = 0 if params in ("void", "") else len(params.split(","))
        assert count == len(_lib._SIGNATURES[name][1]), name
