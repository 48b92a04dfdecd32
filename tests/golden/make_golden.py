"""Generate golden vectors from the reference's own CPU-runnable module.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/reference

It imports ``benchmarks/reference.py`` from that checkout (nothing is copied),
feeds it seeded inputs and stores inputs and outputs in
``tests/golden/reference_vectors.npz``.  The test suite only reads the ``.npz``;
the reference checkout is not needed to run the tests.
"""

import importlib.util
import pathlib
import sys

import numpy as np
import torch


def _load_reference(root: pathlib.Path):
    spec = importlib.util.spec_from_file_location(
        "reference_module", root / "benchmarks" / "reference.py"
    )
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def _bits(t: torch.Tensor) -> np.ndarray:
    """Raw bits of a tensor as a numpy array (bf16 -> int16, fp8 -> uint8)."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().copy()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def main() -> None:
    root = pathlib.Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    ref = _load_reference(root)
    out: dict[str, np.ndarray] = {}

    # 1. divide-chain row quantization, three magnitudes (seeds 0..2)
    for seed, (rows, k, spread) in enumerate(((96, 256, 1.0), (40, 192, 0.02), (33, 64, 300.0))):
        g = torch.Generator().manual_seed(seed)
        x = (torch.randn(rows, k, generator=g) * spread).to(torch.bfloat16)
        if seed == 0:
            x[3, 16:32] = 0  # one all-zero group: exercises the 2^-9 scale floor
            x[5, 0:16] = x[5, 0:16] * 1e-4  # tiny group
        pts = ref.per_tensor_scale_from_amax(x.abs().max()).reshape(1)
        q, sf = ref.quantize_nvfp4_lastdim(x, pts)
        deq = ref.dequantize_nvfp4_lastdim(q, sf, pts)
        out[f"quant{seed}_x"] = _bits(x)
        out[f"quant{seed}_pts"] = pts.numpy()
        out[f"quant{seed}_q"] = _bits(q)
        out[f"quant{seed}_sf"] = _bits(sf)
        out[f"quant{seed}_deq"] = deq.numpy()

    # 2. fused-epilogue requantization contract
    g = torch.Generator().manual_seed(10)
    h = torch.randn(64, 128, generator=g) * 3.0
    h[7, 32:48] = 0
    h[9, 0:16] *= 1e-6
    pts = ref.per_tensor_scale_from_amax(h.abs().max()).reshape(1)
    q, sf = ref.quantize_nvfp4_fused_epilogue(h, pts)
    out["epi_x"] = h.numpy()
    out["epi_pts"] = pts.numpy()
    out["epi_q"] = _bits(q)
    out["epi_sf"] = _bits(sf)

    # 3. multiply-chain (TE) quantization on a power-of-two scale, where the
    #    reference's TE helper and the inference kernel's te-math coincide
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(48, 256, generator=g) * 60.0).to(torch.bfloat16)
    x.clamp_(-330, 330)
    x[0, 0] = 336.0  # amax = 2688 / 8  ->  pts = 2^-3 exactly
    amax = x.abs().max().float()
    q, sf, gds = ref.quantize_nvfp4_lastdim_te(x, amax)
    out["te_x"] = _bits(x)
    out["te_pts"] = gds.reshape(1).numpy()
    out["te_q"] = _bits(q)
    out["te_sf"] = _bits(sf)

    # 4. blocked scale-factor packing, ragged shapes
    for idx, (rows, cols) in enumerate(((128, 4), (300, 47), (17, 8))):
        g = torch.Generator().manual_seed(20 + idx)
        dense = torch.randint(0, 120, (rows, cols), generator=g, dtype=torch.uint8)
        blocked = ref.pack_sf_blocked(dense.view(torch.float8_e4m3fn))
        out[f"pack{idx}_dense"] = dense.numpy()
        out[f"pack{idx}_blocked"] = _bits(blocked)

    # 5. varlen offsets and the fused gather + rowwise quantize composition
    cu = torch.tensor([0, 100, 300, 300, 812], dtype=torch.int32)
    out["varlen_cu"] = cu.numpy()
    out["varlen_starts"] = np.array(ref.varlen_sf_tile_offsets(cu), dtype=np.int32)
    out["varlen_total"] = np.array([ref.varlen_sf_num_tiles(cu)], dtype=np.int32)

    g = torch.Generator().manual_seed(30)
    tokens, hidden = 64, 128
    lens = [40, 0, 137, 3, 0, 130]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    gather = torch.randint(0, tokens, (int(cu[-1]),), generator=g, dtype=torch.int32)
    pts = ref.per_tensor_scale_from_amax(x.abs().max()).reshape(1)
    fused = ref.fused_gather_dual_quantize_ref(x, gather, cu, pts, want_colwise=False)["rowwise"]
    out["gather_x"] = _bits(x)
    out["gather_idx"] = gather.numpy()
    out["gather_cu"] = cu.numpy()
    out["gather_pts"] = pts.numpy()
    out["gather_q"] = _bits(fused["qdata"])
    out["gather_sf"] = _bits(fused["sf"])

    target = pathlib.Path(__file__).with_name("reference_vectors.npz")
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({target.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
