"""GPU parity tests: each CUDA kernel, called through the C-ABI, against the CPU oracle.

Bit-exact classes: packed E2M1 bytes, E4M3 scale-factor bytes of valid rows,
gather / m_indptr / probs / slots / padded_offsets / decode plan, combine.
Tolerance classes (stated beside each assert): GEMM outputs and the fused
activation + requantization epilogue.
"""

import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

GEMM_REL_TOL = 1e-2  # relative Frobenius error vs the dequantized-matmul oracle rounded to BF16


def _cuda(t):
    return t.cuda()


def _indptr(lens):
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens).cumsum(0)
    return cu


# --------------------------------------------------------------------------
# quantize
# --------------------------------------------------------------------------


@pytest.mark.parametrize("te_math", (False, True))
@pytest.mark.parametrize("features", (64, 256, 2048, 2688))
def test_rowwise_quantize_varlen_bit_exact(te_math, features):
    from nvfp4moe_b200.kernels.quantize import nvfp4_quantize_rowwise

    # segment lengths of the reference's own quantizer test (tests/test_training_gpu.py:231-263)
    lens = [400, 0, 137, 256, 71, 0, 128, 32]
    cu = _indptr(lens)
    rows = int(cu[-1])
    g = torch.Generator().manual_seed(features + int(te_math))
    x = torch.randn(rows, features, generator=g).to(torch.bfloat16)
    x[3, :16] = 0
    x[5, 16:32] *= 1e-5
    pts = O.tensor_scale(x)
    q_ref, sf_ref = O.quantize_rows(x, pts, te_math=te_math)
    tiles = -(-rows // 128) + len(lens)
    sf_buf_ref = O.sf_to_varlen(sf_ref, cu, tiles)

    pair = torch.cat((pts, 1.0 / pts)).cuda()
    q = torch.zeros(rows, features // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(1, tiles, features // 64, 32, 4, 4, dtype=torch.float8_e4m3fn, device="cuda")
    nvfp4_quantize_rowwise(x.cuda(), cu.cuda(), pair, q, sf, te_math=te_math)
    torch.cuda.synchronize()
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(sf.view(torch.uint8).cpu(), sf_buf_ref)


def test_rowwise_quantize_gathered_and_garbage_buffer():
    from nvfp4moe_b200.kernels.quantize import nvfp4_quantize_rowwise

    g = torch.Generator().manual_seed(7)
    tokens, features, experts, k = 96, 512, 6, 3
    x = torch.randn(tokens, features, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens)]).int()
    ids[ids == 4] = 0  # expert 4 gets nothing (ids may repeat inside a token: still a valid sort)
    gather, cu, *_ = O.dispatch(ids, torch.rand(tokens, k, generator=g), experts)
    rows = tokens * k
    pts = O.tensor_scale(x)
    q_ref, sf_ref = O.quantize_rows(x[gather.long()], pts, te_math=True)
    tiles = -(-rows // 128) + experts
    pair = torch.cat((pts, 1.0 / pts)).cuda()
    q = torch.empty(rows, features // 2, dtype=torch.uint8, device="cuda")
    sf = torch.full((1, tiles, features // 64, 32, 4, 4), 0x7F, dtype=torch.uint8, device="cuda")
    nvfp4_quantize_rowwise(x.cuda(), cu.cuda(), pair, q, sf.view(torch.float8_e4m3fn),
                           gather_idx=gather.cuda(), te_math=True)
    torch.cuda.synchronize()
    assert torch.equal(q.cpu(), q_ref)
    # only valid rows are defined when the buffer started as garbage
    assert torch.equal(O.sf_from_varlen(sf.cpu(), cu, features // 16), sf_ref)


def test_rowwise_quantize_fp32_input_and_linear_layout():
    from nvfp4moe_b200.kernels.quantize import nvfp4_quantize_rowwise

    g = torch.Generator().manual_seed(8)
    rows, features = 70, 256
    x = torch.randn(rows, features, generator=g) * 3
    cu = _indptr([rows])
    pts = O.tensor_scale(x)
    q_ref, sf_ref = O.quantize_rows(x, pts)
    pair = torch.cat((pts, 1.0 / pts)).cuda()
    q = torch.empty(rows, features // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(rows, features // 16, dtype=torch.uint8, device="cuda")
    nvfp4_quantize_rowwise(x.cuda(), cu.cuda(), pair, q, sf, sf_layout="linear")
    torch.cuda.synchronize()
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(sf.cpu(), sf_ref)


def test_public_quantize_helpers_match_oracle():
    from nvfp4moe_b200 import gemm

    g = torch.Generator().manual_seed(9)
    x = torch.randn(300, 192, generator=g).to(torch.bfloat16)
    q, sf, scale = gemm.quantize(x.cuda())
    # torch divides by a constant on the GPU as a multiplication by its reciprocal, so the
    # scale may sit one ulp from the CPU value; the quantizer is checked on the scale it was given
    pts = scale.cpu()
    assert abs(float(pts) / float(O.tensor_scale(x)) - 1.0) < 3e-7
    q_ref, sf_ref = O.quantize_rows(x, pts)
    assert q.dtype == torch.float4_e2m1fn_x2 and tuple(sf.shape) == (3, 3, 32, 4, 4)
    assert torch.equal(q.view(torch.uint8).cpu(), q_ref)
    assert torch.equal(sf.view(torch.uint8).cpu(), O.sf_to_blocked(sf_ref))

    with pytest.raises(ValueError, match="contiguous CUDA matrix"):
        gemm.quantize(x)  # CPU tensor: tests/test_gemm_api.py:22-26


# --------------------------------------------------------------------------
# dispatch
# --------------------------------------------------------------------------


def _route(tokens, experts, k, dist, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(tokens, experts, generator=g)
    if dist == "hot":
        logits[:, seed % experts] += 4.0
    elif dist == "sparse":
        logits[:, : experts // 2] -= 6.0
    topv, topi = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    topv = (topv / topv.sum(-1, keepdim=True)).float().contiguous()
    return topi.to(torch.int32).contiguous(), topv


@pytest.mark.parametrize(
    "shape",
    ((2048, 8, 8), (1024, 32, 8), (512, 64, 8), (4096, 8, 2), (8192, 32, 8), (65, 256, 8),
     (65, 48, 8), (17, 4, 2), (1, 4, 2), (8192, 256, 8), (3000, 128, 4)),
)
def test_dispatch_matches_stable_sort(shape):
    from nvfp4moe_b200 import MoEDispatch

    tokens, experts, k = shape
    disp = MoEDispatch(tokens, experts, k)
    for dist in ("uniform", "hot", "sparse"):
        for seed in (0, 1):
            ids, w = _route(tokens, experts, k, dist, seed)
            ref = O.dispatch(ids, w, experts)
            ids_d, w_d = ids.cuda(), w.cuda()
            got = [t.clone() for t in disp(ids_d, w_d)]
            off = disp.off_pad.clone()
            torch.cuda.synchronize()
            for a, b in zip(got, ref[:4]):
                assert torch.equal(a.cpu(), b)
            assert torch.equal(off.cpu(), ref[4])
            assert torch.equal(ids_d.cpu(), ids) and torch.equal(w_d.cpu(), w)
            again = disp(ids_d, w_d)
            assert all(torch.equal(a, b) for a, b in zip(got, again))


@pytest.mark.parametrize("plan_tile_rows", (8, 16, 32, 128))
def test_dispatch_decode_plan(plan_tile_rows):
    from nvfp4moe_b200.kernels.routing.dispatch import moe_dispatch, scratch_elems

    tokens, experts, k = 64, 128, 8
    ids, w = _route(tokens, experts, k, "hot", 3)
    rows = tokens * k
    n = scratch_elems(rows, experts)
    ref = O.dispatch(ids, w, experts, plan_tile_rows, n)
    dev = "cuda"
    gi = torch.empty(rows, dtype=torch.int32, device=dev)
    cu = torch.empty(experts + 1, dtype=torch.int32, device=dev)
    ps = torch.empty(rows, dtype=torch.float32, device=dev)
    slots = torch.empty(rows, dtype=torch.int32, device=dev)
    part = torch.zeros(n, dtype=torch.int32, device=dev)
    off = torch.empty(experts, dtype=torch.int32, device=dev)
    moe_dispatch(ids.cuda(), w.cuda(), experts, gi, cu, ps, slots, part, off,
                 plan_tile_rows=plan_tile_rows)
    torch.cuda.synchronize()
    assert torch.equal(off.cpu(), ref[4])
    plan = part.cpu()
    tiles = int(ref[5][0])
    assert int(plan[0]) == tiles
    assert torch.equal(plan[1 : 1 + tiles], ref[5][1 : 1 + tiles])
    assert torch.equal(plan[-experts:], ref[5][-experts:])


# --------------------------------------------------------------------------
# combine
# --------------------------------------------------------------------------


@pytest.mark.parametrize("weighted", (False, True))
def test_combine_exact(weighted):
    from nvfp4moe_b200.kernels.routing.combine import moe_finalize

    # tests/test_finalize.py:28-75
    g = torch.Generator().manual_seed(0)
    tokens, k, d = 1024, 8, 2048
    rows = tokens * k
    yw = (torch.randn(rows, d, generator=g) * 0.1).to(torch.bfloat16)
    order = torch.randperm(rows, generator=g)
    slots = torch.empty(rows, dtype=torch.int32)
    slots[order] = torch.arange(rows, dtype=torch.int32)
    slots[torch.rand(rows, generator=g) < 0.1] = -1
    slots[:k] = -1  # token 0 loses every route
    w = torch.rand(rows, generator=g) if weighted else None
    ref = O.combine(yw, slots, k, w)
    out = torch.empty(tokens, d, dtype=torch.bfloat16, device="cuda")
    yw_d, slots_d = yw.cuda(), slots.cuda()
    w_d = w.cuda() if weighted else None
    moe_finalize(yw_d, slots_d, out, k, weights=w_d)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), ref)
    assert (out[0] == 0).all()
    base = out.clone()
    for _ in range(5):
        moe_finalize(yw_d, slots_d, out, k, weights=w_d, tile_t=2, n_frag=2)
        assert torch.equal(out, base)


# --------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------


def _grouped_case(lens, n, k, seed, a_std=1.0, b_std=0.02):
    g = torch.Generator().manual_seed(seed)
    cu = _indptr(lens)
    rows = int(cu[-1])
    a = (torch.randn(rows, k, generator=g) * a_std).to(torch.bfloat16)
    b = (torch.randn(len(lens), n, k, generator=g) * b_std).to(torch.bfloat16)
    return cu, a, b


def _device_scales(a, b):
    """Per-tensor scales as the library derives them (on the GPU), copied to the host."""
    from nvfp4moe_b200.gemm import _tensor_scale

    return _tensor_scale(a.cuda(), None).cpu(), _tensor_scale(b.cuda(), None).cpu()


def _run_grouped(cu, a, b, alpha_scale=None, out_dtype=torch.bfloat16, tile_n=128, max_ctas=0, tile_m=128):
    from nvfp4moe_b200 import gemm

    experts, n, k = b.shape
    qa, qb, sfa, sfb, alpha = gemm.quantize_grouped(a.cuda(), b.cuda(), cu.cuda())
    pa, pb = _device_scales(a, b)
    assert torch.equal(alpha.cpu(), pa * pb)
    if alpha_scale is not None:
        alpha = alpha * alpha_scale.cuda()
    out = torch.full((a.shape[0], n), float("nan"), dtype=out_dtype, device="cuda")
    plan = gemm.GroupedGemm(experts, n, k, tile_m, tile_n, output_dtype=out_dtype)
    plan.max_ctas = max_ctas
    plan(qa, qb, out, cu.cuda(), sfa, sfb, alpha)
    torch.cuda.synchronize()
    return out, (qa, qb, sfa, sfb, alpha)


def _oracle_grouped(cu, a, b, alpha_scale=None):
    pa, pb = _device_scales(a, b)
    assert abs(float(pa) / float(O.tensor_scale(a)) - 1.0) < 3e-7
    assert abs(float(pb) / float(O.tensor_scale(b)) - 1.0) < 3e-7
    qa, sfa = O.quantize_rows(a, pa)
    qb, sfb = O.quantize_rows(b, pb)
    alpha = pa * pb
    if alpha_scale is not None:
        alpha = alpha * alpha_scale
    return O.grouped_gemm(qa, sfa, qb, sfb, cu, alpha), (qa, sfa, qb, sfb)


def test_grouped_gemm_config1():
    """E=8, K=2048, N=1024, 512 rows from top-2 routing of 256 tokens, experts 3 and 6 empty."""
    g = torch.Generator().manual_seed(0)
    allowed = torch.tensor([0, 1, 2, 4, 5, 7])
    picks = torch.stack([allowed[torch.randperm(6, generator=g)[:2]] for _ in range(256)])
    counts = torch.bincount(picks.flatten(), minlength=8)
    assert counts[3] == 0 and counts[6] == 0
    cu, a, b = _grouped_case(counts.tolist(), 1024, 2048, 0)
    from nvfp4moe_b200.gemm import GroupedGemm  # noqa: F401

    out, packed = _run_grouped(cu, a, b)
    ref, packed_ref = _oracle_grouped(cu, a, b)
    # operands are bit-exact ...
    assert torch.equal(packed[0].view(torch.uint8).cpu(), packed_ref[0])
    assert torch.equal(packed[1].view(torch.uint8).cpu(), packed_ref[2])
    assert torch.equal(O.sf_from_varlen(packed[2].view(torch.uint8).cpu(), cu, 128), packed_ref[1])
    # ... and the product is within tolerance of the dequantized matmul
    ref_bf16 = ref.to(torch.bfloat16)
    assert torch.isfinite(out).all()
    assert O.rel_frobenius(out.cpu().float(), ref_bf16.float()) <= GEMM_REL_TOL
    # quantization band vs the unquantized operands (reference gate: cosine >= 0.99086)
    full = torch.zeros_like(ref)
    for e in range(8):
        lo, hi = int(cu[e]), int(cu[e + 1])
        full[lo:hi] = a[lo:hi].float() @ b[e].float().T
    assert O.cosine(out.cpu().float(), full) >= 0.99


@pytest.mark.parametrize(
    ("lens", "n", "k"),
    (
        ([3, 5, 2, 7], 128, 256),            # tests/test_inference.py:504-531
        ([1, 15, 16, 127, 128, 129, 255, 256, 257, 0], 256, 512),  # edge counts of routing_counts
        ([130, 0, 0, 77], 384, 2688),        # K not a multiple of 256
        ([64] * 16, 128, 64),                # single 64-wide K step
        ([300], 136, 320),                   # N tail inside a tile
    ),
)
def test_grouped_gemm_ragged_shapes(lens, n, k):
    cu, a, b = _grouped_case(lens, n, k, seed=len(lens) + n + k, b_std=0.05)
    out, _ = _run_grouped(cu, a, b)
    ref, _ = _oracle_grouped(cu, a, b)
    assert torch.isfinite(out).all()
    assert O.rel_frobenius(out.cpu().float(), ref.to(torch.bfloat16).float()) <= GEMM_REL_TOL


@pytest.mark.parametrize("out_dtype", (torch.bfloat16, torch.float32))
@pytest.mark.parametrize("max_ctas", (0, 3))
@pytest.mark.parametrize("k", (1280, 2048))
def test_grouped_gemm_wide_tiles_bit_identical(out_dtype, max_ctas, k):
    """128 x 256 tiles accumulate every output in the same order as 128 x 128 tiles, with the
    even split of the epilogue (K = 1280) and the uneven one (K >= 1536)."""
    lens = [130, 0, 257, 5, 128, 300, 0, 64]
    cu, a, b = _grouped_case(lens, 1024, k, seed=77, b_std=0.05)
    narrow, _ = _run_grouped(cu, a, b, out_dtype=out_dtype)
    wide, _ = _run_grouped(cu, a, b, out_dtype=out_dtype, tile_n=256, max_ctas=max_ctas)
    ref, _ = _oracle_grouped(cu, a, b)
    assert torch.isfinite(wide).all()
    assert torch.equal(wide, narrow)
    tol = GEMM_REL_TOL if out_dtype == torch.bfloat16 else 1e-5
    ref = ref.to(out_dtype).float()
    assert O.rel_frobenius(wide.cpu().float(), ref) <= tol
    from nvfp4moe_b200 import _lib

    assert _lib.device_status() == 0


@pytest.mark.parametrize("out_dtype", (torch.bfloat16, torch.float32))
@pytest.mark.parametrize("max_ctas", (0, 4))
@pytest.mark.parametrize("k", (1280, 2048))
def test_grouped_gemm_cta_pairs_bit_identical(out_dtype, max_ctas, k):
    """256 x 256 tiles on CTA pairs accumulate every output in the same order as 128 x 128 tiles
    (both splits of the epilogue, as above)."""
    lens = [130, 0, 257, 5, 128, 300, 0, 64, 513, 256]
    cu, a, b = _grouped_case(lens, 1024, k, seed=78, b_std=0.05)
    narrow, _ = _run_grouped(cu, a, b, out_dtype=out_dtype)
    pairs, _ = _run_grouped(cu, a, b, out_dtype=out_dtype, tile_n=256, tile_m=256, max_ctas=max_ctas)
    assert torch.isfinite(pairs).all()
    assert torch.equal(pairs, narrow)
    from nvfp4moe_b200 import _lib

    assert _lib.device_status() == 0


@pytest.mark.parametrize("out_dtype", (torch.bfloat16, torch.float32))
@pytest.mark.parametrize("n", (384, 640))
@pytest.mark.parametrize("tile_m", (128, 256))
def test_grouped_gemm_half_empty_last_wide_tile(out_dtype, n, tile_m):
    """N of an odd number of 128-column blocks on 256-column tiles: the last tile's second half
    has no weights (its loads reach into the next expert or past the tensor) and stores nothing;
    every stored value equals the 128 x 128 result, and nothing beyond column N is written."""
    lens = [130, 0, 257, 5, 128, 300, 64]
    cu, a, b = _grouped_case(lens, n, 1280, seed=90 + n, b_std=0.05)
    narrow, _ = _run_grouped(cu, a, b, out_dtype=out_dtype)
    wide, _ = _run_grouped(cu, a, b, out_dtype=out_dtype, tile_n=256, tile_m=tile_m)
    ref, _ = _oracle_grouped(cu, a, b)
    assert torch.isfinite(wide).all()
    assert torch.equal(wide, narrow)
    tol = GEMM_REL_TOL if out_dtype == torch.bfloat16 else 1e-5
    assert O.rel_frobenius(wide.cpu().float(), ref.to(out_dtype).float()) <= tol
    from nvfp4moe_b200 import _lib

    assert _lib.device_status() == 0


@pytest.mark.parametrize(("n", "k"), ((256, 2688), (512, 64), (768, 192)))
def test_grouped_gemm_cta_pairs_ragged_k(n, k):
    """CTA pairs when K is not a multiple of the 256-element stage: the last stage holds fewer
    64-element chunks (its scale-factor box reaches past K and reads zeros), down to a single
    chunk for the whole contraction."""
    lens = [259, 0, 1, 128, 640]
    cu, a, b = _grouped_case(lens, n, k, seed=n + k, b_std=0.05)
    narrow, _ = _run_grouped(cu, a, b)
    pairs, _ = _run_grouped(cu, a, b, tile_n=256, tile_m=256)
    ref, _ = _oracle_grouped(cu, a, b)
    assert torch.isfinite(pairs).all()
    assert torch.equal(pairs, narrow)
    assert O.rel_frobenius(pairs.cpu().float(), ref.to(torch.bfloat16).float()) <= GEMM_REL_TOL
    from nvfp4moe_b200 import _lib

    assert _lib.device_status() == 0


def test_grouped_gemm_fp32_output_and_per_expert_alpha():
    lens = [3, 5, 2, 7]
    cu, a, b = _grouped_case(lens, 128, 256, seed=20260822, b_std=1.0)
    scale = torch.arange(1, 5, dtype=torch.float32)
    out, _ = _run_grouped(cu, a, b, alpha_scale=scale, out_dtype=torch.float32)
    ref, _ = _oracle_grouped(cu, a, b, alpha_scale=scale)
    # FP32 output: only the accumulation order differs from the oracle
    assert O.rel_frobenius(out.cpu(), ref) <= 1e-5


def test_dense_gemm_matches_oracle():
    from nvfp4moe_b200 import gemm

    g = torch.Generator().manual_seed(5)
    m, n, k = 333, 512, 1024
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
    qa, sfa, pa = gemm.quantize(a.cuda())
    qb, sfb, pb = gemm.quantize(b.cuda())
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    plan = gemm.DenseGemm(n, k, 128, 128)
    plan(qa, qb, out, sfa, sfb, pa * pb)
    torch.cuda.synchronize()
    qa_r, sfa_r = O.quantize_rows(a, pa.cpu())
    qb_r, sfb_r = O.quantize_rows(b, pb.cpu())
    ref = O.dense_gemm(qa_r, sfa_r, qb_r, sfb_r, pa.cpu() * pb.cpu())
    assert O.rel_frobenius(out.cpu().float(), ref.to(torch.bfloat16).float()) <= GEMM_REL_TOL
    # the other tilings the constructor admits (wide tiles, CTA pairs) give the same bits
    for tile_m, tile_n in ((128, 256), (256, 256)):
        other = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
        gemm.DenseGemm(n, k, tile_m, tile_n)(qa, qb, other, sfa, sfb, pa * pb)
        torch.cuda.synchronize()
        assert torch.equal(other, out), (tile_m, tile_n)
    with pytest.raises(RuntimeError, match="prepare must run before launch"):
        gemm.DenseGemm(n, k, 128, 128).launch()


# --------------------------------------------------------------------------
# fused activation + requantization epilogue
# --------------------------------------------------------------------------


@pytest.mark.parametrize(
    ("activation", "clamp"),
    (("swiglu", None), ("swiglu", 10.0), ("swiglu_oai", None), ("geglu", None), ("reglu", None),
     ("relu2", None)),
)
@pytest.mark.parametrize(("tile_m", "tile_n"), ((128, 128), (128, 256), (256, 256)))
@pytest.mark.parametrize("inter", (256, 384))
def test_fused_epilogue_matches_oracle(activation, clamp, tile_m, tile_n, inter):
    """``inter`` 384: N = 768 (gated) is whole 256-column tiles, N = 384 (ReLU squared) leaves
    half of the last wide tile empty."""
    from nvfp4moe_b200 import gemm
    from nvfp4moe_b200.kernels.gated import GatedEpilogue
    from nvfp4moe_b200.kernels.unary import UnaryEpilogue

    lens = [40, 0, 200, 129]
    hidden = 512
    n = inter if activation == "relu2" else 2 * inter
    cu, a, b = _grouped_case(lens, n, hidden, seed=11, b_std=hidden**-0.5)
    rows = a.shape[0]
    qa, qb, sfa, sfb, alpha = gemm.quantize_grouped(a.cuda(), b.cuda(), cu.cuda())
    ref_pre, _ = _oracle_grouped(cu, a, b)
    if activation == "relu2":
        policy = UnaryEpilogue(activation)
        hidden_ref = O.apply_activation(ref_pre, activation)
    else:
        policy = GatedEpilogue(activation, clamp_limit=clamp)
        hidden_ref = O.apply_activation(ref_pre, activation, policy.clamp_limit,
                                        policy.sigmoid_alpha, policy.up_bias)
    h_pts = O.tensor_scale(hidden_ref)
    q_ref, sf_ref = O.quantize_epilogue(hidden_ref, h_pts)

    tiles = -(-rows // 128) + len(lens)
    qh = torch.zeros(rows, inter // 2, dtype=torch.uint8, device="cuda")
    sfh = torch.zeros(1, tiles, inter // 64, 32, 4, 4, dtype=torch.float8_e4m3fn, device="cuda")
    pair = torch.cat((h_pts, 1.0 / h_pts)).cuda()
    plan = gemm.GroupedGemm(len(lens), n, hidden, tile_m, tile_n, output_dtype=torch.float4_e2m1fn_x2,
                            epilogue=policy)
    plan.max_ctas = 2 if tile_n == 256 else 0
    plan(qa, qb, qh.view(torch.float4_e2m1fn_x2), cu.cuda(), sfa, sfb, alpha, output_sf=sfh,
         output_scale=pair)
    torch.cuda.synchronize()
    sf_got = O.sf_from_varlen(sfh.view(torch.uint8).cpu(), cu, inter // 16)
    q_got = qh.cpu()
    # approximate exp / reciprocal and a different accumulation order may move a value
    # across a rounding boundary: at least 99 % of bytes identical ...
    assert (sf_got == sf_ref).float().mean() >= 0.99
    assert (q_got == q_ref).float().mean() >= 0.99
    # ... and the dequantized result within 2 % of the oracle's
    deq = O.dequantize_rows(q_got, sf_got, h_pts)
    deq_ref = O.dequantize_rows(q_ref, sf_ref, h_pts)
    assert O.rel_frobenius(deq, deq_ref) <= 2e-2


# --------------------------------------------------------------------------
# decode-shaped GEMM: weights on the 128-row side of the MMA (swap_ab), direct routes
# --------------------------------------------------------------------------


def _run_swapped(cu, packed, n, k, out_dtype=torch.bfloat16, max_ctas=0, use_pdl=False):
    from nvfp4moe_b200 import gemm

    qa, qb, sfa, sfb, alpha = packed
    out = torch.full((qa.shape[0], n), float("nan"), dtype=out_dtype, device="cuda")
    plan = gemm.GroupedGemm(qb.shape[0], n, k, 128, 32, output_dtype=out_dtype, swap_ab=True,
                            use_pdl=use_pdl)
    plan.max_ctas = max_ctas
    plan(qa, qb, out, cu.cuda(), sfa, sfb, alpha)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("out_dtype", (torch.bfloat16, torch.float32))
@pytest.mark.parametrize(
    ("lens", "n", "k", "max_ctas"),
    (
        ([1, 0, 2, 1], 256, 512, 0),                       # fewer blocks than SMs: quarter-block shares
        ([1, 0, 0, 0, 1, 0, 1, 1], 1024, 2048, 0),          # one token, four experts
        ([3, 8, 9, 16, 17, 0, 31, 32], 384, 768, 0),        # every token-box size up to 32 rows
        ([5, 33, 64, 65, 0, 130, 1, 200], 512, 1280, 0),    # 64-row chunks, several per expert
        ([5, 33, 64, 65, 0, 130, 1, 200], 512, 1280, 5),    # few CTAs: whole blocks, many tiles each
        ([7, 2, 0, 12], 136, 320, 3),                       # N tail inside a block, K tail inside a stage
        ([2] * 64, 256, 256, 0),                            # many experts
    ),
)
def test_swapped_decode_gemm_bit_identical(lens, n, k, max_ctas, out_dtype):
    """The decode-shaped kernel accumulates every output over the whole K in the same order as
    the 128 x 128 tiles: identical bits, and within tolerance of the oracle."""
    from nvfp4moe_b200 import _lib

    cu, a, b = _grouped_case(lens, n, k, seed=n + k + len(lens), b_std=0.05)
    base, packed = _run_grouped(cu, a, b, out_dtype=out_dtype)
    for pdl in (False, True):
        got = _run_swapped(cu, packed, n, k, out_dtype, max_ctas, use_pdl=pdl)
        assert torch.isfinite(got).all()
        assert torch.equal(got, base), (lens, n, k, pdl)
    ref, _ = _oracle_grouped(cu, a, b)
    tol = GEMM_REL_TOL if out_dtype == torch.bfloat16 else 1e-5
    assert O.rel_frobenius(base.cpu().float(), ref.to(out_dtype).float()) <= tol
    assert _lib.device_status() == 0


@pytest.mark.parametrize(
    ("activation", "clamp"),
    (("swiglu", None), ("swiglu_oai", None), ("swiglu", 10.0), ("geglu", None), ("reglu", None),
     ("relu2", None)),
)
def test_swapped_decode_fused_epilogue_bit_identical(activation, clamp):
    """Activation + NVFP4 requantization of the decode-shaped kernel: byte for byte the codes
    and scale factors of the 128 x 128 kernel (whose bytes are checked against the oracle in
    test_fused_epilogue_matches_oracle)."""
    from nvfp4moe_b200 import gemm
    from nvfp4moe_b200.kernels.gated import GatedEpilogue
    from nvfp4moe_b200.kernels.unary import UnaryEpilogue

    lens = [1, 0, 9, 40, 2, 70, 129]
    inter, hidden = 256, 512
    n = inter if activation == "relu2" else 2 * inter
    cu, a, b = _grouped_case(lens, n, hidden, seed=13, b_std=hidden**-0.5)
    rows = a.shape[0]
    qa, qb, sfa, sfb, alpha = gemm.quantize_grouped(a.cuda(), b.cuda(), cu.cuda())
    policy = UnaryEpilogue(activation) if activation == "relu2" else GatedEpilogue(activation, clamp_limit=clamp)
    tiles = -(-rows // 128) + len(lens)
    pair = torch.tensor([0.004, 250.0], device="cuda")
    results = []
    for swap in (False, True):
        qh = torch.full((rows, inter // 2), 0xEE, dtype=torch.uint8, device="cuda")
        sfh = torch.zeros(1, tiles, inter // 64, 32, 4, 4, dtype=torch.float8_e4m3fn, device="cuda")
        plan = gemm.GroupedGemm(len(lens), n, hidden, 128, 32 if swap else 128,
                                output_dtype=torch.float4_e2m1fn_x2, epilogue=policy, swap_ab=swap)
        plan(qa, qb, qh.view(torch.float4_e2m1fn_x2), cu.cuda(), sfa, sfb, alpha, output_sf=sfh,
             output_scale=pair)
        torch.cuda.synchronize()
        results.append((qh.cpu(), O.sf_from_varlen(sfh.view(torch.uint8).cpu(), cu, inter // 16)))
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1], results[1][1])
    assert (results[1][0] != 0xEE).any()


def test_direct_routes_equal_the_dispatched_token():
    """One token, k routes, no dispatch: fc1 reads row 0 for every route (broadcast) and fc2 row
    r for route r; expert ids come from the route table.  Equal, bit for bit, to the same token
    run through the expert-major path."""
    from nvfp4moe_b200 import gemm
    from nvfp4moe_b200.kernels.gated import GatedEpilogue

    experts, hidden, inter, k = 16, 512, 256, 4
    g = torch.Generator().manual_seed(21)
    x = torch.randn(1, hidden, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(experts, 2 * inter, hidden, generator=g) * hidden**-0.5).to(torch.bfloat16)
    w2 = (torch.randn(experts, hidden, inter, generator=g) * inter**-0.5).to(torch.bfloat16)
    routes = torch.tensor([9, 2, 14, 5], dtype=torch.int32)  # not sorted: route order is kept
    order = torch.argsort(routes)
    counts = torch.bincount(routes.long(), minlength=experts)
    cu = torch.zeros(experts + 1, dtype=torch.int32)
    cu[1:] = counts.cumsum(0)
    rows = x.expand(k, hidden).contiguous()
    qa, qb1, sfa, sfb1, alpha1 = gemm.quantize_grouped(rows.cuda(), w1.cuda(), cu.cuda())
    pair = torch.tensor([0.004, 250.0], device="cuda")
    policy = GatedEpilogue("swiglu")
    sf_rows = 1 + experts

    def buffers():
        qh = torch.zeros(k, inter // 2, dtype=torch.uint8, device="cuda")
        sfh = torch.zeros(1, sf_rows, inter // 64, 32, 4, 4, dtype=torch.float8_e4m3fn, device="cuda")
        out = torch.zeros(k, hidden, dtype=torch.bfloat16, device="cuda")
        return qh, sfh, out

    # fc2 operands: packed once through the public helper (its activations are unused here)
    _, qb2, _, sfb2, _ = gemm.quantize_grouped(torch.zeros(k, inter, dtype=torch.bfloat16, device="cuda"),
                                                w2.cuda(), cu.cuda())
    alpha2 = torch.tensor([0.5], device="cuda")
    # expert-major path
    qh, sfh, out = buffers()
    fc1 = gemm.GroupedGemm(experts, 2 * inter, hidden, 128, 128, output_dtype=torch.float4_e2m1fn_x2,
                           epilogue=policy)
    fc1(qa, qb1, qh.view(torch.float4_e2m1fn_x2), cu.cuda(), sfa, sfb1, alpha1, output_sf=sfh, output_scale=pair)
    fc2 = gemm.GroupedGemm(experts, hidden, inter, 128, 128)
    fc2(qh.view(torch.float4_e2m1fn_x2), qb2, out, cu.cuda(), sfh, sfb2, alpha2)
    torch.cuda.synchronize()
    want = out[torch.argsort(order).cuda()].cpu()  # back to route order
    # direct path: the token quantized once into row 0 / atom row 0
    qx1 = qa[:1].contiguous()
    sfx1 = torch.zeros(1, 1 + experts, hidden // 64, 32, 4, 4, dtype=torch.float8_e4m3fn, device="cuda")
    first_tile = int(cu[int(routes.min())]) // 128 + int(routes.min())
    # row 0 of the lowest expert's atom row holds this token's factors
    sfx1.view(torch.uint8)[0, 0] = sfa.view(torch.uint8)[0, first_tile]
    qh, sfh, out = buffers()
    table = routes.cuda()
    d1 = gemm.GroupedGemm(experts, 2 * inter, hidden, 128, 128, output_dtype=torch.float4_e2m1fn_x2,
                          epilogue=policy, use_dynamic_sched=False, use_pdl=True, direct_routes=k,
                          broadcast_a=True)
    qx_rows = torch.zeros(k, hidden // 2, dtype=torch.uint8, device="cuda")
    qx_rows[0] = qx1.view(torch.uint8)[0]
    d1(qx_rows.view(torch.float4_e2m1fn_x2), qb1, qh.view(torch.float4_e2m1fn_x2), table, sfx1, sfb1, alpha1,
       output_sf=sfh, output_scale=pair)
    d2 = gemm.GroupedGemm(experts, hidden, inter, 128, 128, use_dynamic_sched=False, use_pdl=True,
                          direct_routes=k)
    d2(qh.view(torch.float4_e2m1fn_x2), qb2, out, table, sfh, sfb2, alpha2)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and float(out.float().abs().sum()) > 0
    assert torch.equal(out.cpu(), want)


# --------------------------------------------------------------------------
# decode preparation: dispatch + plan + quantize in one launch
# --------------------------------------------------------------------------


@pytest.mark.parametrize(("tokens", "experts", "k", "features"),
                         ((1, 8, 2, 256), (17, 64, 4, 2048), (64, 256, 8, 6144), (128, 32, 8, 512)))
def test_fused_decode_prepare_matches_oracle(tokens, experts, k, features):
    from nvfp4moe_b200.kernels.quantize import nvfp4_dispatch_quantize_decode
    from nvfp4moe_b200.kernels.routing.dispatch import scratch_elems

    ids, w = _route(tokens, experts, k, "hot", tokens)
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, features, generator=g).to(torch.bfloat16)
    rows = tokens * k
    n = scratch_elems(rows, experts)
    ref = O.dispatch(ids, w, experts, 8, n)
    pts = O.tensor_scale(x)
    q_ref, sf_ref = O.quantize_rows(x[ref[0].long()], pts, te_math=True)
    tiles = -(-rows // 128) + experts
    dev = "cuda"
    gi = torch.empty(rows, dtype=torch.int32, device=dev)
    cu = torch.empty(experts + 1, dtype=torch.int32, device=dev)
    ps = torch.empty(rows, dtype=torch.float32, device=dev)
    slots = torch.empty(rows, dtype=torch.int32, device=dev)
    part = torch.zeros(n, dtype=torch.int32, device=dev)
    off = torch.empty(experts, dtype=torch.int32, device=dev)
    q = torch.empty(rows, features // 2, dtype=torch.uint8, device=dev)
    sf = torch.full((1, tiles, features // 64, 32, 4, 4), 0x7F, dtype=torch.uint8, device=dev)
    pair = torch.cat((pts, 1.0 / pts)).cuda()
    nvfp4_dispatch_quantize_decode(x.cuda(), ids.cuda(), w.cuda(), part, gi, cu, ps, slots, off,
                                   pair, q, sf, plan_tile_rows=8)
    torch.cuda.synchronize()
    for got, want in zip((gi, cu, ps, slots, off), ref[:5]):
        assert torch.equal(got.cpu(), want)
    plan = part.cpu()
    count = int(ref[5][0])
    assert torch.equal(plan[: 1 + count], ref[5][: 1 + count])
    assert torch.equal(plan[-experts:], ref[5][-experts:])
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(O.sf_from_varlen(sf.cpu(), ref[1], features // 16), sf_ref)


@pytest.mark.parametrize(("tokens", "experts", "k", "features"),
                         ((333, 64, 4, 2048), (1500, 256, 8, 2048), (96, 32, 6, 6144), (2048, 128, 4, 6144)))
def test_quantize_once_scatter_matches_oracle_bytes(tokens, experts, k, features):
    """The quantizer of the prefill step (and of decode steps beyond 1024 routes): each token
    is quantized once and its bytes are stored to every expert-major row it was routed to.
    Byte for byte the result must be the row quantizer applied to the gathered rows, as the
    reference pins it (tests/test_training_gpu.py:231-263); routes whose slot is -1 are
    dropped and leave their destination bytes untouched."""
    from nvfp4moe_b200.kernels.quantize import nvfp4_quantize_decode

    ids, w = _route(tokens, experts, k, "hot", features + tokens)
    g = torch.Generator().manual_seed(tokens + experts)
    x = torch.randn(tokens, features, generator=g).to(torch.bfloat16)
    x[1, :32] = 0
    x[2, 16:48] *= 1e-6
    rows = tokens * k
    gather, cu, _, slots, off, _ = O.dispatch(ids, w, experts)
    pts = O.tensor_scale(x)
    q_ref, sf_ref = O.quantize_rows(x[gather.long()], pts, te_math=True)
    tiles = -(-rows // 128) + experts
    # drop every 7th route: its row keeps the fill pattern
    dropped = slots.clone()
    dropped[::7] = -1
    lost_rows = slots[::7].long()
    dev = "cuda"
    pair = torch.cat((pts, 1.0 / pts)).to(dev)
    for slot_table, lost in ((slots, None), (dropped, lost_rows)):
        q = torch.full((rows, features // 2), 0xA5, dtype=torch.uint8, device=dev)
        sf = torch.full((1, tiles, features // 64, 32, 4, 4), 0x7F, dtype=torch.uint8, device=dev)
        nvfp4_quantize_decode(x.to(dev), ids.to(dev), slot_table.to(dev), cu.to(dev), off.to(dev), pair,
                              q, sf.view(torch.float8_e4m3fn))
        torch.cuda.synchronize()
        q_want = q_ref.clone()
        sf_want = sf_ref.clone()
        if lost is not None:
            q_want[lost] = 0xA5
            sf_want[lost] = 0x7F
        assert torch.equal(q.cpu(), q_want)
        assert torch.equal(O.sf_from_varlen(sf.cpu(), cu, features // 16), sf_want)


@pytest.mark.parametrize(("experts", "k", "features"), ((8, 2, 256), (256, 8, 6144), (64, 32, 2048), (5, 5, 512)))
def test_one_token_prepare_matches_oracle(experts, k, features):
    """``nvfp4_decode_prepare`` / ``nvfp4_direct_decode_prepare``: one token, no scratch, one
    launch.  Expert-major form: the oracle's dispatch and gathered-row quantizer, bit for bit.
    Direct form: identity slots, the expert ids as the route table, the row quantized once."""
    from nvfp4moe_b200.kernels import nvfp4_decode_prepare
    from nvfp4moe_b200.kernels.quantize import nvfp4_direct_decode_prepare

    g = torch.Generator().manual_seed(experts + k)
    ids = torch.randperm(experts, generator=g)[:k].to(torch.int32).reshape(1, k)
    w = torch.rand(1, k, generator=g)
    x = torch.randn(1, features, generator=g).to(torch.bfloat16)
    pts = O.tensor_scale(x)
    pair = torch.cat((pts, 1.0 / pts)).cuda()
    gather_ref, cu_ref, probs_ref, slots_ref, padded_ref, _ = O.dispatch(ids, w, experts)
    q_ref, sf_ref = O.quantize_rows(x, pts, te_math=True)
    dev = "cuda"
    tiles = 1 + experts

    def buffers(table):
        return dict(gather=torch.full((k,), -1, dtype=torch.int32, device=dev),
                    slots=torch.full((k,), -1, dtype=torch.int32, device=dev),
                    table=torch.full((table,), -1, dtype=torch.int32, device=dev),
                    probs=torch.full((k,), -1.0, device=dev),
                    padded=torch.full((experts,), -1, dtype=torch.int32, device=dev),
                    q=torch.zeros(k, features // 2, dtype=torch.uint8, device=dev),
                    sf=torch.zeros(1, tiles, features // 64, 32, 4, 4, dtype=torch.uint8, device=dev))

    b = buffers(experts + 1)
    nvfp4_decode_prepare(x.cuda(), ids.cuda(), w.cuda(), b["gather"], b["slots"], b["table"], b["probs"],
                         b["padded"], pair, b["q"], b["sf"].view(torch.float8_e4m3fn))
    torch.cuda.synchronize()
    for got, want in ((b["gather"], gather_ref), (b["slots"], slots_ref), (b["table"], cu_ref),
                      (b["probs"], probs_ref), (b["padded"], padded_ref)):
        assert torch.equal(got.cpu(), want)
    assert torch.equal(b["q"].cpu(), q_ref.expand(k, -1))
    assert torch.equal(O.sf_from_varlen(b["sf"].cpu(), cu_ref, features // 16), sf_ref.expand(k, -1))

    d = buffers(k)
    nvfp4_direct_decode_prepare(x.cuda(), ids.cuda(), w.cuda(), d["gather"], d["slots"], d["table"], d["probs"],
                                d["padded"], pair, d["q"], d["sf"].view(torch.float8_e4m3fn))
    torch.cuda.synchronize()
    assert torch.equal(d["slots"].cpu(), torch.arange(k, dtype=torch.int32))
    assert torch.equal(d["table"].cpu(), ids[0])
    assert torch.equal(d["probs"].cpu(), w[0])
    assert torch.equal(d["q"][0].cpu(), q_ref[0]) and not d["q"][1:].any()
    assert torch.equal(O.sf_from_blocked(d["sf"][0, :1].cpu(), 1, features // 16), sf_ref)
    with pytest.raises(ValueError, match="one token"):
        nvfp4_decode_prepare(x.cuda().expand(2, -1).contiguous(), ids.cuda().expand(2, -1).contiguous(),
                             w.cuda().expand(2, -1).contiguous(), b["gather"], b["slots"], b["table"],
                             b["probs"], b["padded"], pair, b["q"], b["sf"].view(torch.float8_e4m3fn))


# --------------------------------------------------------------------------
# router step: softmax -> top-k -> renormalise
# --------------------------------------------------------------------------


@pytest.mark.parametrize(("tokens", "experts", "k", "dtype"),
                         ((1, 8, 2, torch.float32), (333, 256, 8, torch.float32), (64, 128, 4, torch.bfloat16),
                          (1000, 48, 6, torch.float32), (17, 5, 5, torch.float32)))
def test_route_topk_matches_torch_recipe(tokens, experts, k, dtype):
    from nvfp4moe_b200.routing import route_topk

    g = torch.Generator().manual_seed(tokens + experts)
    logits = (torch.randn(tokens, experts, generator=g) * 3.0).to(dtype)
    ids_ref, w_ref = O.route_topk(logits, k)
    ids, w = route_topk(logits.cuda(), k)
    torch.cuda.synchronize()
    assert ids.dtype == torch.int32 and w.dtype == torch.float32
    if dtype == torch.float32:
        assert torch.equal(ids.cpu(), ids_ref)
    else:  # BF16 logits tie often: the winners must carry the same probabilities
        probs = torch.softmax(logits.float(), -1)
        assert torch.equal(probs.gather(1, ids.cpu().long()), probs.gather(1, ids_ref.long()))
        assert (ids.cpu().sort(1).values[:, 1:] != ids.cpu().sort(1).values[:, :-1]).all()
    assert torch.allclose(w.cpu(), w_ref, rtol=2e-6, atol=1e-8)
    assert torch.allclose(w.cpu().sum(1), torch.ones(tokens), atol=1e-6)
    # feeds the dispatch directly
    from nvfp4moe_b200.kernels.routing.dispatch import MoEDispatch

    _, m_indptr, _, _ = MoEDispatch(tokens, experts, k)(ids, w)
    assert int(m_indptr[-1]) == tokens * k


def test_route_topk_rejects_bad_arguments():
    from nvfp4moe_b200.routing import route_topk

    logits = torch.zeros(4, 300, device="cuda")
    with pytest.raises(ValueError, match="at most 256 experts"):
        route_topk(logits, 2)
    with pytest.raises(ValueError, match="top_k"):
        route_topk(torch.zeros(4, 8, device="cuda"), 9)
    with pytest.raises(ValueError, match="BF16 or FP32"):
        route_topk(torch.zeros(4, 8, device="cuda", dtype=torch.float16), 2)
