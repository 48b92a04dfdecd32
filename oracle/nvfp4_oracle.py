"""CPU oracle for the NVFP4 routed-expert inference path.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain torch-on-CPU code,
the arithmetic that the reference project (roycho96/nvfp4moe, package
``lightmoe``) defines for its inference hot path.  It is imported by the test
suite, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py`` -- never by the product package, which must fail loudly when its
CUDA extension is missing.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imported the
reference's own CPU-runnable module (``benchmarks/reference.py``) and stored
its outputs as fixtures; ``tests/test_oracle_golden.py`` checks every function
below against those fixtures and against the known-answer vectors the
reference's tests hold (``tests/test_reference.py:10-52``).

Formats (``benchmarks/reference.py:8-22``)
  q      E2M1 codes, two per byte, even contraction index in the low nibble.
  sf     one E4M3 byte per 16 contraction elements.
  pts    one FP32 per-tensor scale;  value = e2m1 * sf * pts.
  blocked SF  128 rows x 4 scale factors form one 512-byte atom; row m of the
         atom sits at byte (m % 32) * 16 + (m // 32) * 4 + (k % 4).
  varlen SF   expert e's first atom row is m_indptr[e] // 128 + e.
"""

from __future__ import annotations

import math

import torch

F4_MAX = 6.0
E4M3_MAX = 448.0
E4M3_MIN_SF = 2.0**-9
SCALE_DEN = E4M3_MAX * F4_MAX  # 2688
F32_MAX = torch.finfo(torch.float32).max

_E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_TABLE = torch.tensor(
    _E2M1_MAGNITUDES + tuple(-v for v in _E2M1_MAGNITUDES), dtype=torch.float32
)


def _f32(v) -> torch.Tensor:
    return torch.as_tensor(v, dtype=torch.float32).reshape(-1)[:1]


# --------------------------------------------------------------------------
# scalar formats
# --------------------------------------------------------------------------


def e2m1_encode(v: torch.Tensor) -> torch.Tensor:
    """FP32 -> 4-bit E2M1 code, round-to-nearest-even, saturating at 6.

    Follows ``benchmarks/reference.py:52-69`` (hardware
    ``cvt.rn.satfinite.e2m1x2.f32``).  Written as a count of crossed decision
    thresholds: a tie goes to the neighbour whose code is even, which makes
    the thresholds 0.75, 1.75 and 3.5 inclusive and 0.25, 1.25, 2.5 and 5
    exclusive.
    """
    v = v.to(torch.float32)
    mag = v.abs()
    code = torch.zeros(v.shape, dtype=torch.uint8)
    for threshold, inclusive in (
        (0.25, False),
        (0.75, True),
        (1.25, False),
        (1.75, True),
        (2.5, False),
        (3.5, True),
        (5.0, False),
    ):
        crossed = (mag >= threshold) if inclusive else (mag > threshold)
        code += crossed.to(torch.uint8)
    negative = torch.signbit(v)
    return code | (negative.to(torch.uint8) << 3)


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """(..., K) codes -> (..., K/2) bytes (``benchmarks/reference.py:72-77``)."""
    lo = codes[..., 0::2]
    hi = codes[..., 1::2]
    return (lo | (hi << 4)).contiguous()


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """(..., K/2) bytes -> (..., K) FP32 values (``reference.py:80-85,196-199``)."""
    lo = (packed & 0xF).long()
    hi = (packed >> 4).long()
    codes = torch.stack((lo, hi), dim=-1).reshape(*packed.shape[:-1], -1)
    return _E2M1_TABLE[codes]


def e4m3_bytes(v: torch.Tensor) -> torch.Tensor:
    """FP32 (already clamped to <= 448) -> E4M3 byte, round-to-nearest-even."""
    return v.to(torch.float32).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_value(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).to(torch.float32)


def tensor_scale(x: torch.Tensor) -> torch.Tensor:
    """Per-tensor scale amax / 2688, floor 1e-30 (``lightmoe/gemm.py:25-28``)."""
    return (x.abs().amax().float() / SCALE_DEN).clamp_min(1e-30).reshape(1)


# --------------------------------------------------------------------------
# row-wise quantization
# --------------------------------------------------------------------------


def quantize_rows(x: torch.Tensor, pts, *, te_math: bool = False):
    """Quantize (..., K) along K in groups of 16.  Returns (q u8, sf u8).

    ``te_math=False`` is the divide chain of ``benchmarks/reference.py:92-110``
    and ``lightmoe/kernels/quantize/kernel.py:864-868,877``::

        sf    = e4m3(clamp((amax / 6) / pts, 2^-9, 448))
        q     = e2m1(x * ((1 / pts) / sf))

    ``te_math=True`` is the multiply chain the inference layer asks for
    (``kernel.py:861-862,875``)::

        sf    = e4m3(clamp(amax * ((1 / pts) * fp32(1/6)), 2^-9, 448))
        q     = e2m1(x * (1 / (sf * pts)))

    Every step is a separately rounded FP32 operation.
    """
    k = x.shape[-1]
    assert k % 16 == 0
    pts = _f32(pts)
    inv_pts = 1.0 / pts
    groups = x.to(torch.float32).reshape(*x.shape[:-1], k // 16, 16)
    amax = groups.abs().amax(dim=-1)
    if te_math:
        inv6 = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(6.0, dtype=torch.float32)
        scaled = amax * (inv_pts * inv6)
    else:
        scaled = (amax / F4_MAX) / pts
    sf = e4m3_bytes(scaled.clamp(min=E4M3_MIN_SF, max=E4M3_MAX))
    sf_value = e4m3_value(sf)
    if te_math:
        factor = 1.0 / (sf_value * pts)
    else:
        factor = inv_pts / sf_value
    scaled_x = groups * factor.unsqueeze(-1)
    q = pack_e2m1(e2m1_encode(scaled_x.reshape(x.shape)))
    return q, sf


def quantize_epilogue(x: torch.Tensor, pts):
    """Requantization contract of the fused fc1 epilogue.

    ``benchmarks/reference.py:113-126``: like the divide chain but with no
    lower clamp on the scale factor and the reciprocal capped at FLT_MAX (a
    group of zeros gets sf = 0 and codes 0).  The device kernel
    (``lightmoe/kernels/gated.py:309-344``) evaluates the same quantities with
    a multiply chain and ``rcp.approx``, so it is compared to this function
    with a tolerance on the number of differing codes, not bit for bit.
    """
    k = x.shape[-1]
    assert k % 16 == 0
    pts = _f32(pts)
    groups = x.to(torch.float32).reshape(*x.shape[:-1], k // 16, 16)
    amax = groups.abs().amax(dim=-1)
    sf = e4m3_bytes(((amax / F4_MAX) / pts).clamp(max=E4M3_MAX))
    factor = ((1.0 / pts) / e4m3_value(sf)).clamp(max=F32_MAX)
    scaled_x = (groups * factor.unsqueeze(-1)).clamp(-F4_MAX, F4_MAX)
    scaled_x = torch.nan_to_num(scaled_x, nan=0.0)
    q = pack_e2m1(e2m1_encode(scaled_x.reshape(x.shape)))
    return q, sf


def dequantize_rows(q: torch.Tensor, sf: torch.Tensor, pts) -> torch.Tensor:
    """(q u8 (..., K/2), sf u8 (..., K/16)) -> FP32 (``reference.py:196-202``)."""
    values = unpack_e2m1(q)
    scale = e4m3_value(sf).repeat_interleave(16, dim=-1)
    return values * scale * _f32(pts)


# --------------------------------------------------------------------------
# blocked scale-factor layout
# --------------------------------------------------------------------------


def sf_atom_offset(row_in_tile: int, k_group: int) -> int:
    """Byte offset of (row, k_group % 4) inside its 512-byte atom."""
    return (row_in_tile % 32) * 16 + (row_in_tile // 32) * 4 + (k_group % 4)


def sf_to_blocked(sf: torch.Tensor, tiles: int | None = None) -> torch.Tensor:
    """(rows, K/16) u8 -> (tiles, ceil(K/64), 32, 4, 4) u8, zero padded.

    ``benchmarks/reference.py:210-224``.
    """
    rows, groups = sf.shape
    tiles = tiles if tiles is not None else -(-rows // 128)
    chunks = -(-groups // 4)
    padded = torch.zeros(tiles * 128, chunks * 4, dtype=torch.uint8)
    padded[:rows, :groups] = sf
    # index order: tile, quarter (row // 32), lane (row % 32), chunk, k % 4
    v = padded.reshape(tiles, 4, 32, chunks, 4)
    return v.permute(0, 3, 2, 1, 4).contiguous()


def sf_from_blocked(blocked: torch.Tensor, rows: int, groups: int) -> torch.Tensor:
    """Inverse of :func:`sf_to_blocked` (``benchmarks/reference.py:227-232``)."""
    tiles, chunks = blocked.shape[:2]
    v = blocked.reshape(tiles, chunks, 32, 4, 4).permute(0, 3, 2, 1, 4)
    return v.reshape(tiles * 128, chunks * 4)[:rows, :groups].contiguous()


def varlen_tile_starts(m_indptr) -> list[int]:
    """First atom row of each expert (``benchmarks/reference.py:235-238``)."""
    cu = [int(v) for v in m_indptr]
    return [cu[e] // 128 + e for e in range(len(cu) - 1)]


def varlen_tile_total(m_indptr) -> int:
    """Atom rows needed for a varlen buffer (``reference.py:241-246``)."""
    cu = [int(v) for v in m_indptr]
    e = len(cu) - 1
    return cu[e - 1] // 128 + (e - 1) + -(-(cu[e] - cu[e - 1]) // 128)


def sf_to_varlen(sf: torch.Tensor, m_indptr, tiles: int | None = None) -> torch.Tensor:
    """(rows, K/16) u8 expert-major -> (1, tiles, K/64, 32, 4, 4) varlen buffer.

    Buffer size convention ``ceil(rows / 128) + E`` follows
    ``lightmoe/gemm.py:97-106``; placement follows
    ``benchmarks/reference.py:300-309``.
    """
    cu = [int(v) for v in m_indptr]
    experts = len(cu) - 1
    rows, groups = sf.shape
    tiles = tiles if tiles is not None else -(-rows // 128) + experts
    out = torch.zeros(1, tiles, -(-groups // 4), 32, 4, 4, dtype=torch.uint8)
    for e, start in enumerate(varlen_tile_starts(cu)):
        lo, hi = cu[e], cu[e + 1]
        if hi > lo:
            blk = sf_to_blocked(sf[lo:hi])
            out[0, start : start + blk.shape[0]] = blk
    return out


def sf_from_varlen(buf: torch.Tensor, m_indptr, groups: int) -> torch.Tensor:
    """Varlen buffer -> (rows, K/16) u8, valid rows only."""
    cu = [int(v) for v in m_indptr]
    out = torch.zeros(cu[-1], groups, dtype=torch.uint8)
    flat = buf.reshape(-1, *buf.shape[-4:])
    for e, start in enumerate(varlen_tile_starts(cu)):
        lo, hi = cu[e], cu[e + 1]
        if hi > lo:
            n = -(-(hi - lo) // 128)
            out[lo:hi] = sf_from_blocked(flat[start : start + n], hi - lo, groups)
    return out


# --------------------------------------------------------------------------
# dispatch (stable counting sort by expert)
# --------------------------------------------------------------------------


def route_topk(logits: torch.Tensor, top_k: int):
    """softmax -> topk -> renormalise, the recipe the reference's tests build their routing
    inputs with (``tests/test_training_gpu.py:23-27``)."""
    probs = torch.softmax(logits.float(), dim=-1)
    topv, topi = torch.topk(probs, top_k, dim=-1)
    return topi.to(torch.int32), (topv / topv.sum(-1, keepdim=True)).float()


def dispatch(topk_ids: torch.Tensor, topk_weights: torch.Tensor, experts: int,
             plan_tile_rows: int = 128, plan_len: int | None = None):
    """Stable expert-major permutation of (token, route) pairs.

    The torch chain of ``tests/test_training_gpu.py:577-587`` and
    ``tests/test_inference.py:337-348``: position p = token * k + route is
    sorted by expert id with ties in p order.  ``padded_offsets`` is the
    inclusive prefix of ``ceil(count / plan_tile_rows) * 128``
    (``lightmoe/kernels/routing/dispatch.py:139-141,158``; the two-kernel path
    always uses 128, ``:277``).  The decode plan (``dispatch.py:162-169``):
    ``plan[0]`` = number of row tiles, ``plan[1 + i]`` = expert + tile * E for
    the i-th tile in expert order, and the last E entries hold each expert's
    first scale-factor atom row.
    """
    tokens, k = topk_ids.shape
    flat = topk_ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    gather = (order // k).to(torch.int32)
    counts = torch.bincount(flat, minlength=experts)
    m_indptr = torch.zeros(experts + 1, dtype=torch.int32)
    m_indptr[1:] = counts.cumsum(0).to(torch.int32)
    probs = topk_weights.reshape(-1)[order].to(torch.float32)
    slots = torch.empty(tokens * k, dtype=torch.int32)
    slots[order] = torch.arange(tokens * k, dtype=torch.int32)
    tile_counts = (counts + plan_tile_rows - 1) // plan_tile_rows
    padded_offsets = (tile_counts * 128).cumsum(0).to(torch.int32)
    plan = None
    if plan_len is not None:
        plan = torch.zeros(plan_len, dtype=torch.int32)
        plan[0] = int(tile_counts.sum())
        cursor = 1
        first = 0
        for e in range(experts):
            n = int(tile_counts[e])
            for t in range(n):
                plan[cursor] = e + t * experts
                cursor += 1
            plan[plan_len - experts + e] = first
            first += n
    return gather, m_indptr, probs, slots, padded_offsets, plan


# --------------------------------------------------------------------------
# expert-parallel route plan (no reference code: the reference leaves the exchange to the
# host framework, README.md:227-228; this states the row order the peer transport uses)
# --------------------------------------------------------------------------


def ep_route_plan(counts_all, rank: int):
    """Where rows go when ``world`` ranks shard the experts contiguously.

    ``counts_all[g][e]`` = rows rank ``g`` routed to global expert ``e``.  On its owner an
    expert's rows are ordered by source rank, within a source in the source's own expert-major
    order.  Returns for ``rank``: ``own_indptr`` (bounds of the rows it receives),
    ``dest_base[e]`` (owner row where its rows of expert e begin), ``owner_start[e]`` (owner
    row where expert e begins), ``origin`` (for every row it receives: source rank, source row)
    and ``owner_rows`` (rows every rank receives).
    """
    counts = [[int(v) for v in row] for row in counts_all]
    world, experts = len(counts), len(counts[0])
    local = experts // world
    src_start = []
    for g in range(world):
        run, starts = 0, []
        for e in range(experts):
            starts.append(run)
            run += counts[g][e]
        src_start.append(starts)
    total = [sum(counts[g][e] for g in range(world)) for e in range(experts)]
    owner_start, owner_rows = [0] * experts, []
    for o in range(world):
        run = 0
        for l in range(local):
            owner_start[o * local + l] = run
            run += total[o * local + l]
        owner_rows.append(run)
    dest_base = [owner_start[e] + sum(counts[g][e] for g in range(rank)) for e in range(experts)]
    own_indptr = [owner_start[rank * local + l] for l in range(local)] + [owner_rows[rank]]
    origin = []
    for l in range(local):
        e = rank * local + l
        for g in range(world):
            origin += [(g, src_start[g][e] + i) for i in range(counts[g][e])]
    return own_indptr, dest_base, owner_start, origin, owner_rows


# --------------------------------------------------------------------------
# grouped / dense GEMM on dequantized operands
# --------------------------------------------------------------------------


def grouped_gemm(qa, sfa, qb, sfb, m_indptr, alpha) -> torch.Tensor:
    """FP32 ``out[rows_e] = alpha_e * deq(A_e) @ deq(B_e).T``.

    qa (rows, K/2) u8, sfa (rows, K/16) u8 row-major (not blocked),
    qb (E, N, K/2) u8, sfb (E, N, K/16) u8, alpha (1,) or (E,).
    The per-expert dequantized matmul of
    ``tests/test_training_gpu.py:265-279`` with both per-tensor scales folded
    into alpha as ``lightmoe/gemm.py:118`` does.
    """
    cu = [int(v) for v in m_indptr]
    experts, n, _ = qb.shape
    alpha = torch.as_tensor(alpha, dtype=torch.float32).reshape(-1)
    out = torch.zeros(qa.shape[0], n, dtype=torch.float32)
    for e in range(experts):
        lo, hi = cu[e], cu[e + 1]
        if hi == lo:
            continue
        a = dequantize_rows(qa[lo:hi], sfa[lo:hi], 1.0)
        b = dequantize_rows(qb[e], sfb[e], 1.0)
        scale = alpha[e] if alpha.numel() > 1 else alpha[0]
        out[lo:hi] = (a @ b.T) * scale
    return out


def dense_gemm(qa, sfa, qb, sfb, alpha) -> torch.Tensor:
    """FP32 ``alpha * deq(A) @ deq(B).T`` (``lightmoe/kernels/dense/runtime.py:54-143``)."""
    a = dequantize_rows(qa, sfa, 1.0)
    b = dequantize_rows(qb, sfb, 1.0)
    return (a @ b.T) * _f32(alpha)


# --------------------------------------------------------------------------
# activations
# --------------------------------------------------------------------------


def gated_activation(gate, up, activation: str, clamp: float | None = None,
                     sigmoid_alpha: float = 1.0, up_bias: float = 0.0) -> torch.Tensor:
    """``lightmoe/kernels/gated.py:148-172`` with exact exp / tanh.

    ``inference.py:763-777`` is the same math in torch form.
    """
    gate = gate.to(torch.float32)
    up = up.to(torch.float32)
    if clamp is not None and clamp > 0:
        gate = gate.clamp(max=clamp)
        up = up.clamp(min=-clamp, max=clamp)
    if activation in ("swiglu", "swiglu_oai"):
        return gate * torch.sigmoid(sigmoid_alpha * gate) * (up + up_bias)
    if activation == "geglu":
        return torch.nn.functional.gelu(gate, approximate="tanh") * up
    if activation == "reglu":
        return torch.relu(gate) * up
    raise ValueError(activation)


def unary_activation(v, activation: str) -> torch.Tensor:
    """``lightmoe/kernels/unary.py:42-51``."""
    if activation != "relu2":
        raise ValueError(activation)
    return torch.relu(v.to(torch.float32)).square()


def apply_activation(preact: torch.Tensor, activation: str, clamp=None,
                     sigmoid_alpha=1.0, up_bias=0.0) -> torch.Tensor:
    """fc1 accumulator (rows, 2I) with gate/up interleaved, or (rows, I) for relu2."""
    if activation == "relu2":
        return unary_activation(preact, activation)
    return gated_activation(preact[:, 0::2], preact[:, 1::2], activation, clamp,
                            sigmoid_alpha, up_bias)


# --------------------------------------------------------------------------
# combine
# --------------------------------------------------------------------------


def combine(routed_out: torch.Tensor, slots: torch.Tensor, top_k: int,
            weights: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = bf16(sum_j f32(routed_out[slot]) * w[slot])`` in route order.

    ``tests/test_finalize.py:28-37`` (unweighted) and
    ``tests/test_training_gpu.py:657-661`` (weighted).  The product is rounded
    to FP32 before the add (no fused multiply-add); slots of -1 contribute
    nothing.
    """
    tokens = slots.numel() // top_k
    acc = torch.zeros(tokens, routed_out.shape[1], dtype=torch.float32)
    table = slots.reshape(tokens, top_k).long()
    for j in range(top_k):
        s = table[:, j]
        valid = s >= 0
        rows = routed_out[s[valid]].to(torch.float32)
        if weights is not None:
            rows = rows * weights[s[valid]].to(torch.float32).unsqueeze(1)
        acc[valid] += rows
    return acc.to(torch.bfloat16)


# --------------------------------------------------------------------------
# weights and whole layer
# --------------------------------------------------------------------------


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """(E, I, H) x2 -> (E, 2I, H), row 2j = gate_j, row 2j+1 = up_j (``inference.py:389``)."""
    e, i, h = gate.shape
    return torch.stack((gate, up), dim=2).reshape(e, 2 * i, h)


def pack_weights(w: torch.Tensor, pts=None):
    """(E, N, K) -> q (E, N, K/2) u8, sf (E, N, K/16) u8, pts (1,)."""
    pts = tensor_scale(w) if pts is None else _f32(pts)
    q, sf = quantize_rows(w, pts, te_math=False)
    return q, sf, pts


def moe_layer(x, topk_ids, topk_weights, w1_q, w1_sf, w1_pts, w2_q, w2_sf, w2_pts,
              x_scale, h_scale, activation="swiglu", clamp=None, sigmoid_alpha=1.0,
              up_bias=0.0, return_stages=False):
    """Quantization-aware layer: the stage order of ``inference.py:883-930``.

    dispatch -> gather + te-math quantize -> fc1 on dequantized operands ->
    activation -> epilogue requantization -> fc2 -> BF16 round -> weighted
    combine.
    """
    experts = w1_q.shape[0]
    gather, m_indptr, probs, slots, padded, _ = dispatch(topk_ids, topk_weights, experts)
    xg = x[gather.long()]
    qx, sfx = quantize_rows(xg, x_scale, te_math=True)
    alpha1 = _f32(x_scale) * torch.as_tensor(w1_pts, dtype=torch.float32).reshape(-1)
    pre = grouped_gemm(qx, sfx, w1_q, w1_sf, m_indptr, alpha1)
    hidden = apply_activation(pre, activation, clamp, sigmoid_alpha, up_bias)
    qh, sfh = quantize_epilogue(hidden, h_scale)
    alpha2 = _f32(h_scale) * torch.as_tensor(w2_pts, dtype=torch.float32).reshape(-1)
    routed = grouped_gemm(qh, sfh, w2_q, w2_sf, m_indptr, alpha2).to(torch.bfloat16)
    out = combine(routed, slots, topk_ids.shape[1], probs)
    if return_stages:
        return out, dict(gather=gather, m_indptr=m_indptr, probs=probs, slots=slots,
                         padded_offsets=padded, qx=qx, sfx=sfx, pre=pre, hidden=hidden,
                         qh=qh, sfh=sfh, routed=routed)
    return out


def moe_layer_sampled(x, topk_ids, topk_weights, expert_weights, w1_pts, w2_pts, x_scale, h_scale,
                      activation="swiglu", clamp=None, sigmoid_alpha=1.0, up_bias=0.0):
    """:func:`moe_layer` for a handful of tokens of a large batch.

    Every output row of the layer depends on its own token only, so a sample of the tokens can
    be checked end to end without the whole batch: ``x`` (T, H), ``topk_ids`` / ``topk_weights``
    (T, k) are the sampled rows and ``expert_weights[e]`` = ``(w1_q, w1_sf, w2_q, w2_sf)`` holds
    the packed weights (row-major scale factors) of every expert the sample touches.  Same
    stage order and arithmetic as :func:`moe_layer` (``inference.py:883-930``).
    """
    tokens, k = topk_ids.shape
    w1_pts = torch.as_tensor(w1_pts, dtype=torch.float32).reshape(-1)
    w2_pts = torch.as_tensor(w2_pts, dtype=torch.float32).reshape(-1)
    qx, sfx = quantize_rows(x, x_scale, te_math=True)
    xd = dequantize_rows(qx, sfx, 1.0)
    routed = torch.zeros(tokens, k, x.shape[1], dtype=torch.bfloat16)
    for e in topk_ids.unique().tolist():
        tok, route = (topk_ids == e).nonzero(as_tuple=True)
        w1_q, w1_sf, w2_q, w2_sf = expert_weights[e]
        alpha1 = _f32(x_scale) * (w1_pts[e] if w1_pts.numel() > 1 else w1_pts[0])
        alpha2 = _f32(h_scale) * (w2_pts[e] if w2_pts.numel() > 1 else w2_pts[0])
        pre = (xd[tok] @ dequantize_rows(w1_q, w1_sf, 1.0).T) * alpha1
        hidden = apply_activation(pre, activation, clamp, sigmoid_alpha, up_bias)
        qh, sfh = quantize_epilogue(hidden, h_scale)
        out = (dequantize_rows(qh, sfh, 1.0) @ dequantize_rows(w2_q, w2_sf, 1.0).T) * alpha2
        routed[tok, route] = out.to(torch.bfloat16)
    acc = torch.zeros(tokens, x.shape[1], dtype=torch.float32)
    for j in range(k):
        acc += routed[:, j].to(torch.float32) * topk_weights[:, j].to(torch.float32).unsqueeze(1)
    return acc.to(torch.bfloat16)


def calibrate(x, topk_ids, topk_weights, w1_q, w1_sf, w1_pts, activation="swiglu",
              clamp=None, sigmoid_alpha=1.0, up_bias=0.0):
    """Static activation scales as ``inference.py:723-805`` derives them.

    x_scale = amax(gathered x) / 2688; fc1 runs un-fused to BF16, the
    activation is applied in FP32, h_scale = amax(hidden) / 2688.
    """
    experts = w1_q.shape[0]
    gather, m_indptr, *_ = dispatch(topk_ids, topk_weights, experts)
    xg = x[gather.long()]
    x_scale = tensor_scale(xg)
    qx, sfx = quantize_rows(xg, x_scale, te_math=True)
    alpha1 = x_scale * torch.as_tensor(w1_pts, dtype=torch.float32).reshape(-1)
    pre = grouped_gemm(qx, sfx, w1_q, w1_sf, m_indptr, alpha1).to(torch.bfloat16)
    hidden = apply_activation(pre.float(), activation, clamp, sigmoid_alpha, up_bias)
    return x_scale, tensor_scale(hidden)


def bf16_layer(x, topk_ids, topk_weights, first, second, down, activation="swiglu",
               clamp=None, sigmoid_alpha=1.0, up_bias=0.0) -> torch.Tensor:
    """Unquantized FP32 layer on the BF16 master weights.

    Same contract as ``tests/test_inference.py:25-53`` and
    ``tests/test_training_gpu.py:40-53``; used for the cosine gates only.
    """
    tokens, k = topk_ids.shape
    out = torch.zeros(tokens, x.shape[1], dtype=torch.float32)
    xf = x.to(torch.float32)
    for e in topk_ids.unique().tolist():
        tok, route = (topk_ids == e).nonzero(as_tuple=True)
        src = xf[tok]
        g = src @ first[e].to(torch.float32).T
        if activation == "relu2":
            hidden = unary_activation(g, activation)
        else:
            u = src @ second[e].to(torch.float32).T
            hidden = gated_activation(g, u, activation, clamp, sigmoid_alpha, up_bias)
        y = hidden @ down[e].to(torch.float32).T
        out.index_add_(0, tok, y * topk_weights[tok, route].to(torch.float32).unsqueeze(1))
    return out


def rel_frobenius(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a = actual.to(torch.float64)
    b = expected.to(torch.float64)
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def cosine(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a = actual.to(torch.float64).flatten()
    b = expected.to(torch.float64).flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm()).clamp_min(1e-300))


__all__ = [name for name in dir() if not name.startswith("_") and name not in ("math", "torch", "annotations")]
