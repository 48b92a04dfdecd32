"""Pin the CPU oracle to vectors produced by the reference's own CPU code.

Fixtures come from ``tests/golden/make_golden.py`` (which imported the
reference's ``benchmarks/reference.py``); known answers come from the
reference's tests (``tests/test_reference.py:10-52``,
``tests/test_inference.py:208-231``).
"""

import numpy as np
import torch

from conftest import bf16_from_bits
from oracle import nvfp4_oracle as O


def _u8(a):
    return torch.from_numpy(a.copy())


def test_divide_chain_quantize_matches_reference(golden):
    for seed in range(3):
        x = bf16_from_bits(golden[f"quant{seed}_x"])
        pts = torch.from_numpy(golden[f"quant{seed}_pts"])
        q, sf = O.quantize_rows(x, pts, te_math=False)
        assert torch.equal(q, _u8(golden[f"quant{seed}_q"])), seed
        assert torch.equal(sf, _u8(golden[f"quant{seed}_sf"])), seed
        deq = O.dequantize_rows(q, sf, pts)
        assert torch.equal(deq, torch.from_numpy(golden[f"quant{seed}_deq"])), seed


def test_epilogue_requant_matches_reference(golden):
    x = torch.from_numpy(golden["epi_x"])
    q, sf = O.quantize_epilogue(x, torch.from_numpy(golden["epi_pts"]))
    assert torch.equal(q, _u8(golden["epi_q"]))
    assert torch.equal(sf, _u8(golden["epi_sf"]))


def test_multiply_chain_quantize_matches_reference_on_pow2_scale(golden):
    x = bf16_from_bits(golden["te_x"])
    pts = torch.from_numpy(golden["te_pts"])
    assert float(pts) == 0.125
    q, sf = O.quantize_rows(x, pts, te_math=True)
    assert torch.equal(q, _u8(golden["te_q"]))
    assert torch.equal(sf, _u8(golden["te_sf"]))


def test_blocked_layout_matches_reference(golden):
    for idx in range(3):
        dense = _u8(golden[f"pack{idx}_dense"])
        blocked = O.sf_to_blocked(dense)
        assert torch.equal(blocked, _u8(golden[f"pack{idx}_blocked"]))
        back = O.sf_from_blocked(blocked, *dense.shape)
        assert torch.equal(back, dense)


def test_atom_mapping_known_answer():
    # tests/test_reference.py:10-18
    dense = (torch.arange(512) % 200).reshape(128, 4).to(torch.uint8)
    flat = O.sf_to_blocked(dense).reshape(-1)
    for row in (0, 1, 31, 32, 33, 95, 127):
        for col in range(4):
            assert flat[O.sf_atom_offset(row, col)] == dense[row, col]


def test_varlen_known_answer(golden):
    # tests/test_reference.py:42-52
    cu = golden["varlen_cu"]
    assert O.varlen_tile_starts(cu) == [0, 1, 4, 5]
    assert O.varlen_tile_starts(cu) == golden["varlen_starts"].tolist()
    assert O.varlen_tile_total(cu) == 9 == int(golden["varlen_total"][0])


def test_gather_quantize_varlen_matches_reference(golden):
    x = bf16_from_bits(golden["gather_x"])
    gather = torch.from_numpy(golden["gather_idx"])
    cu = golden["gather_cu"]
    pts = torch.from_numpy(golden["gather_pts"])
    q, sf = O.quantize_rows(x[gather.long()], pts)
    assert torch.equal(q, _u8(golden["gather_q"]))
    expected = _u8(golden["gather_sf"])
    buf = O.sf_to_varlen(sf, cu, tiles=expected.shape[0])
    assert torch.equal(buf[0], expected)
    assert torch.equal(O.sf_from_varlen(buf, cu, sf.shape[1]), sf)


def test_e2m1_ties_round_to_even():
    v = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -0.75, -0.0, 0.26])
    codes = O.e2m1_encode(v).tolist()
    assert codes == [0, 2, 2, 4, 4, 6, 6, 7, 8, 10, 8, 1]


def test_dispatch_known_answers():
    # tests/test_inference.py:208-231
    ids = torch.tensor([[1, 3]], dtype=torch.int32)
    w = torch.tensor([[0.625, 0.375]])
    gather, cu, probs, slots, padded, _ = O.dispatch(ids, w, 4)
    assert gather.tolist() == [0, 0]
    assert cu.tolist() == [0, 0, 1, 1, 2]
    assert probs.tolist() == [0.625, 0.375]
    assert slots.tolist() == [0, 1]
    assert padded.tolist() == [0, 128, 128, 256]


def test_dispatch_is_a_stable_sort():
    g = torch.Generator().manual_seed(20260821)
    for experts in (48, 128, 256):
        ids = torch.randint(experts, (65, 8), generator=g, dtype=torch.int32)
        w = torch.rand(65, 8, generator=g)
        gather, cu, probs, slots, padded, plan = O.dispatch(ids, w, experts, 8, 128 * experts)
        flat = ids.flatten()
        assert torch.equal(flat[slots.argsort().long()].sort(stable=True).values, flat.sort().values)
        # rows of one expert keep source order
        for e in range(experts):
            rows = gather[int(cu[e]) : int(cu[e + 1])]
            assert (rows[1:] >= rows[:-1]).all()
        assert torch.equal(probs[slots.long()], w.flatten())
        counts = (cu[1:] - cu[:-1]).long()
        tiles = (counts + 7) // 8
        assert int(plan[0]) == int(tiles.sum())
        assert torch.equal(padded.long(), (tiles * 128).cumsum(0))
        firsts = plan[-experts:].long()
        assert torch.equal(firsts, tiles.cumsum(0) - tiles)


def test_combine_orders_and_drops():
    g = torch.Generator().manual_seed(0)
    rows = torch.randn(24, 32, generator=g).to(torch.bfloat16)
    slots = torch.randperm(24, generator=g).to(torch.int32)
    slots[5] = -1
    w = torch.rand(24, generator=g)
    out = O.combine(rows, slots, 3, w)
    t = 1
    acc = torch.zeros(32)
    for j in range(3):
        s = int(slots[t * 3 + j])
        if s >= 0:
            acc = acc + rows[s].float() * w[s]
    assert torch.equal(out[t], acc.to(torch.bfloat16))


def test_layer_tracks_bf16_reference():
    g = torch.Generator().manual_seed(20260819)
    tokens, hidden, inter, experts, k = 17, 256, 128, 4, 2
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    gate = (torch.randn(experts, inter, hidden, generator=g) * hidden**-0.5).to(torch.bfloat16)
    up = (torch.randn(experts, inter, hidden, generator=g) * hidden**-0.5).to(torch.bfloat16)
    down = (torch.randn(experts, hidden, inter, generator=g) * inter**-0.5).to(torch.bfloat16)
    ids = torch.tensor([[0, 1], [1, 0]] * 8 + [[0, 1]], dtype=torch.int32)
    w = torch.rand(tokens, k, generator=g)
    w /= w.sum(1, keepdim=True)
    w1 = O.pack_weights(O.interleave_gate_up(gate, up))
    w2 = O.pack_weights(down)
    xs, hs = O.calibrate(x, ids, w, *w1)
    out = O.moe_layer(x, ids, w, *w1, *w2, xs, hs)
    ref = O.bf16_layer(x, ids, w, gate, up, down)
    assert O.cosine(out, ref) > 0.95  # tests/test_inference.py:166-170
    assert np.isfinite(out.float().numpy()).all()


def test_sampled_layer_oracle_equals_whole_batch_oracle():
    """``moe_layer_sampled`` (used by the full-size GPU tests) computes the same rows as
    ``moe_layer`` run on the whole batch."""
    tokens, hidden, inter, experts, k = 40, 128, 64, 6, 3
    g = torch.Generator().manual_seed(11)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    gate = (torch.randn(experts, inter, hidden, generator=g) * 0.09).to(torch.bfloat16)
    up = (torch.randn(experts, inter, hidden, generator=g) * 0.09).to(torch.bfloat16)
    down = (torch.randn(experts, hidden, inter, generator=g) * 0.12).to(torch.bfloat16)
    ids, w = O.route_topk(torch.randn(tokens, experts, generator=g), k)
    w1 = O.pack_weights(O.interleave_gate_up(gate, up))
    w2 = O.pack_weights(down)
    xs, hs = O.calibrate(x, ids, w, *w1, "swiglu_oai", 7.0, 1.702, 1.0)
    full = O.moe_layer(x, ids, w, *w1, *w2, xs, hs, "swiglu_oai", 7.0, 1.702, 1.0)
    sample = torch.tensor([0, 7, 8, 23, 39])
    table = {e: (w1[0][e], w1[1][e], w2[0][e], w2[1][e]) for e in ids[sample].unique().tolist()}
    part = O.moe_layer_sampled(x[sample], ids[sample], w[sample], table, w1[2], w2[2], xs, hs,
                               "swiglu_oai", 7.0, 1.702, 1.0)
    # same arithmetic on the same values; only the row count of the FP32 matmuls differs
    assert O.rel_frobenius(part.float(), full[sample].float()) < 1e-3
