"""Peer-memory expert parallelism on ONE GPU: several virtual ranks in one process.

The kernels that move rows between ranks (route plan, quantize-and-send, the fc2 epilogue
that writes through a row-pointer table) take plain device addresses, so every rank's arena
can live on the same GPU and stream order can stand in for the cross-rank fences.  The
result of every rank must be, bit for bit, what a single GPU holding all experts computes
for that rank's tokens.
"""

import ctypes

import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _routing(tokens, experts, k, seed, skew=False):
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand(tokens, experts, generator=g)
    if skew:  # most routes go to the first quarter of the experts: one rank is overloaded
        scores[:, : experts // 4] += 0.75
    w, ids = scores.topk(k, dim=-1)
    return ids.to(torch.int32), (w / w.sum(-1, keepdim=True)).float()


def _weights(experts, hidden, inter, seed):
    g = torch.Generator().manual_seed(seed)
    return ((torch.randn(experts, inter, hidden, generator=g) * 0.05).to(torch.bfloat16),
            (torch.randn(experts, inter, hidden, generator=g) * 0.05).to(torch.bfloat16),
            (torch.randn(experts, hidden, inter, generator=g) * 0.05).to(torch.bfloat16))


@pytest.mark.parametrize("world", (1, 2, 4, 8))
def test_route_plan_matches_restatement(world):
    from nvfp4moe_b200 import _lib

    experts, row_bytes, max_rows = 16 * world if world < 8 else 64, 512, 4096
    g = torch.Generator().manual_seed(world)
    counts = torch.randint(0, 40, (world, experts), generator=g, dtype=torch.int32)
    counts[:, 3] = 0  # an expert nobody routes to
    counts[0] = 0     # a rank with no rows at all
    if world > 1:
        counts[1, 5] = 300
    local = experts // world
    bases = (ctypes.c_uint64 * world)(*[(g_ + 1) << 32 for g_ in range(world)])
    dev = torch.device("cuda", 0)
    counts_dev = counts.to(dev)
    for rank in range(world):
        own = torch.full((local + 1,), -1, dtype=torch.int32, device=dev)
        dest = torch.full((experts,), -1, dtype=torch.int32, device=dev)
        start = torch.full((experts,), -1, dtype=torch.int32, device=dev)
        ptrs = torch.zeros(max_rows, dtype=torch.int64, device=dev)
        valid = torch.zeros(1, dtype=torch.int32, device=dev)
        blocks = torch.full(((max_rows // 128 + local) * 4, 2), -9, dtype=torch.int32, device=dev)
        _lib.check(_lib.lib().lm_ep_plan(counts_dev.data_ptr(), world, rank, experts, max_rows, row_bytes,
                                         bases, own.data_ptr(), dest.data_ptr(), start.data_ptr(),
                                         ptrs.data_ptr(), blocks.data_ptr(), valid.data_ptr(),
                                         _lib.stream_handle()))
        torch.cuda.synchronize()
        own_r, dest_r, start_r, origin, owner_rows = O.ep_route_plan(counts.tolist(), rank)
        assert max(owner_rows) <= max_rows and int(valid) == 1
        assert own.tolist() == own_r
        assert dest.tolist() == dest_r
        assert start.tolist() == start_r
        expected = [((g_ + 1) << 32) + row * row_bytes for g_, row in origin]
        assert ptrs[: len(expected)].tolist() == expected
        # block table: a 32-row block of a tile is marked with (rank, first row) exactly when its
        # rows are 32 consecutive rows of one source, else -1; tiles start at atom row
        # own_indptr[l] // 128 + l
        table = blocks.cpu()
        for l in range(local):
            lo, hi = own_r[l], own_r[l + 1]
            first_tile = lo // 128 + l
            for b in range(-(-(hi - lo) // 128) * 4):
                rows = origin[lo + 32 * b : min(lo + 32 * b + 32, hi)]
                whole = (len(rows) == 32 and len({g_ for g_, _ in rows}) == 1
                         and [r for _, r in rows] == list(range(rows[0][1], rows[0][1] + 32)))
                want = [rows[0][0], rows[0][1]] if whole else [-1, 0]
                assert table[first_tile * 4 + b].tolist() == want, (rank, l, b)


def test_route_plan_flags_oversized_step():
    from nvfp4moe_b200 import _lib

    dev = torch.device("cuda", 0)
    counts = torch.tensor([[10, 20, 5, 5], [10, 30, 5, 5]], dtype=torch.int32, device=dev)
    bases = (ctypes.c_uint64 * 2)(1 << 32, 2 << 32)
    own = torch.full((3,), -1, dtype=torch.int32, device=dev)
    other = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(2)]
    ptrs = torch.zeros(64, dtype=torch.int64, device=dev)
    valid = torch.ones(1, dtype=torch.int32, device=dev)
    # rank 0 would receive 70 rows, the buffers hold 64
    _lib.check(_lib.lib().lm_ep_plan(counts.data_ptr(), 2, 1, 4, 64, 512, bases, own.data_ptr(),
                                     other[0].data_ptr(), other[1].data_ptr(), ptrs.data_ptr(), None,
                                     valid.data_ptr(), _lib.stream_handle()))
    torch.cuda.synchronize()
    assert int(valid) == 0
    assert own.tolist() == [0, 0, 0]
    assert int(ptrs.abs().sum()) == 0
    # the skipped step shows in the device status word until it is cleared
    assert _lib.device_status() & 32
    _lib.device_status_clear()
    assert _lib.device_status() == 0


@pytest.mark.parametrize(("world", "skew"), ((2, False), (4, False), (4, True), (8, False)))
def test_virtual_ranks_match_single_gpu(world, skew):
    from nvfp4moe_b200 import InferenceMoE, _lib
    from nvfp4moe_b200.expert_parallel import (ExpertParallelMoE, connect_virtual_ranks,
                                               run_virtual_ranks)

    tokens, hidden, inter, experts, k = 160, 256, 128, 16, 4
    dev = torch.device("cuda", 0)
    gate, up, down = (t.to(dev) for t in _weights(experts, hidden, inter, 5))
    batches = []
    for rank in range(world):
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(dev)
        ids, w = _routing(tokens, experts, k, 200 + rank, skew)
        batches.append((x, ids.to(dev), w.to(dev)))
    plain = InferenceMoE(hidden, inter, experts, k, tokens, device=dev)
    plain.load_weights(gate, up, down)
    plain.calibrate(*batches[0])
    expected = [plain.run_prefill(*batch).clone() for batch in batches]

    local = experts // world
    layers = []
    for rank in range(world):
        layer = ExpertParallelMoE(hidden, inter, experts, k, tokens, device=dev, rank=rank, world=world)
        shard = slice(rank * local, (rank + 1) * local)
        # one weight scale for the whole layer, as the single-GPU plan derives it
        layer.load_packed_weights(plain.qb1[shard].contiguous(), plain.sfb1[shard].contiguous(), plain.p_w1,
                                  plain.qb2[shard].contiguous(), plain.sfb2[shard].contiguous(), plain.p_w2)
        layer.set_activation_scales(plain._x_scale[:1], plain._h_scale[:1])
        layers.append(layer)
    connect_virtual_ranks(layers)
    for _ in range(2):  # the second step reuses every buffer
        outs = [out.clone() for out in run_virtual_ranks(layers, batches)]
        torch.cuda.synchronize()
        for rank in range(world):
            assert layers[rank].step_is_valid()
            assert torch.equal(outs[rank], expected[rank]), f"rank {rank} of {world}"
    assert _lib.device_status() == 0


def test_virtual_ranks_on_cta_pairs():
    """Enough rows per expert that both projections run 256 x 256 tiles on CTA pairs, fc2
    writing every row through the row-pointer table; still bit-identical to one GPU."""
    from nvfp4moe_b200 import InferenceMoE, _lib
    from nvfp4moe_b200.expert_parallel import (ExpertParallelMoE, connect_virtual_ranks,
                                               run_virtual_ranks)

    tokens, hidden, inter, experts, k, world = 1024, 256, 128, 4, 2, 2
    dev = torch.device("cuda", 0)
    gate, up, down = (t.to(dev) for t in _weights(experts, hidden, inter, 9))
    batches = []
    for rank in range(world):
        g = torch.Generator().manual_seed(300 + rank)
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(dev)
        ids, w = _routing(tokens, experts, k, 400 + rank)
        batches.append((x, ids.to(dev), w.to(dev)))
    plain = InferenceMoE(hidden, inter, experts, k, tokens, device=dev)
    plain.load_weights(gate, up, down)
    plain.calibrate(*batches[0])
    expected = [plain.run_prefill(*batch).clone() for batch in batches]
    layers = []
    for rank in range(world):
        layer = ExpertParallelMoE(hidden, inter, experts, k, tokens, device=dev, rank=rank, world=world)
        shard = slice(rank * 2, rank * 2 + 2)
        layer.load_packed_weights(plain.qb1[shard].contiguous(), plain.sfb1[shard].contiguous(), plain.p_w1,
                                  plain.qb2[shard].contiguous(), plain.sfb2[shard].contiguous(), plain.p_w2)
        layer.set_activation_scales(plain._x_scale[:1], plain._h_scale[:1])
        layers.append(layer)
    connect_virtual_ranks(layers)
    outs = [out.clone() for out in run_virtual_ranks(layers, batches)]
    torch.cuda.synchronize()
    for rank in range(world):
        fc1, fc2 = layers[rank]._peer_gemms()
        assert (fc1.tile_m, fc1.tile_n, fc2.tile_m, fc2.tile_n) == (256, 256, 256, 256)
        assert layers[rank].step_is_valid()
        assert torch.equal(outs[rank], expected[rank]), f"rank {rank}"
    assert _lib.device_status() == 0


def test_virtual_ranks_skip_an_oversized_step():
    from nvfp4moe_b200.expert_parallel import (ExpertParallelMoE, connect_virtual_ranks,
                                               run_virtual_ranks)

    tokens, hidden, inter, experts, k, world = 64, 256, 128, 8, 2, 2
    dev = torch.device("cuda", 0)
    gate, up, down = (t.to(dev) for t in _weights(experts, hidden, inter, 6))
    layers, batches = [], []
    for rank in range(world):
        # every route goes to experts 0 and 1: rank 0 would receive all 256 rows, it holds 128
        layer = ExpertParallelMoE(hidden, inter, experts, k, tokens, device=dev, rank=rank, world=world,
                                  max_recv_rows=128)
        shard = slice(rank * 4, rank * 4 + 4)
        layer.load_weights(gate[shard], up[shard], down[shard])
        layer.set_activation_scales(torch.tensor([1e-3], device=dev), torch.tensor([1e-3], device=dev))
        layers.append(layer)
        ids = torch.tensor([[0, 1]] * tokens, dtype=torch.int32, device=dev)
        w = torch.full((tokens, k), 0.5, device=dev)
        batches.append((torch.randn(tokens, hidden, device=dev).to(torch.bfloat16), ids, w))
    connect_virtual_ranks(layers)
    from nvfp4moe_b200 import _lib

    _lib.device_status_clear()
    for layer in layers:  # stale rows from an earlier step must not leak into the result
        layer._peer["ret"].fill_(7.0)
    outs = run_virtual_ranks(layers, batches)
    torch.cuda.synchronize()
    assert not layers[0].step_is_valid() and not layers[1].step_is_valid()
    assert layers[0].local._m_indptr.tolist() == [0] * 5
    # the skipped step has a defined result (zeros) and shows in the device status word
    for out in outs:
        assert not out.any()
    assert _lib.device_status() & 32
    _lib.device_status_clear()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("features", (256, 2048, 6144))
def test_sf_swizzle_matches_varlen_layout(features):
    """Row-major scale factors -> the varlen atoms the GEMM reads (zero in a tile's unused rows)."""
    from nvfp4moe_b200 import _lib

    lens = [130, 0, 257, 5, 128, 0, 64]
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens).cumsum(0)
    rows = int(cu[-1])
    g = torch.Generator().manual_seed(features)
    linear = torch.randint(1, 255, (rows + 50, features // 16), generator=g, dtype=torch.uint8)
    tiles = -(-(rows + 50) // 128) + len(lens)
    expected = O.sf_to_varlen(linear[:rows], cu, tiles)
    dev = torch.device("cuda", 0)
    atoms = torch.full((tiles, features // 64, 512), 0xEE, dtype=torch.uint8, device=dev)
    lin_dev, cu_dev = linear.to(dev), cu.to(dev)
    _lib.check(_lib.lib().lm_ep_sf_swizzle(lin_dev.data_ptr(), rows + 50, features, cu_dev.data_ptr(),
                                           len(lens), atoms.data_ptr(), _lib.stream_handle()))
    torch.cuda.synchronize()
    got = atoms.cpu().reshape(-1)
    want = expected.reshape(-1)
    # atom rows that belong to no expert tile keep the caller's bytes
    used = torch.zeros(tiles, dtype=torch.bool)
    for e, n in enumerate(lens):
        first = int(cu[e]) // 128 + e
        used[first : first + -(-n // 128)] = True
    mask = used.repeat_interleave((features // 64) * 512)
    assert torch.equal(got[mask], want[mask])
    assert bool((got[~mask] == 0xEE).all())


def test_signal_wait_runs_out_and_reports():
    """A rank whose peer never signals gives up after the limit and sets the status bit; the
    context stays usable.  (One launch on one GPU: nothing else waits on it.)"""
    from nvfp4moe_b200 import _lib

    dev = torch.device("cuda", 0)
    _lib.check(_lib.lib().lm_device_status_clear(_lib.stream_handle()))
    pads = torch.zeros(2, 64, dtype=torch.int32, device=dev)      # pad of rank 0 and of the absent rank 1
    tables = torch.zeros(2, 2, 8, dtype=torch.int32, device=dev)  # both ranks' (world, experts) tables
    m_indptr = torch.tensor([0, 3, 3, 4, 9, 9, 9, 10, 12], dtype=torch.int32, device=dev)
    sig = (ctypes.c_uint64 * 2)(pads[0].data_ptr(), pads[1].data_ptr())
    cnt = (ctypes.c_uint64 * 2)(tables[0].data_ptr(), tables[1].data_ptr())
    _lib.check(_lib.lib().lm_ep_signal(m_indptr.data_ptr(), 8, 2, 0, cnt, sig, 20, _lib.stream_handle()))
    assert _lib.device_status() == 16  # LM_STATUS_EP_TIMEOUT
    # its own part was done before the wait: counts in both tables, signals in both pads
    assert tables[0, 0].tolist() == [3, 0, 1, 5, 0, 0, 1, 2] and tables[1, 0].tolist() == tables[0, 0].tolist()
    assert int(pads[0, 0]) == 1 and int(pads[1, 0]) == 1 and int(pads[0, 1]) == 0
    _lib.check(_lib.lib().lm_device_status_clear(_lib.stream_handle()))
    assert _lib.device_status() == 0
    # once the peer's word is there the same call returns at once
    pads[0, 1] = 2
    assert int(pads[0, 2]) == 1  # the rank's own call count
    _lib.check(_lib.lib().lm_ep_signal(None, 8, 2, 0, None, sig, 20, _lib.stream_handle()))
    assert _lib.device_status() == 0
