"""The dispatch entry point that allocates nothing, against the regular one.

``lm_dispatch_static`` serves callers that cannot hand the library any scratch
memory (their host owns the whole GPU, or forbids allocator calls): its
per-chunk counts live in a fixed array inside the shared library.  The check
is bit-exact equality with ``lm_dispatch`` on two calls in a row -- the second
with a different shape, so whatever the first call left in the shared array
must not matter.  The file name sorts last so that a run that stops at the
first failure has already run every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _route(tokens, experts, k, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(tokens, experts, generator=g)
    logits[:, seed % experts] += 3.0
    topv, topi = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    return topi.to(torch.int32).contiguous().cuda(), topv.float().contiguous().cuda()


def _buffers(rows, experts, scratch):
    dev = "cuda"
    return dict(
        gather=torch.full((rows,), -7, dtype=torch.int32, device=dev),
        m_indptr=torch.full((experts + 1,), -7, dtype=torch.int32, device=dev),
        probs=torch.full((rows,), -7.0, dtype=torch.float32, device=dev),
        slots=torch.full((rows,), -7, dtype=torch.int32, device=dev),
        padded=torch.full((experts,), -7, dtype=torch.int32, device=dev),
        scratch=torch.full((scratch,), -7, dtype=torch.int32, device=dev),
    )


def _both(tokens, experts, k, seed, plan_tile_rows=128):
    from nvfp4moe_b200 import _lib

    lib = _lib.lib()
    ids, w = _route(tokens, experts, k, seed)
    rows = tokens * k
    n = int(lib.lm_dispatch_scratch_elems(rows, experts))
    a = _buffers(rows, experts, n)
    b = _buffers(rows, experts, n)  # b["scratch"] only receives the plan of the small path
    stream = _lib.stream_handle()
    _lib.check(lib.lm_dispatch(ids.data_ptr(), w.data_ptr(), tokens, k, experts,
                               a["gather"].data_ptr(), a["m_indptr"].data_ptr(),
                               a["probs"].data_ptr(), a["slots"].data_ptr(),
                               a["padded"].data_ptr(), a["scratch"].data_ptr(), n,
                               plan_tile_rows, stream))
    plan_ptr = b["scratch"].data_ptr() if rows <= 1024 else None
    _lib.check(lib.lm_dispatch_static(ids.data_ptr(), w.data_ptr(), tokens, k, experts,
                                      b["gather"].data_ptr(), b["m_indptr"].data_ptr(),
                                      b["probs"].data_ptr(), b["slots"].data_ptr(),
                                      b["padded"].data_ptr(), plan_ptr, n, plan_tile_rows, stream))
    torch.cuda.synchronize()
    for name in ("gather", "m_indptr", "probs", "slots", "padded"):
        assert torch.equal(a[name], b[name]), (name, tokens, experts, k)
    assert int(a["m_indptr"][-1]) == rows
    # and directly against the CPU oracle's stable sort
    from oracle import nvfp4_oracle as O

    want = O.dispatch(ids.cpu(), w.cpu(), experts, plan_tile_rows if rows <= 1024 else 128)
    for name, ref in zip(("gather", "m_indptr", "probs", "slots", "padded"), want):
        assert torch.equal(b[name].cpu(), ref), (name, tokens, experts, k)
    if rows <= 1024:
        assert torch.equal(a["scratch"], b["scratch"])  # the decode plan


def test_static_dispatch_matches_regular_dispatch_twice_in_a_row():
    _both(8192, 256, 8, seed=1)            # 64 chunks: fills much of the shared array
    _both(700, 64, 4, seed=2)              # fewer chunks, other expert count: stale counts around
    _both(64, 128, 8, seed=3, plan_tile_rows=8)   # single-block path with a decode plan
    _both(16384, 8, 8, seed=4)             # the stated maximum: 131072 assignments


def test_static_dispatch_replays_inside_a_cuda_graph():
    """The documented order of use: one plain call first (it looks up the array's device
    address), then a capture of a second call, then replays of the graph on new routing."""
    from nvfp4moe_b200 import _lib

    lib = _lib.lib()
    tokens, experts, k = 2048, 64, 4
    rows = tokens * k
    n = int(lib.lm_dispatch_scratch_elems(rows, experts))
    _both(tokens, experts, k, seed=5)  # the first call on this device, outside any capture
    ids, w = _route(tokens, experts, k, 6)
    got = _buffers(rows, experts, 1)

    def call():
        _lib.check(lib.lm_dispatch_static(ids.data_ptr(), w.data_ptr(), tokens, k, experts,
                                          got["gather"].data_ptr(), got["m_indptr"].data_ptr(),
                                          got["probs"].data_ptr(), got["slots"].data_ptr(),
                                          got["padded"].data_ptr(), None, 0, 128, _lib.stream_handle()))

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    for seed in (7, 8):
        new_ids, new_w = _route(tokens, experts, k, seed)
        ids.copy_(new_ids)
        w.copy_(new_w)
        graph.replay()
        ref = _buffers(rows, experts, n)
        _lib.check(lib.lm_dispatch(ids.data_ptr(), w.data_ptr(), tokens, k, experts,
                                   ref["gather"].data_ptr(), ref["m_indptr"].data_ptr(),
                                   ref["probs"].data_ptr(), ref["slots"].data_ptr(),
                                   ref["padded"].data_ptr(), ref["scratch"].data_ptr(), n, 128,
                                   _lib.stream_handle()))
        torch.cuda.synchronize()
        for name in ("gather", "m_indptr", "probs", "slots", "padded"):
            assert torch.equal(got[name], ref[name]), (name, seed)


def test_static_dispatch_rejects_sizes_beyond_its_scratch():
    from nvfp4moe_b200 import _lib

    lib = _lib.lib()
    assert lib.lm_dispatch_static_max_rows() == 131072
    ids, w = _route(16, 8, 2, 0)
    bufs = _buffers(32, 8, 1)
    status = lib.lm_dispatch_static(ids.data_ptr(), w.data_ptr(), 131072 // 2 + 1, 2, 8,
                                    bufs["gather"].data_ptr(), bufs["m_indptr"].data_ptr(),
                                    bufs["probs"].data_ptr(), bufs["slots"].data_ptr(),
                                    bufs["padded"].data_ptr(), None, 0, 128, _lib.stream_handle())
    assert status == 3
    assert b"exceed the built-in scratch" in lib.lm_last_error_string()
    torch.cuda.synchronize()
    assert (bufs["gather"] == -7).all()  # nothing was launched
