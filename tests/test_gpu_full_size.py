"""BASELINE-size runs checked through size-independent properties.

The CPU oracle needs minutes for these sizes, so the full-size workloads are checked against
each other instead: the same layer computed with different tilings, through the decode entry,
sharded over virtual expert-parallel ranks, and on a subset of the tokens must agree bit for
bit (every output row depends only on its own token), and the dispatch metadata must be a
permutation consistent with the routing.  Small cases of the same code are compared with the
oracle in the other test files.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(hidden, inter, experts, k, tokens, activation="swiglu", clamp=None, seed=0):
    from nvfp4moe_b200 import InferenceMoE

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(seed)
    plan = InferenceMoE(hidden, inter, experts, k, tokens, activation=activation, activation_clamp=clamp,
                        device=dev)
    gate = (torch.randn(experts, inter, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    up = (torch.randn(experts, inter, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    down = (torch.randn(experts, hidden, inter, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    plan.load_weights(gate, up, down)
    del gate, up, down
    x = torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, generator=g, device=dev)
    topv, topi = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    ids = topi.to(torch.int32).contiguous()
    w = (topv / topv.sum(-1, keepdim=True)).float().contiguous()
    plan.calibrate(x, ids, w)
    return plan, x, ids, w


def _with_tiles(plan, tile_m, tile_n, fn):
    """Run ``fn`` with every GEMM of the plan forced to one tiling."""
    plan.tile_override = (tile_m, tile_n)
    plan._full_executions.clear()
    plan._routed_gemms.clear()
    try:
        return fn()
    finally:
        plan.tile_override = None
        plan._full_executions.clear()
        plan._routed_gemms.clear()


def test_c2_full_size_properties():
    """Config C2: hidden 2048, intermediate 512, 256 experts, top-8, 8192 tokens."""
    from nvfp4moe_b200 import _lib

    hidden, inter, experts, k, tokens = 2048, 512, 256, 8, 8192
    plan, x, ids, w = _layer(hidden, inter, experts, k, tokens)
    rows = tokens * k
    base = _with_tiles(plan, 128, 128, lambda: plan.run_prefill(x, ids, w).clone())
    assert torch.isfinite(base).all() and float(base.float().abs().mean()) > 0
    # dispatch metadata: a permutation consistent with the routing
    gather, slots, m_indptr = plan._gather[:rows], plan._slots[:rows], plan._m_indptr
    counts = torch.bincount(ids.flatten().long(), minlength=experts)
    assert torch.equal((m_indptr[1:] - m_indptr[:-1]).long(), counts)
    assert torch.equal(torch.sort(slots.long()).values, torch.arange(rows, device=slots.device))
    assert torch.equal(gather[slots.long()].long(),
                       torch.arange(rows, device=slots.device) // k)
    expert_of_row = torch.repeat_interleave(torch.arange(experts, device=slots.device), counts)
    assert torch.equal(expert_of_row[slots.long()], ids.flatten().long())
    # tilings, entry points and repetitions agree bit for bit
    for tile_m, tile_n in ((128, 256), (256, 256)):
        other = _with_tiles(plan, tile_m, tile_n, lambda: plan.run_prefill(x, ids, w).clone())
        assert torch.equal(other, base), (tile_m, tile_n)
    assert torch.equal(plan.run_prefill(x, ids, w), base)
    # a row of the output depends on its own token only: any subset of the batch gives the same rows
    half = tokens // 2
    small, xs, _, _ = _layer(hidden, inter, experts, k, half)
    small.load_packed_weights(plan.qb1, plan.sfb1, plan.p_w1, plan.qb2, plan.sfb2, plan.p_w2)
    small.set_activation_scales(plan._x_scale[:1], plan._h_scale[:1])
    part = small.run_prefill(x[half:].contiguous(), ids[half:].contiguous(), w[half:].contiguous())
    assert torch.equal(part, base[half:])
    assert _lib.device_status() == 0


def test_c3_bounded_swiglu_full_width_properties():
    """Config C3 shapes (hidden 4096, intermediate 2048, top-6, gate/up clamped at 10) on a
    32-expert shard as one rank of eight holds it, 8192 tokens' worth of rows."""
    from nvfp4moe_b200 import _lib

    hidden, inter, experts, k, tokens = 4096, 2048, 32, 6, 8192
    plan, x, ids, w = _layer(hidden, inter, experts, k, tokens, clamp=10.0, seed=3)
    base = _with_tiles(plan, 128, 128, lambda: plan.run_prefill(x, ids, w).clone())
    assert torch.isfinite(base).all()
    for tile_m, tile_n in ((128, 256), (256, 256)):
        other = _with_tiles(plan, tile_m, tile_n, lambda: plan.run_prefill(x, ids, w).clone())
        assert torch.equal(other, base), (tile_m, tile_n)
    # the routed entry point (expert-major rows given) equals the full path
    rows = tokens * k
    gathered = x.index_select(0, plan._gather[:rows].long())
    routed = plan.run_routed(gathered, plan._m_indptr, plan._padded_offsets).clone()
    plan.run_prefill(x, ids, w)
    ex = plan._full_execution(tokens, decode=False)
    assert torch.equal(routed, ex.routed_out[:rows])
    assert _lib.device_status() == 0
