"""GPU acceptance tests of ``InferenceMoE``: the assertions of the reference's
``tests/test_inference.py`` restated against this implementation, plus parity
with the quantization-aware CPU oracle.
"""

import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

LAYER_REL_TOL = 2e-2  # relative Frobenius error vs the quantization-aware layer oracle


def _weights(experts, hidden, inter, seed, unary=False, scale=None):
    g = torch.Generator().manual_seed(seed)
    s1 = hidden**-0.5 if scale is None else scale
    s2 = inter**-0.5 if scale is None else scale
    first = (torch.randn(experts, inter, hidden, generator=g) * s1).to(torch.bfloat16)
    second = None if unary else (torch.randn(experts, inter, hidden, generator=g) * s1).to(torch.bfloat16)
    down = (torch.randn(experts, hidden, inter, generator=g) * s2).to(torch.bfloat16)
    return first, second, down


def _routing(tokens, experts, k, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(tokens, experts, generator=g)
    topv, topi = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    topv = (topv / topv.sum(-1, keepdim=True)).float().contiguous()
    return topi.to(torch.int32).contiguous(), topv


def _oracle_layer(x, ids, w, first, second, down, activation, clamp, alpha, bias, x_scale, h_scale):
    w1 = O.pack_weights(first if second is None else O.interleave_gate_up(first, second))
    w2 = O.pack_weights(down)
    return O.moe_layer(x, ids, w, *w1, *w2, x_scale, h_scale, activation, clamp, alpha, bias,
                       return_stages=True)


@pytest.mark.parametrize(
    ("activation", "clamp"),
    (("swiglu", None), ("swiglu_oai", None), ("relu2", None), ("swiglu", 10.0), ("geglu", None),
     ("reglu", None)),
)
def test_prefill_layer_matches_oracle_and_bf16_reference(activation, clamp):
    from nvfp4moe_b200 import InferenceMoE

    tokens, hidden, inter, experts, k = 300, 512, 256, 8, 2
    unary = activation == "relu2"
    first, second, down = _weights(experts, hidden, inter, 20260825, unary)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    ids, w = _routing(tokens, experts, k, 2)
    ids[ids == 5] = 4  # expert 5 receives nothing
    plan = InferenceMoE(hidden, inter, experts, k, tokens, activation=activation,
                        activation_clamp=clamp)
    if unary:
        plan.load_weights(first.cuda(), down.cuda())
    else:
        plan.load_weights(first.cuda(), second.cuda(), down.cuda())
    plan.calibrate(x.cuda(), ids.cuda(), w.cuda())
    out = plan.run_prefill(x.cuda(), ids.cuda(), w.cuda()).clone()
    torch.cuda.synchronize()

    x_scale = plan._x_scale[:1].cpu()
    h_scale = plan._h_scale[:1].cpu()
    ref, stages = _oracle_layer(x, ids, w, first, second, down, activation, plan.activation_clamp,
                                plan.activation_sigmoid_alpha, plan.activation_up_bias, x_scale,
                                h_scale)
    rows = tokens * k
    # integer stages are bit-exact
    assert torch.equal(plan._gather[:rows].cpu(), stages["gather"])
    assert torch.equal(plan._m_indptr.cpu(), stages["m_indptr"])
    assert torch.equal(plan._slots[:rows].cpu(), stages["slots"])
    assert torch.equal(plan._probs[:rows].cpu(), stages["probs"])
    assert torch.equal(plan._padded_offsets.cpu(), stages["padded_offsets"])
    # calibration reproduces the oracle's scales to FP32 rounding of the BF16 pre-activation
    xs_ref, hs_ref = O.calibrate(x, ids, w, *O.pack_weights(
        first if unary else O.interleave_gate_up(first, second)), activation,
        plan.activation_clamp, plan.activation_sigmoid_alpha, plan.activation_up_bias)
    assert abs(float(x_scale) / float(xs_ref) - 1.0) < 3e-7  # GPU divide-by-constant: one ulp
    assert abs(float(h_scale) / float(hs_ref) - 1.0) < 2e-2
    # floating-point result
    assert torch.isfinite(out).all()
    assert O.rel_frobenius(out.cpu().float(), ref.float()) <= LAYER_REL_TOL
    bf16 = O.bf16_layer(x, ids, w, first, second, down, activation, plan.activation_clamp,
                        plan.activation_sigmoid_alpha, plan.activation_up_bias)
    assert O.cosine(out.cpu().float(), bf16) > 0.95


def test_inference_plan_is_repeatable_allocation_free_and_graph_safe():
    from nvfp4moe_b200 import InferenceMoE

    tokens, hidden, inter, experts, k = 17, 256, 128, 4, 2
    gate, up, down = (t.cuda() for t in _weights(experts, hidden, inter, 20260819))
    g = torch.Generator().manual_seed(3)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda()
    ids = torch.tensor([[0, 1], [1, 0]] * 8 + [[0, 1]], dtype=torch.int32, device="cuda")
    w = torch.rand(tokens, k, generator=g)
    w = (w / w.sum(1, keepdim=True)).cuda()

    plan = InferenceMoE(hidden, inter, experts, k, tokens)
    assert plan._qx_u8.data_ptr() == plan._routed_out.data_ptr()
    assert plan._qh_u8.data_ptr() == plan._out.data_ptr()
    plan.load_weights(gate, up, down)
    plan.calibrate(x, ids, w)
    plan.warmup(x, ids, w)

    first = plan(x, ids, w).clone()
    prefill = plan.run_prefill(x, ids, w).clone()
    plan._sfh.view(torch.uint8).fill_(0)
    second = plan(x, ids, w).clone()
    torch.cuda.synchronize()
    assert torch.equal(first, second)
    assert torch.equal(first, prefill)

    before = torch.cuda.memory_allocated()
    ptr = plan(x, ids, w).data_ptr()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert ptr == plan.output.data_ptr()

    x_original = x.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = plan(x, ids, w)
    graph.replay()
    graph_first = captured.clone()
    assert torch.equal(graph_first, first)
    x.mul_(0.5)
    graph.replay()
    torch.cuda.synchronize()
    assert not torch.equal(graph_first, captured)
    x.copy_(x_original)

    ref = O.bf16_layer(x.cpu(), ids.cpu(), w.cpu(), gate.cpu(), up.cpu(), down.cpu())
    assert O.cosine(first.cpu().float(), ref) > 0.95


def test_routed_and_full_paths_match():
    from nvfp4moe_b200 import InferenceMoE
    from nvfp4moe_b200.kernels.routing.combine import moe_finalize

    tokens, hidden, inter, experts, k = 8, 256, 128, 4, 2
    gate, up, down = (t.cuda() for t in _weights(experts, hidden, inter, 20260820, scale=1.0))
    g = torch.Generator().manual_seed(4)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda()
    ids = torch.tensor([[0, 1], [1, 2], [2, 0], [0, 2]] * 2, device="cuda").int()
    w = torch.full((tokens, k), 0.5, device="cuda")
    plan = InferenceMoE(hidden, inter, experts, k, tokens)
    plan.load_weights(gate, up, down)
    plan.calibrate(x, ids, w)
    full = plan(x, ids, w).clone()
    rows = tokens * k
    routed_x = x.index_select(0, plan._gather[:rows].long())
    routed_y = plan.run_routed(routed_x, plan._m_indptr, plan._padded_offsets).clone()
    combined = torch.empty_like(full)
    moe_finalize(routed_y, plan._slots[:rows], combined, k, tile_t=2, n_frag=2,
                 weights=plan._probs[:rows])
    torch.cuda.synchronize()
    assert torch.equal(full, combined)


def test_batch_one_decode_matches_prefill():
    from nvfp4moe_b200 import InferenceMoE

    hidden, inter, experts, k = 256, 128, 4, 2
    gate, up, down = (t.cuda() for t in _weights(experts, hidden, inter, 20260822, scale=1.0))
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1, hidden, generator=g).to(torch.bfloat16).cuda()
    ids = torch.tensor([[1, 3]], dtype=torch.int32, device="cuda")
    w = torch.tensor([[0.625, 0.375]], dtype=torch.float32, device="cuda")
    plan = InferenceMoE(hidden, inter, experts, k, 1)
    plan.load_weights(gate, up, down)
    plan.calibrate(x, ids, w)
    decode = plan.run_decode(x, ids, w).clone()
    prefill = plan.run_prefill(x, ids, w).clone()
    torch.cuda.synchronize()
    assert torch.equal(decode, prefill)
    assert torch.equal(plan._gather[:k], torch.tensor([0, 0], device="cuda").int())
    assert torch.equal(plan._m_indptr, torch.tensor([0, 0, 1, 1, 2], device="cuda").int())


def test_clamped_swiglu_matches_across_decode_and_prefill():
    from nvfp4moe_b200 import InferenceMoE

    tokens, hidden, inter, experts, k = 8, 256, 128, 4, 2
    gate, up, down = (t.cuda() for t in _weights(experts, hidden, inter, 20260824, scale=1.0))
    g = torch.Generator().manual_seed(6)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda()
    ids = torch.tensor([[0, 1], [1, 2], [2, 3], [3, 0]] * 2, device="cuda").int()
    w = torch.full((tokens, k), 0.5, device="cuda")
    clamped = InferenceMoE(hidden, inter, experts, k, tokens, activation_clamp=10.0)
    unclamped = InferenceMoE(hidden, inter, experts, k, tokens)
    for plan in (clamped, unclamped):
        plan.load_weights(gate, up, down)
        plan.set_activation_scales(1.0, 1.0)
    decode = clamped.run_decode(x, ids, w).clone()
    prefill = clamped.run_prefill(x, ids, w).clone()
    plain = unclamped.run_prefill(x, ids, w).clone()
    torch.cuda.synchronize()
    assert torch.equal(decode, prefill)
    assert not torch.equal(prefill, plain)


@pytest.mark.parametrize("routing", ("balanced", "single_expert_skew"))
def test_fast_decode_plan_matches_prefill(routing):
    from nvfp4moe_b200 import InferenceMoE

    tokens, hidden, inter, experts, k = 8, 2048, 128, 16, 2
    gate, up, down = (t.cuda() for t in _weights(experts, hidden, inter, 20260823, scale=1.0))
    g = torch.Generator().manual_seed(7)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda()
    token = torch.arange(tokens, dtype=torch.int32, device="cuda")[:, None]
    route = torch.arange(k, dtype=torch.int32, device="cuda")[None, :]
    ids = ((token * k + route) % experts).contiguous()
    if routing == "single_expert_skew":
        ids = route.expand(tokens, -1).contiguous()
    w = torch.rand(tokens, k, generator=g)
    w = (w / w.sum(1, keepdim=True)).cuda()
    plan = InferenceMoE(hidden, inter, experts, k, tokens)
    plan.load_weights(gate, up, down)
    plan.set_activation_scales(1.0, 1.0)
    decode = plan.run_decode(x, ids, w).clone()
    prefill = plan.run_prefill(x, ids, w).clone()
    torch.cuda.synchronize()
    assert plan._full_execution(tokens, decode=True).fc1.fast_decode_sched
    assert torch.equal(decode, prefill)


def test_large_plans_with_sparse_routing_share_a_workspace():
    from nvfp4moe_b200 import InferenceMoE
    from nvfp4moe_b200.inference import InferenceWorkspace

    tokens, hidden, inter, experts, k = 1024, 2048, 768, 128, 8
    active_sets = ((40, 45, 65, 73, 98, 99, 100, 114), (10, 64, 70, 94, 108, 111, 120, 125))
    g = torch.Generator().manual_seed(8)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda()
    w = torch.full((tokens, k), 1 / k, device="cuda")
    fc1 = torch.randint(256, (experts, 2 * inter, hidden // 2), dtype=torch.uint8, device="cuda")
    fc2 = torch.randint(256, (experts, hidden, inter // 2), dtype=torch.uint8, device="cuda")
    sf1 = torch.ones(experts, 2 * inter // 128, hidden // 64, 32, 4, 4, device="cuda").to(torch.float8_e4m3fn)
    sf2 = torch.ones(experts, hidden // 128, inter // 64, 32, 4, 4, device="cuda").to(torch.float8_e4m3fn)
    scale = torch.ones(experts, dtype=torch.float32, device="cuda")
    workspace = InferenceWorkspace.allocate(hidden, inter, experts, k, tokens,
                                            torch.device("cuda", torch.cuda.current_device()))
    plans = []
    for _ in active_sets:
        plan = InferenceMoE(hidden, inter, experts, k, tokens, workspace=workspace)
        plan.load_packed_weights(fc1.view(torch.float4_e2m1fn_x2), sf1, scale,
                                 fc2.view(torch.float4_e2m1fn_x2), sf2, scale)
        plan.set_activation_scales(1.0, 1.0)
        plans.append(plan)
    assert all(plan.workspace is workspace for plan in plans)
    for plan, active in zip(plans, active_sets):
        ids = torch.tensor(active, dtype=torch.int32, device="cuda").repeat(tokens, 1)
        out = plan(x, ids, w)
        torch.cuda.synchronize()
        assert int(plan._gather[: tokens * k].min()) == 0
        assert int(plan._gather[: tokens * k].max()) == tokens - 1
        assert torch.isfinite(out).all()
    decode_tokens = 64
    token = torch.arange(decode_tokens, dtype=torch.int32, device="cuda")[:, None]
    route = torch.arange(k - 1, dtype=torch.int32, device="cuda")[None, :]
    other = ((token * (k - 1) + route) % (experts - 1)) + 1
    ids = torch.cat((torch.zeros(decode_tokens, 1, dtype=torch.int32, device="cuda"), other), 1).contiguous()
    dw = torch.full((decode_tokens, k), 1 / k, dtype=torch.float32, device="cuda")
    decode = plans[0].run_decode(x[:decode_tokens], ids, dw)
    torch.cuda.synchronize()
    assert torch.isfinite(decode).all()


def test_decode_equals_prefill_up_to_the_row_threshold():
    """run() switches to the decode path at rows <= 16 * experts; both paths agree bitwise."""
    from nvfp4moe_b200 import InferenceMoE

    hidden, inter, experts, k = 256, 128, 8, 2
    gate, up, down = (t.cuda() for t in _weights(experts, hidden, inter, 99))
    plan = InferenceMoE(hidden, inter, experts, k, 80)
    plan.load_weights(gate, up, down)
    plan.set_activation_scales(0.01, 0.01)
    for tokens in (1, 2, 7, 33, 64, 65, 80):
        g = torch.Generator().manual_seed(tokens)
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda()
        ids, w = _routing(tokens, experts, k, tokens)
        decode = plan.run_decode(x, ids.cuda(), w.cuda()).clone()
        prefill = plan.run_prefill(x, ids.cuda(), w.cuda()).clone()
        torch.cuda.synchronize()
        assert torch.equal(decode, prefill), tokens


def test_no_kernel_reported_a_timed_out_wait():
    from nvfp4moe_b200 import _lib

    assert _lib.device_status() == 0


def test_expert_parallel_layer_on_one_rank_equals_the_plain_layer():
    """With a single rank the exchange is the identity: same bits as InferenceMoE."""
    from nvfp4moe_b200 import InferenceMoE
    from nvfp4moe_b200.expert_parallel import ExpertParallelMoE

    tokens, hidden, inter, experts, k = 200, 256, 128, 8, 2
    gate, up, down = (t.cuda() for t in _weights(experts, hidden, inter, 123))
    g = torch.Generator().manual_seed(9)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda()
    ids, w = _routing(tokens, experts, k, 10)
    ids, w = ids.cuda(), w.cuda()
    plain = InferenceMoE(hidden, inter, experts, k, tokens)
    plain.load_weights(gate, up, down)
    plain.calibrate(x, ids, w)
    expected = plain.run_prefill(x, ids, w).clone()
    sharded = ExpertParallelMoE(hidden, inter, experts, k, tokens)
    sharded.load_weights(gate, up, down)
    sharded.set_activation_scales(plain._x_scale[:1], plain._h_scale[:1])
    got = sharded(x, ids, w).clone()
    again = sharded(x, ids, w).clone()
    torch.cuda.synchronize()
    assert torch.equal(got, expected)
    assert torch.equal(got, again)


def test_host_pipeline_matches_direct_steps():
    """Overlapped host-buffer steps give the bits of plain device steps, batch by batch."""
    from nvfp4moe_b200 import HostPipeline, InferenceMoE

    hidden, inter, experts, k, tokens = 256, 128, 8, 2, 192
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(99)
    layer = InferenceMoE(hidden, inter, experts, k, tokens, device=dev)
    layer.load_weights((torch.randn(experts, inter, hidden, generator=g) * 0.05).to(torch.bfloat16).to(dev),
                       (torch.randn(experts, inter, hidden, generator=g) * 0.05).to(torch.bfloat16).to(dev),
                       (torch.randn(experts, hidden, inter, generator=g) * 0.05).to(torch.bfloat16).to(dev))
    batches = []
    for _ in range(5):
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).pin_memory()
        scores = torch.rand(tokens, experts, generator=g)
        w, ids = scores.topk(k, dim=-1)
        batches.append((x, ids.to(torch.int32).pin_memory(), (w / w.sum(-1, keepdim=True)).pin_memory(),
                        torch.zeros(tokens, hidden, dtype=torch.bfloat16).pin_memory()))
    layer.calibrate(batches[0][0].to(dev), batches[0][1].to(dev), batches[0][2].to(dev))
    direct = [layer.run(x.to(dev), ids.to(dev), w.to(dev)).clone().cpu() for x, ids, w, _ in batches]
    pipe = HostPipeline(layer, tokens, hidden, k, depth=2, device=dev)
    tickets = [pipe.submit(*batch) for batch in batches]
    assert tickets == list(range(5))
    pipe.wait(tickets[1])
    assert torch.equal(batches[1][3], direct[1])
    pipe.wait()
    for batch, ref in zip(batches, direct):
        assert torch.equal(batch[3], ref)
    with pytest.raises(ValueError, match="pinned"):
        pipe.submit(batches[0][0].clone(), *batches[0][1:])
    with pytest.raises(ValueError, match="unknown ticket"):
        pipe.wait(99)


def test_packed_weights_with_per_expert_scales():
    """Checkpoint-style weights: every expert packed on its own FP32 scale, passed as (E,)
    tensors to ``load_packed_weights`` (reference ``inference.py:398-469``)."""
    from nvfp4moe_b200 import InferenceMoE

    tokens, hidden, inter, experts, k = 160, 256, 128, 6, 2
    first, second, down = _weights(experts, hidden, inter, 31)
    # make the experts' magnitudes differ so that a shared scale would not do
    gain = torch.tensor([0.25, 1.0, 4.0, 0.5, 2.0, 8.0]).view(experts, 1, 1)
    first, second, down = (first.float() * gain).to(torch.bfloat16), (second.float() * gain).to(torch.bfloat16), \
        (down.float() * gain).to(torch.bfloat16)
    gate_up = O.interleave_gate_up(first, second)
    packed1 = [O.pack_weights(gate_up[e : e + 1]) for e in range(experts)]
    packed2 = [O.pack_weights(down[e : e + 1]) for e in range(experts)]
    q1 = torch.cat([p[0] for p in packed1]); sf1 = torch.cat([p[1] for p in packed1])
    s1 = torch.cat([torch.as_tensor(p[2], dtype=torch.float32).reshape(1) for p in packed1])
    q2 = torch.cat([p[0] for p in packed2]); sf2 = torch.cat([p[1] for p in packed2])
    s2 = torch.cat([torch.as_tensor(p[2], dtype=torch.float32).reshape(1) for p in packed2])
    assert float(s1.max() / s1.min()) > 8.0

    g = torch.Generator().manual_seed(32)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    ids, w = _routing(tokens, experts, k, 33)
    x_scale, h_scale = torch.tensor([2.0e-3]), torch.tensor([4.0e-3])
    ref = O.moe_layer(x, ids, w, q1, sf1, s1, q2, sf2, s2, x_scale, h_scale)

    def blocked(sf, rows, cols):  # (E, rows, cols/16) bytes -> the (E, rows/128, cols/64, 32, 4, 4) weight layout
        return torch.stack([O.sf_to_blocked(sf[e]) for e in range(experts)]).view(
            experts, -(-rows // 128), cols // 64, 32, 4, 4)

    dev = torch.device("cuda", 0)
    plan = InferenceMoE(hidden, inter, experts, k, tokens, device=dev)
    plan.load_packed_weights(q1.to(dev).view(torch.float4_e2m1fn_x2), blocked(sf1, 2 * inter, hidden).to(dev).view(torch.float8_e4m3fn),
                             s1.to(dev), q2.to(dev).view(torch.float4_e2m1fn_x2),
                             blocked(sf2, hidden, inter).to(dev).view(torch.float8_e4m3fn), s2.to(dev))
    plan.set_activation_scales(x_scale.to(dev), h_scale.to(dev))
    out = plan.run(x.to(dev), ids.to(dev), w.to(dev)).cpu()
    assert torch.isfinite(out).all()
    assert O.rel_frobenius(out.float(), ref.float()) <= LAYER_REL_TOL
