"""Every BASELINE configuration at its full size against the CPU oracle.

The oracle needs minutes for a whole batch of these sizes, so each test runs the full-size
layer on the GPU and then checks
  * the integer stages of the WHOLE batch bit for bit (stable expert-major permutation,
    ``m_indptr``, slots, routing weights, padded offsets), and
  * a sample of the tokens end to end: the packed weights of the experts the sample touches
    are copied to the host and the oracle computes those tokens from the BF16 input to the
    combined output (te-math quantize -> dequantized fc1 -> activation -> requantize ->
    dequantized fc2 -> BF16 -> fixed-order weighted combine).
An output row depends on its own token only, so the sample is a direct check of the full-size
run, not of a smaller stand-in.  Tolerance: 2e-2 relative Frobenius error over the sampled
rows (FP32 summation order and the approximate exp / reciprocal of the fused epilogue are
not part of the contract).
"""

import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

LAYER_REL_TOL = 2e-2


def _build(hidden, inter, experts, k, max_tokens, activation, clamp, seed):
    from nvfp4moe_b200 import InferenceMoE

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(seed)
    plan = InferenceMoE(hidden, inter, experts, k, max_tokens, activation=activation,
                        activation_clamp=clamp, device=dev)
    gate = (torch.randn(experts, inter, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    up = (torch.randn(experts, inter, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    down = (torch.randn(experts, hidden, inter, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    plan.load_weights(gate, up, down)
    del gate, up, down
    torch.cuda.empty_cache()
    return plan, g


def _batch(tokens, hidden, experts, k, routing, g):
    from nvfp4moe_b200.bench_configs import _routing

    dev = torch.device("cuda", 0)
    x = torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16)
    ids, w = _routing(tokens, experts, k, routing, dev)
    return x, ids, w


def _host_expert_weights(plan, touched):
    """Packed weights of the touched experts with row-major scale factors, on the host."""
    n1, h = plan.qb1.shape[1], plan.hidden_size
    inter = plan.intermediate_size
    table = {}
    for e in touched:
        w1_q = plan.qb1[e].view(torch.uint8).cpu()
        w2_q = plan.qb2[e].view(torch.uint8).cpu()
        w1_sf = O.sf_from_blocked(plan.sfb1[e].view(torch.uint8).cpu(), n1, h // 16)
        w2_sf = O.sf_from_blocked(plan.sfb2[e].view(torch.uint8).cpu(), h, inter // 16)
        table[e] = (w1_q, w1_sf, w2_q, w2_sf)
    return table


def _check(plan, x, ids, w, out, sample, *, decode=False):
    from nvfp4moe_b200 import _lib

    tokens, k = ids.shape
    rows = tokens * k
    experts = plan.experts
    assert _lib.device_status() == 0
    assert torch.isfinite(out).all()
    # ---- integer stages of the whole batch, bit for bit
    if decode and tokens == 1:
        # the one-token step keeps the routes in their own order: identity slots, the expert
        # ids in place of m_indptr (lightmoe/kernels/quantize/decode.py:629-637)
        assert torch.equal(plan._slots[:rows].cpu(), torch.arange(rows, dtype=torch.int32))
        assert torch.equal(plan._m_indptr[:k].cpu(), ids[0].cpu())
        assert torch.equal(plan._probs[:rows].cpu(), w[0].cpu())
    else:
        gather, cu, probs, slots, padded, _ = O.dispatch(ids.cpu(), w.cpu(), experts)
        assert torch.equal(plan._gather[:rows].cpu(), gather)
        assert torch.equal(plan._m_indptr.cpu(), cu)
        assert torch.equal(plan._slots[:rows].cpu(), slots)
        assert torch.equal(plan._probs[:rows].cpu(), probs)
        if not decode:
            assert torch.equal(plan._padded_offsets.cpu(), padded)
    # ---- sampled tokens end to end
    sample = torch.as_tensor(sample, dtype=torch.long)
    xs, ids_s, w_s = x[sample.cuda()].cpu(), ids[sample.cuda()].cpu(), w[sample.cuda()].cpu()
    table = _host_expert_weights(plan, ids_s.unique().tolist())
    ref = O.moe_layer_sampled(xs, ids_s, w_s, table, plan.p_w1.cpu(), plan.p_w2.cpu(),
                              plan._x_scale[:1].cpu(), plan._h_scale[:1].cpu(), plan.activation,
                              plan.activation_clamp, plan.activation_sigmoid_alpha,
                              plan.activation_up_bias)
    got = out[sample.cuda()].cpu()
    rel = O.rel_frobenius(got.float(), ref.float())
    assert rel <= LAYER_REL_TOL, f"sampled rows off by {rel:.3e} (relative Frobenius)"
    # no sampled row may be far off on its own either (a wrong row hides in a Frobenius norm
    # over many rows)
    per_row = (got.float() - ref.float()).norm(dim=1) / ref.float().norm(dim=1).clamp_min(1e-20)
    assert float(per_row.max()) <= 5e-2, f"worst sampled row off by {float(per_row.max()):.3e}"
    return rel


def _spread(tokens, count):
    step = max(tokens // count, 1)
    return sorted({min(i * step + (i * 7) % step, tokens - 1) for i in range(min(count, tokens))})


def test_c2_prefill_against_oracle():
    """hidden 2048, intermediate 512, 256 experts, top-8, SwiGLU, 8192 tokens; 64 sampled tokens."""
    hidden, inter, experts, k, tokens = 2048, 512, 256, 8, 8192
    plan, g = _build(hidden, inter, experts, k, tokens, "swiglu", None, 2)
    x, ids, w = _batch(tokens, hidden, experts, k, "uniform", g)
    plan.calibrate(x, ids, w)
    out = plan.run(x, ids, w).clone()
    torch.cuda.synchronize()
    _check(plan, x, ids, w, out, _spread(tokens, 64))


def test_c3_bounded_swiglu_against_oracle():
    """hidden 4096, intermediate 2048, 256 experts, top-6, gate/up clamped at 10; 8192 and
    32768 tokens (196,608 rows in one call); 12 sampled tokens each."""
    hidden, inter, experts, k = 4096, 2048, 256, 6
    plan, g = _build(hidden, inter, experts, k, 32768, "swiglu", 10.0, 3)
    for tokens in (8192, 32768):
        x, ids, w = _batch(tokens, hidden, experts, k, "uniform", g)
        if tokens == 8192:
            plan.calibrate(x, ids, w)
        out = plan.run(x, ids, w).clone()
        torch.cuda.synchronize()
        _check(plan, x, ids, w, out, _spread(tokens, 12))


def test_c4_decode_against_oracle():
    """hidden 6144, intermediate 2048, 256 experts, top-8, SwiGLU; decode steps of 1, 8, 32 and
    64 tokens, eager and as a CUDA Graph replay; up to 8 sampled tokens per step."""
    hidden, inter, experts, k = 6144, 2048, 256, 8
    plan, g = _build(hidden, inter, experts, k, 64, "swiglu", None, 4)
    x64, ids64, w64 = _batch(64, hidden, experts, k, "uniform", g)
    plan.calibrate(x64, ids64, w64)
    for tokens in (1, 8, 32, 64):
        x, ids, w = x64[:tokens].contiguous(), ids64[:tokens].contiguous(), w64[:tokens].contiguous()
        out = plan.run(x, ids, w).clone()
        torch.cuda.synchronize()
        _check(plan, x, ids, w, out, _spread(tokens, 8), decode=True)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            plan.run(x, ids, w)
        plan.output[:tokens].zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(plan.output[:tokens], out)
        # the decode entry equals the prefill entry bit for bit
        assert torch.equal(plan.run_prefill(x, ids, w), out)


def test_c5_zipf_swiglu_oai_against_oracle():
    """hidden 6144, intermediate 3072, 128 experts, top-4, SwiGLU-OAI, 16384 tokens, Zipf(1.2)
    expert popularity: about 20 experts without a token, the top expert with 15-19 % of the
    assignments; 8 sampled tokens plus the integer stages of all 65,536 assignments."""
    hidden, inter, experts, k, tokens = 6144, 3072, 128, 4, 16384
    plan, g = _build(hidden, inter, experts, k, tokens, "swiglu_oai", None, 5)
    x, ids, w = _batch(tokens, hidden, experts, k, "zipf", g)
    counts = torch.bincount(ids.flatten().long(), minlength=experts)
    assert int((counts == 0).sum()) >= 20
    assert 0.10 <= float(counts.max()) / (tokens * k) <= 0.25
    plan.calibrate(x, ids, w)
    out = plan.run(x, ids, w).clone()
    torch.cuda.synchronize()
    # sample tokens of the hottest expert as well as evenly spread ones
    hot = int(counts.argmax())
    hot_tokens = (ids == hot).any(dim=1).nonzero().flatten()[:3].tolist()
    _check(plan, x, ids, w, out, sorted(set(_spread(tokens, 5) + hot_tokens)))
