"""A small, fixed MoE layer run for profiler captures.

    python -m nvfp4moe_b200.profile_case [hidden inter experts top_k tokens] [--decode] [--virtual-ranks]

Default: hidden 2048, intermediate 512, 128 experts, top-8, 4096 tokens -- the
per-expert shapes of the headline workload (256 rows per expert) at half its
size, so that operands (about 380 MB) still exceed the L2 while a profiler
replaying each launch dozens of times finishes in a minute.  Runs three
steps after loading weights with fixed activation scales.  ``--virtual-ranks``
runs the same batch through two expert-parallel ranks that live in this
process (peer-memory transport on one GPU), so that a profiler sees the route
plan, the quantize-and-send kernel, the scale-factor swizzle and the fc2 GEMM
that writes through the row-pointer table.
"""

from __future__ import annotations

import sys

import torch

from nvfp4moe_b200 import InferenceMoE


def main(argv: list[str]) -> None:
    decode = "--decode" in argv
    numbers = [int(a) for a in argv if a.lstrip("-").isdigit()]
    hidden, inter, experts, top_k, tokens = (numbers + [2048, 512, 128, 8, 4096][len(numbers):])[:5]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    gate = (torch.randn(experts, inter, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    up = (torch.randn(experts, inter, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    down = (torch.randn(experts, hidden, inter, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, generator=g, device=dev)
    topv, topi = torch.topk(torch.softmax(logits, -1), top_k, dim=-1)
    ids = topi.to(torch.int32).contiguous()
    w = (topv / topv.sum(-1, keepdim=True)).float().contiguous()
    plan = InferenceMoE(hidden, inter, experts, top_k, tokens, device=dev)
    plan.load_weights(gate, up, down)
    plan.set_activation_scales(2e-3, 2e-4)
    if "--virtual-ranks" in argv:
        from nvfp4moe_b200.expert_parallel import (ExpertParallelMoE, connect_virtual_ranks,
                                                   run_virtual_ranks)

        ranks = []
        for rank in range(2):
            shard = slice(rank * experts // 2, (rank + 1) * experts // 2)
            layer = ExpertParallelMoE(hidden, inter, experts, top_k, tokens, device=dev, rank=rank, world=2)
            layer.load_packed_weights(plan.qb1[shard].contiguous(), plan.sfb1[shard].contiguous(), plan.p_w1,
                                      plan.qb2[shard].contiguous(), plan.sfb2[shard].contiguous(), plan.p_w2)
            layer.set_activation_scales(2e-3, 2e-4)
            ranks.append(layer)
        connect_virtual_ranks(ranks)
        for _ in range(3):
            outs = run_virtual_ranks(ranks, [(x, ids, w), (x, ids, w)])
        torch.cuda.synchronize()
        print("ok", float(outs[0].float().abs().mean()))
        return
    step = plan.run_decode if decode else plan.run_prefill
    for _ in range(3):
        step(x, ids, w)
    torch.cuda.synchronize()
    print("ok", float(plan.output[:tokens].float().abs().mean()))


if __name__ == "__main__":
    main(sys.argv[1:])
