"""A small, fixed MoE layer run for profiler captures.

    python -m nvfp4moe_b200.profile_case [hidden inter experts top_k tokens] [--decode]

Default: hidden 2048, intermediate 512, 128 experts, top-8, 4096 tokens -- the
per-expert shapes of the headline workload (256 rows per expert) at half its
size, so that operands (about 380 MB) still exceed the L2 while a profiler
replaying each launch dozens of times finishes in a minute.  Runs three
steps after loading weights with fixed activation scales.
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
    step = plan.run_decode if decode else plan.run_prefill
    for _ in range(3):
        step(x, ids, w)
    torch.cuda.synchronize()
    print("ok", float(plan.output[:tokens].float().abs().mean()))


if __name__ == "__main__":
    main(sys.argv[1:])
