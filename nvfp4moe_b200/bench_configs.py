"""Latency of the MoE layer and its two grouped GEMMs on the named workloads.

    python -m nvfp4moe_b200.bench_configs [name ...]
    python -m nvfp4moe_b200.bench_configs --steps 3 [--virtual-ranks] [--nvtx] name

The second form runs ``--steps`` plain steps of one workload and times nothing: the command
line a profiler wraps (the ``*_half`` workloads keep the per-expert shapes of their parents at
half the size, so that operands still exceed the L2 while a capture that replays every launch
dozens of times ends in a minute or two).  ``--virtual-ranks`` sends the batch through two
expert-parallel ranks that live in this process (peer-memory transport on one GPU); ``--nvtx``
opens an NVTX range per stage (``nvfp4moe_b200.tracing``).

Prints one JSON line per workload: median [IQR] of 21 CUDA-event samples after
warm-up (the reference's protocol, BENCHMARKS.md:19-25), layer tokens/s, and
grouped-GEMM TFLOP/s counted as 2 * rows * N * K without tile padding.  The layer
is timed as CUDA Graph replays.  Inputs are seeded synthetic draws:
activations N(0,1), router logits N(0,1) -> softmax -> top-k -> renormalise,
weights N(0,0.02) packed to NVFP4 on the GPU; the Zipf workload skews expert
popularity with exponent 1.2 over a seeded permutation of the experts.
"""

from __future__ import annotations

import json
import statistics
import sys
import time

import torch

from nvfp4moe_b200 import InferenceMoE

# name: (hidden, intermediate, experts, top_k, tokens, activation, clamp, routing, graph)
WORKLOADS = {
    "c2": (2048, 512, 256, 8, 8192, "swiglu", None, "uniform", False),
    "c3_8192": (4096, 2048, 256, 6, 8192, "swiglu", 10.0, "uniform", False),
    "c3_32768": (4096, 2048, 256, 6, 32768, "swiglu", 10.0, "uniform", False),
    "c5_zipf": (6144, 3072, 128, 4, 16384, "swiglu_oai", None, "zipf", False),
    "c4_decode_1": (6144, 2048, 256, 8, 1, "swiglu", None, "uniform", True),
    "c4_decode_8": (6144, 2048, 256, 8, 8, "swiglu", None, "uniform", True),
    "c4_decode_32": (6144, 2048, 256, 8, 32, "swiglu", None, "uniform", True),
    "c4_decode_64": (6144, 2048, 256, 8, 64, "swiglu", None, "uniform", True),
    # local expert-parallel shards the reference publishes (BENCHMARKS.md:92-97), 8192 tokens
    "shard_qwen35_35b": (2048, 512, 16, 8, 8192, "swiglu", None, "uniform", False),
    "shard_deepseek_v4_flash": (4096, 2048, 8, 6, 8192, "swiglu", 10.0, "uniform", False),
    "shard_glm_5_2": (6144, 2048, 16, 8, 8192, "swiglu", None, "uniform", False),
    "shard_minimax_m3": (6144, 3072, 8, 4, 8192, "swiglu_oai", None, "uniform", False),
    "shard_qwen35_397b": (4096, 1024, 16, 10, 8192, "swiglu", None, "uniform", False),
    "shard_nemotron_35": (2688, 1920, 8, 6, 8192, "relu2", None, "uniform", False),
    # the same shards at 1 and 128 tokens (the reference's layer table, BENCHMARKS.md:92-97)
    "shard_qwen35_35b_m1": (2048, 512, 16, 8, 1, "swiglu", None, "uniform", True),
    "shard_qwen35_35b_m128": (2048, 512, 16, 8, 128, "swiglu", None, "uniform", True),
    "shard_deepseek_v4_flash_m1": (4096, 2048, 8, 6, 1, "swiglu", 10.0, "uniform", True),
    "shard_deepseek_v4_flash_m128": (4096, 2048, 8, 6, 128, "swiglu", 10.0, "uniform", True),
    "shard_glm_5_2_m1": (6144, 2048, 16, 8, 1, "swiglu", None, "uniform", True),
    "shard_glm_5_2_m128": (6144, 2048, 16, 8, 128, "swiglu", None, "uniform", True),
    "shard_minimax_m3_m1": (6144, 3072, 8, 4, 1, "swiglu_oai", None, "uniform", True),
    "shard_minimax_m3_m128": (6144, 3072, 8, 4, 128, "swiglu_oai", None, "uniform", True),
    "shard_qwen35_397b_m1": (4096, 1024, 16, 10, 1, "swiglu", None, "uniform", True),
    "shard_qwen35_397b_m128": (4096, 1024, 16, 10, 128, "swiglu", None, "uniform", True),
    "shard_nemotron_35_m1": (2688, 1920, 8, 6, 1, "relu2", None, "uniform", True),
    "shard_nemotron_35_m128": (2688, 1920, 8, 6, 128, "relu2", None, "uniform", True),
    # half-size cases for profiler captures
    "c2_half": (2048, 512, 128, 8, 4096, "swiglu", None, "uniform", False),
    "shard_deepseek_v4_flash_half": (4096, 2048, 8, 6, 4096, "swiglu", 10.0, "uniform", False),
}


def _routing(tokens, experts, k, kind, device):
    g = torch.Generator(device=device).manual_seed(0)
    if kind == "zipf":
        perm = torch.randperm(experts, generator=g, device=device)
        popularity = torch.empty(experts, device=device)
        popularity[perm] = torch.arange(1, experts + 1, device=device, dtype=torch.float32) ** -1.2
        # the 20 least popular experts receive nothing, as in the imbalanced-routing workload
        popularity[perm[experts - 20:]] = 0.0
        popularity /= popularity.sum()
        # sampling without replacement by exponential keys: the k smallest of -log(U) / p
        keys = -torch.log(torch.rand(tokens, experts, generator=g, device=device)) / popularity
        ids = keys.topk(k, dim=1, largest=False).indices
        weights = torch.rand(tokens, k, generator=g, device=device) + 0.1
    else:
        logits = torch.randn(tokens, experts, generator=g, device=device)
        weights, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    weights = (weights / weights.sum(-1, keepdim=True)).float().contiguous()
    return ids.to(torch.int32).contiguous(), weights


def _samples(fn, count=21, warmup=5, inner=4):
    """``count`` CUDA-event samples; a sample is the mean of ``inner`` back-to-back calls, so
    that the host's launch latency is hidden behind the previous call as it is in a serving
    loop (the reference spins the GPU before each sample for the same reason)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(count):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(inner):
            fn()
        stop.record()
        stop.synchronize()
        out.append(start.elapsed_time(stop) * 1e3 / inner)
    return out


def _stats(samples):
    q = statistics.quantiles(samples, n=4)
    return {"median_us": round(statistics.median(samples), 2), "iqr_us": round(q[2] - q[0], 2),
            "min_us": round(min(samples), 2)}


def _timed(fn):
    """Two protocols.  ``median_us``: samples of four back-to-back calls (sustained clocks under
    the power cap, launch latency hidden).  ``single_us``: the reference's protocol, one call
    per sample right after an untimed call of the same kind that spins the GPU up."""
    stats = _stats(_samples(fn))

    def spun():
        fn()

    singles = []
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    for _ in range(21):
        spun()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        stop.synchronize()
        singles.append(start.elapsed_time(stop) * 1e3)
    stats["single_us"] = round(statistics.median(singles), 2)
    return stats


def build(name: str):
    """The workload's layer with random weights, calibrated on its own batch."""
    hidden, inter, experts, k, tokens, act, clamp, routing, graph = WORKLOADS[name]
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(1)
    unary = act == "relu2"
    plan = InferenceMoE(hidden, inter, experts, k, tokens, activation=act, activation_clamp=clamp,
                        device=dev)
    first = (torch.randn(experts, inter, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    down = (torch.randn(experts, hidden, inter, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    if unary:
        plan.load_weights(first, down)
    else:
        second = (torch.randn(experts, inter, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        plan.load_weights(first, second, down)
        del second
    del first, down
    torch.cuda.empty_cache()
    x = torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16)
    ids, w = _routing(tokens, experts, k, routing, dev)
    plan.calibrate(x, ids, w)
    return plan, x, ids, w


def run_steps(name: str, steps: int, virtual_ranks: bool = False) -> None:
    """``steps`` untimed steps of one workload (for profiler captures)."""
    hidden, inter, experts, k, tokens, act, clamp, _, _ = WORKLOADS[name]
    plan, x, ids, w = build(name)
    if virtual_ranks:
        from nvfp4moe_b200.expert_parallel import (ExpertParallelMoE, connect_virtual_ranks,
                                                   run_virtual_ranks)

        ranks = []
        for rank in range(2):
            shard = slice(rank * experts // 2, (rank + 1) * experts // 2)
            layer = ExpertParallelMoE(hidden, inter, experts, k, tokens, device=plan.device, rank=rank,
                                      world=2, activation=act, activation_clamp=clamp)
            layer.load_packed_weights(plan.qb1[shard].contiguous(), plan.sfb1[shard].contiguous(), plan.p_w1,
                                      plan.qb2[shard].contiguous(), plan.sfb2[shard].contiguous(), plan.p_w2)
            layer.set_activation_scales(plan._x_scale[:1], plan._h_scale[:1])
            ranks.append(layer)
        connect_virtual_ranks(ranks)
        for _ in range(steps):
            outs = run_virtual_ranks(ranks, [(x, ids, w), (x, ids, w)])
        torch.cuda.synchronize()
        print("ok", float(outs[0].float().abs().mean()))
        return
    for _ in range(steps):
        plan.run(x, ids, w)
    torch.cuda.synchronize()
    print("ok", float(plan.output[:tokens].float().abs().mean()))


# GEMM-only cases: name -> (kind, experts, rows, n, k)
GEMM_CASES = {
    # the grouped GEMM correctness case: 8 experts (two of them empty), 512 rows, N 1024, K 2048
    "c1": ("grouped", 8, 512, 1024, 2048),
    "dense_8192x4096x4096": ("dense", 1, 8192, 4096, 4096),
    "dense_8192x2048x6144": ("dense", 1, 8192, 2048, 6144),
}


def _gated(stats: dict, wall_us: float, repeat: list[float]) -> dict:
    """The reference's two validity gates (benchmarks/nvfp4_gemm.py:385-449,934-959): host wall
    time over CUDA-event time of the timed loop at most 1.5, and the medians of repeated
    measurements within 5 % of one another."""
    stats["host_wall_over_event"] = round(wall_us / max(stats["median_us"], 1e-9), 3)
    spread = (max(repeat) - min(repeat)) / max(min(repeat), 1e-9)
    stats["repeat_deviation_pct"] = round(100.0 * spread, 2)
    stats["gates_pass"] = bool(stats["host_wall_over_event"] <= 1.5 and spread <= 0.05)
    return stats


def _timed_with_gates(replay) -> dict:
    import time

    stats = _timed(replay)
    # wall clock of a loop of replays against its event time
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(50):
        replay()
    stop.record()
    stop.synchronize()
    wall_us = (time.perf_counter() - t0) * 1e6 / 50
    event_us = start.elapsed_time(stop) * 1e3 / 50
    repeats = [statistics.median(_samples(replay, count=11, warmup=2)) for _ in range(3)]
    stats = _gated(stats, wall_us * stats["median_us"] / max(event_us, 1e-9), repeats)
    return stats


def run_gemm(name: str) -> dict:
    """One GEMM of GEMM_CASES through the public ``lightmoe.gemm`` calls: TFLOP/s counted as
    2 * rows * N * K without padding."""
    from nvfp4moe_b200 import gemm

    kind, experts, rows, n, k = GEMM_CASES[name]
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)
    a = torch.randn(rows, k, generator=g, device=dev).to(torch.bfloat16)
    if kind == "dense":
        b = (torch.randn(n, k, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        qa, sfa, pa = gemm.quantize(a)
        qb, sfb, pb = gemm.quantize(b)
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
        # a caller's choice in the reference too (tile_m 128 or 256): tall tiles on CTA pairs
        # once the matrix has rows for them
        wide = n % 256 == 0
        plan = gemm.DenseGemm(n, k, 256 if (wide and rows >= 2048) else 128, 256 if wide else 128)
        plan.prepare(qa, qb, out, sfa, sfb, (pa * pb).reshape(1))
    else:
        b = (torch.randn(experts, n, k, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        counts = torch.zeros(experts, dtype=torch.int64)
        allowed = [e for e in range(experts) if e not in (3, 6)]
        picks = torch.randint(0, len(allowed), (rows,), generator=torch.Generator().manual_seed(0))
        for p in picks.tolist():
            counts[allowed[p]] += 1
        cu = torch.zeros(experts + 1, dtype=torch.int32)
        cu[1:] = counts.cumsum(0)
        qa, qb, sfa, sfb, alpha = gemm.quantize_grouped(a, b, cu.to(dev))
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
        plan = gemm.GroupedGemm(experts, n, k, 128, 256 if n % 256 == 0 else 128)
        plan.prepare(qa, qb, out, cu.to(dev), sfa, sfb, alpha)
    plan.launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        plan.launch()
    stats = _timed_with_gates(graph.replay)
    stats["tflops"] = round(2.0 * rows * n * k / (stats["median_us"] * 1e-6) / 1e12, 1)
    stats["pct_of_9000"] = round(stats["tflops"] / 90.0, 2)
    from nvfp4moe_b200 import _lib

    return {"workload": name, "kind": kind, "experts": experts, "rows": rows, "n": n, "k": k, "gemm": stats,
            "kernel": _lib.plan_info(plan._plan), "device_status": _lib.device_status()}


def run(name: str) -> dict:
    if name in GEMM_CASES:
        return run_gemm(name)
    hidden, inter, experts, k, tokens, act, clamp, routing, graph = WORKLOADS[name]
    unary = act == "relu2"
    plan, x, ids, w = build(name)
    rows = tokens * k
    counts = torch.bincount(ids.flatten().long(), minlength=experts)
    result = {"workload": name, "hidden": hidden, "intermediate": inter, "experts": experts, "top_k": k,
              "tokens": tokens, "rows": rows, "activation": act, "routing": routing,
              "empty_experts": int((counts == 0).sum()), "max_expert_share": round(float(counts.max()) / rows, 4)}
    plan.run(x, ids, w)
    torch.cuda.synchronize()
    # the layer is timed as CUDA Graph replays, like the reference's layer table
    cuda_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(cuda_graph):
        plan.run(x, ids, w)
    result["timed_as"] = "cuda graph replay"
    result["layer"] = _timed_with_gates(cuda_graph.replay)
    result["tokens_per_s"] = round(tokens / (result["layer"]["median_us"] * 1e-6))
    decode = rows <= 16 * experts
    ex = (plan._direct_execution() if (decode and tokens == 1 and k <= 32)
          else plan._full_execution(tokens, decode=decode))
    n1 = inter if unary else 2 * inter
    for label, gemm, n, kk in (("fc1", ex.fc1, n1, hidden), ("fc2", ex.fc2, hidden, inter)):
        # one launch per graph: a replay costs the host a few microseconds, a launch through the
        # Python binding 10-20, which would bound the samples of kernels shorter than that
        single = torch.cuda.CUDAGraph()
        with torch.cuda.graph(single):
            gemm.launch()
        stats = _timed(single.replay)
        stats["tflops"] = round(2.0 * rows * n * kk / (stats["median_us"] * 1e-6) / 1e12, 1)
        stats["pct_of_9000"] = round(stats["tflops"] / 90.0, 1)
        result[label] = stats
    from nvfp4moe_b200 import _lib

    result["device_status"] = _lib.device_status()
    return result


def main(argv):
    argv = list(argv)
    if "--steps" in argv:
        at = argv.index("--steps")
        steps = int(argv[at + 1])
        del argv[at : at + 2]
        virtual = "--virtual-ranks" in argv
        if "--nvtx" in argv:  # NVTX ranges around the stages, for a timeline capture
            from nvfp4moe_b200 import tracing

            tracing.enable()
        names = [a for a in argv if not a.startswith("--")]
        if len(names) != 1:
            raise SystemExit("--steps takes exactly one workload name")
        run_steps(names[0], steps, virtual)
        return
    names = argv or [n for n in list(WORKLOADS) + list(GEMM_CASES) if not n.endswith("_half")]
    for name in names:
        print(json.dumps(run(name)), flush=True)
        torch.cuda.empty_cache()
        # every workload starts from an idle GPU, as if it ran in a process of its own: right
        # after a long prefill workload the clocks stay at the power-capped level for a while,
        # and a step of 20 us measured then came out 40 % slower than the same step alone
        time.sleep(2.0)


if __name__ == "__main__":
    main(sys.argv[1:])
