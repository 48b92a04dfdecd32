"""Expert-parallel layer on two, four and eight GPUs (NCCL) against the single-GPU layer.

Every exchanged row is computed by exactly one expert with the same packed
operands and scales as on one GPU, and the combine order is fixed, so the
sharded result must equal the single-GPU result bit for bit.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu]

HIDDEN, INTER, EXPERTS, TOPK, TOKENS = 512, 256, 16, 4, 384


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case(rank: int, device):
    g = torch.Generator().manual_seed(5)
    gate = (torch.randn(EXPERTS, INTER, HIDDEN, generator=g) * HIDDEN**-0.5).to(torch.bfloat16)
    up = (torch.randn(EXPERTS, INTER, HIDDEN, generator=g) * HIDDEN**-0.5).to(torch.bfloat16)
    down = (torch.randn(EXPERTS, HIDDEN, INTER, generator=g) * INTER**-0.5).to(torch.bfloat16)
    g = torch.Generator().manual_seed(50 + rank)
    x = torch.randn(TOKENS, HIDDEN, generator=g).to(torch.bfloat16)
    logits = torch.randn(TOKENS, EXPERTS, generator=g)
    if rank == 1:
        logits[:, 3] = -1e9  # expert 3 gets nothing from rank 1
        logits[:, 9] += 3.0  # and expert 9 is hot
    topv, topi = torch.topk(torch.softmax(logits, -1), TOPK, dim=-1)
    w = (topv / topv.sum(-1, keepdim=True)).float().contiguous()
    to = lambda t: t.to(device)
    return to(gate), to(up), to(down), to(x), to(topi.int().contiguous()), to(w)


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from nvfp4moe_b200 import InferenceMoE
        from nvfp4moe_b200.expert_parallel import ExpertParallelMoE

        gate, up, down, x, ids, w = _case(rank, device)
        plain = InferenceMoE(HIDDEN, INTER, EXPERTS, TOPK, TOKENS, device=device)
        plain.load_weights(gate, up, down)
        plain.set_activation_scales(2e-3, 1e-3)
        expected = plain.run_prefill(x, ids, w).clone()

        local = EXPERTS // world
        sl = slice(rank * local, (rank + 1) * local)
        outcome = {}
        for transport in ("peer", "collective"):
            sharded = ExpertParallelMoE(HIDDEN, INTER, EXPERTS, TOPK, TOKENS, device=device,
                                        transport=transport)
            # one weight scale for the whole layer, as the single-GPU plan derives it
            sharded.local.load_packed_weights(plain.qb1[sl].contiguous(), plain.sfb1[sl].contiguous(),
                                              plain.p_w1, plain.qb2[sl].contiguous(),
                                              plain.sfb2[sl].contiguous(), plain.p_w2)
            sharded.set_activation_scales(2e-3, 1e-3)
            got = sharded(x, ids, w).clone()
            again = sharded(x, ids, w).clone()
            torch.cuda.synchronize()
            received = (int(sharded.last_recv_rows) if transport == "collective"
                        else int(sharded.local._m_indptr[-1]))
            replayed = True
            if transport == "peer":
                # the peer step is a fixed sequence of launches on every rank: capture it once,
                # replay it (the signal epochs live on the device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    captured = sharded(x, ids, w)
                for _ in range(3):
                    captured.zero_()
                    graph.replay()
                    torch.cuda.synchronize()
                    replayed = replayed and bool(torch.equal(captured, expected))
            outcome[transport] = (bool(torch.equal(got, expected)), bool(torch.equal(got, again)) and replayed,
                                  received, sharded.step_is_valid())
            dist.barrier()
        results[rank] = outcome
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", (2, 4, 8))
def test_sharded_layer_equals_single_gpu_layer(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for transport in ("peer", "collective"):
        for rank in range(world):
            equal, stable, _, valid = results[rank][transport]
            assert equal and stable and valid, (transport, rank)
        assert sum(results[rank][transport][2] for rank in range(world)) == world * TOKENS * TOPK, transport
