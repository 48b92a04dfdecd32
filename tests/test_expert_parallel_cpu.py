"""Host-side logic of the expert-parallel exchange on two gloo ranks (CPU)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nvfp4moe_b200.expert_parallel import (ExpertParallelExchange, owner_splits,
                                           received_expert_ids, reference_step)

EXPERTS, TOPK, HIDDEN, TOKENS = 8, 2, 16, 24


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(rank: int):
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(TOKENS, HIDDEN, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(EXPERTS, generator=g)[:TOPK] for _ in range(TOKENS)]).int()
    if rank == 1:
        ids[ids == 6] = 7  # expert 6 gets nothing from rank 1
    w = torch.rand(TOKENS, TOPK, generator=g)
    return x, ids, w


def _expert_fn(rows: torch.Tensor, global_expert: torch.Tensor) -> torch.Tensor:
    """Stand-in for the expert GEMMs: depends on the row and on which expert ran it."""
    return (rows.float() * (global_expert.float().unsqueeze(1) + 1.0)).to(torch.bfloat16)


def _expected(x, ids, w):
    out = torch.zeros(x.shape[0], HIDDEN)
    for t in range(x.shape[0]):
        for j in range(TOPK):
            e = ids[t, j].reshape(1)
            out[t] += _expert_fn(x[t : t + 1], e)[0].float() * w[t, j]
    return out


def _worker(rank: int, world: int, port: int, scenario: str, results):
    """One gloo rank.  Scenarios (every failure is made on the host, none touches a GPU):
    ``ok``           both ranks run a step;
    ``empty``        rank 1 brings a batch of zero tokens;
    ``tamper``       rank 1 corrupts its split lists, the verified exchange must refuse on both;
    ``raise_before`` rank 1 raises before the exchange, rank 0's collective must end with an
                     error (closed connection or the group's short timeout) instead of hanging.
    """
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        exchange = ExpertParallelExchange(EXPERTS)
        assert exchange.local_experts == EXPERTS // world
        x, ids, w = _inputs(rank)
        if scenario == "empty" and rank == 1:
            x, ids, w = x[:0], ids[:0], w[:0]
        first_local = rank * exchange.local_experts

        def compute(rows, local_ids):
            return _expert_fn(rows, local_ids + first_local)

        if scenario == "raise_before" and rank == 1:
            results[rank] = "raised before the exchange"
            raise RuntimeError("injected host failure")
        tamper = None
        if scenario == "tamper" and rank == 1:
            def tamper(send, recv):
                return [send[0] + 1, send[1] - 1], recv
        try:
            out = reference_step(x, ids, w, compute, exchange, verify=scenario == "tamper", tamper=tamper)
        except RuntimeError as error:
            results[rank] = f"error: {error}"
            return
        expected = _expected(x, ids, w)
        results[rank] = bool(torch.allclose(out, expected, rtol=1e-5, atol=1e-5))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # the peer may be gone already
            pass


def _run_ranks(scenario: str, world: int = 2, limit_s: float = 120.0):
    manager = mp.Manager()
    results = manager.dict()
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(rank, world, port, scenario, results)) for rank in range(world)]
    for proc in procs:
        proc.start()
    for proc in procs:
        proc.join(limit_s)
    hung = [proc.pid for proc in procs if proc.is_alive()]
    for proc in procs:
        if proc.is_alive():
            proc.kill()
    assert not hung, f"ranks still running after {limit_s} s: a failure turned into a hang"
    return dict(results)


def test_two_rank_exchange_matches_single_process():
    assert _run_ranks("ok") == {0: True, 1: True}


def test_rank_with_zero_tokens():
    """A rank with an empty batch still takes part in every exchange and computes the rows the
    other rank routes to its experts."""
    assert _run_ranks("empty") == {0: True, 1: True}


def test_mismatched_split_sizes_are_refused_on_every_rank():
    results = _run_ranks("tamper")
    assert set(results) == {0, 1}
    for rank in (0, 1):
        assert isinstance(results[rank], str) and "split sizes disagree" in results[rank], results


def test_rank_that_raises_before_the_exchange_does_not_hang_the_others():
    results = _run_ranks("raise_before")
    assert results[1] == "raised before the exchange"
    assert isinstance(results[0], str) and results[0].startswith("error:"), results


def test_split_helpers():
    m_indptr = torch.tensor([0, 3, 3, 7, 8, 8, 10, 15, 16], dtype=torch.int32)
    assert owner_splits(m_indptr, 2).tolist() == [8, 8]
    assert owner_splits(m_indptr, 4).tolist() == [3, 5, 2, 6]
    assert owner_splits(m_indptr, 1).tolist() == [16]
    counts = torch.tensor([[2, 0, 1], [0, 3, 0]], dtype=torch.int32)
    assert received_expert_ids(counts).tolist() == [0, 0, 2, 1, 1, 1]


def test_single_rank_exchange_is_the_identity():
    exchange = ExpertParallelExchange(EXPERTS)
    assert exchange.world == 1
    x, ids, w = _inputs(0)
    out = reference_step(x, ids, w, lambda rows, e: _expert_fn(rows, e), exchange)
    assert torch.allclose(out, _expected(x, ids, w), rtol=1e-5, atol=1e-5)


def test_expert_count_must_divide_over_ranks(monkeypatch):
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 3)
    monkeypatch.setattr(dist, "get_rank", lambda group=None: 0)
    with pytest.raises(ValueError, match="divisible"):
        ExpertParallelExchange(EXPERTS)


def test_route_plan_restatement_is_a_bijection():
    """Every row a rank sends lands on exactly one owner row, and the owner's table of origins
    points back at it: the two views the peer transport derives from the gathered counts agree."""
    import random

    from oracle import nvfp4_oracle as O

    rng = random.Random(7)
    for world, experts in ((1, 4), (2, 8), (4, 16), (8, 64)):
        local = experts // world
        counts = [[rng.choice((0, 0, 1, 3, 17, 130)) for _ in range(experts)] for _ in range(world)]
        plans = [O.ep_route_plan(counts, rank) for rank in range(world)]
        for owner in range(world):
            own_indptr, _, _, origin, owner_rows = plans[owner]
            assert own_indptr[0] == 0 and own_indptr[-1] == owner_rows[owner] == len(origin)
            assert all(b >= a for a, b in zip(own_indptr, own_indptr[1:]))
        landed = {}
        for source in range(world):
            _, dest_base, owner_start, _, _ = plans[source]
            src_row = 0
            for e in range(experts):
                owner, l = divmod(e, local)
                own_indptr = plans[owner][0]
                assert owner_start[e] == own_indptr[l]
                for j in range(counts[source][e]):
                    key = (owner, dest_base[e] + j)
                    assert key not in landed
                    assert own_indptr[l] <= key[1] < own_indptr[l + 1]
                    landed[key] = (source, src_row)
                    src_row += 1
        for owner in range(world):
            for row, origin in enumerate(plans[owner][3]):
                assert landed[(owner, row)] == origin
        assert len(landed) == sum(map(sum, counts))
