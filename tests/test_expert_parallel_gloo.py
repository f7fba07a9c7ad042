"""Dispatch / combine index arithmetic of expert parallelism on two CPU ranks (gloo), on the torch
restatement of the exchange (``ep_reference.py``) that the GPU tests check the kernels against.

The experts themselves are a stand-in (a seeded linear map per expert), so what is checked is the
exchange: every route reaches the rank that owns its expert, carries the right hidden state and
weight, and comes back to the right token and pick."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

WORLD, EXPERTS, HIDDEN, TOP_K, TOKENS = 2, 6, 16, 3, 5


def expert_matrix(e):
    return torch.from_numpy(np.random.default_rng(100 + e).normal(size=(HIDDEN, HIDDEN)).astype(np.float32))


def reference(x, served_expert, served_weight):
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(served_expert.shape[1]):
            e = int(served_expert[t, j])
            if e >= 0:
                out[t] += (expert_matrix(e) @ x[t]) * served_weight[t, j]
    return out


def worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        import sys
        from pathlib import Path

        sys.path.insert(0, str(Path(__file__).resolve().parent))
        from ep_reference import NO_SLOT, TorchRouteExchange as RouteExchange

        rng = np.random.default_rng(10 + rank)
        x = torch.from_numpy(rng.normal(size=(TOKENS, HIDDEN)).astype(np.float32))
        served = torch.from_numpy(np.stack([rng.choice(EXPERTS, TOP_K, replace=False) for _ in range(TOKENS)]).astype(np.int64))
        served[1, 2] = -1  # a dead pick travels nowhere
        weight = torch.from_numpy(rng.uniform(0.1, 1.0, size=(TOKENS, TOP_K)).astype(np.float32))
        per_rank = EXPERTS // WORLD
        exchange = RouteExchange(per_rank)
        recv_x, recv_slot, recv_weight, position = exchange.dispatch(x, served, weight)
        assert recv_x.shape[0] == WORLD * TOKENS * TOP_K
        live = recv_slot != NO_SLOT
        assert int(live.sum()) > 0 and (recv_slot[live] < per_rank).all()
        y = torch.zeros_like(recv_x)
        for r in torch.nonzero(live).reshape(-1).tolist():  # this rank's experts on the routes it received
            y[r] = (expert_matrix(rank * per_rank + int(recv_slot[r])) @ recv_x[r]) * recv_weight[r]
        out = exchange.combine(y, position, torch.float32)
        want = reference(x, served, weight)
        results[rank] = float((out - want).abs().max() / want.abs().max())
        # every live route got a distinct position; the dead one none
        pos = position.reshape(-1)
        dump = WORLD * TOKENS * TOP_K
        assert int((pos == dump).sum()) == 1 and len(set(pos[pos != dump].tolist())) == TOKENS * TOP_K - 1
    finally:
        dist.destroy_process_group()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_rank_dispatch_and_combine_match_the_single_process_sum():
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(rank, port, results)) for rank in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(results) == WORLD and all(gap < 1e-5 for gap in results.values()), dict(results)


def test_single_rank_plan_is_dense_and_ordered():
    from ep_reference import TorchRouteExchange

    exchange = TorchRouteExchange(4)
    served = torch.tensor([[3, 0], [1, -1], [2, 2]])
    position, capacity = exchange.plan(served)
    assert capacity == 6
    assert position.tolist() == [[0, 1], [2, 6], [3, 4]]  # 6 = the spare row of a dead pick
