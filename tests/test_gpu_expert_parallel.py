"""Expert parallelism on two GPUs (NCCL): the sharded layer gives what one GPU holding every
expert gives.  Needs two devices; on a single-GPU box the test reports itself as skipped."""

import os
import socket

import numpy as np
import pytest
import torch

import synthetic

pytestmark = pytest.mark.gpu
EXPERTS, HIDDEN, INTER, TOP_K, TOKENS = 8, 512, 256, 3, 6


def worker(rank, world, port, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from keep_b200 import expert_parallel, moe

        cfg = synthetic.layer(seed=51, experts=EXPERTS, hidden=HIDDEN, inter=INTER)
        per_rank = EXPERTS // world
        lo = rank * per_rank

        def proj(name, sl):
            codes, scales = cfg[name]
            return moe.Projection(torch.from_numpy(codes[sl]).to(device), torch.from_numpy(scales[sl]).to(device))

        everything = slice(0, EXPERTS)
        full = moe.RoutedMoELayer(cfg["router"].to(device), proj("w1", everything), proj("w3", everything), proj("w2", everything), top_k=TOP_K)
        shard = slice(lo, lo + per_rank)
        local = moe.RoutedMoELayer(torch.zeros((per_rank, HIDDEN), dtype=torch.bfloat16, device=device),
                                   proj("w1", shard), proj("w3", shard), proj("w2", shard), top_k=1)
        layer = expert_parallel.ExpertParallelLayer(cfg["router"].to(device), local, experts_per_rank=per_rank, top_k=TOP_K)
        x = synthetic.tokens(60 + rank, TOKENS, HIDDEN).to(device)
        got = layer.forward(x)
        want, _ = full.decode(x)
        torch.cuda.synchronize()
        ref = want.float().cpu().numpy()
        results[rank] = float(np.abs(got.float().cpu().numpy() - ref).max() / np.abs(ref).max())
    finally:
        dist.destroy_process_group()


def test_two_gpu_expert_parallel_matches_one_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=worker, args=(rank, 2, port, results)) for rank in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    # the same kernels on the same routes: only the bf16 rounding of the final fp32 sum can differ
    assert len(results) == 2 and all(gap <= 1e-2 for gap in results.values()), dict(results)
