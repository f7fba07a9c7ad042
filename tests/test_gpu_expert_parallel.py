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


@pytest.mark.parametrize("tokens,k,world,per_rank,capacity", [(6, 3, 2, 4, None), (256, 6, 8, 48, None), (300, 6, 4, 96, 200), (1, 1, 1, 8, None)])
def test_pack_and_combine_kernels_match_the_torch_exchange(cuda, tokens, k, world, per_rank, capacity):
    """One GPU, no communication: the packing kernel builds the same send buffers and positions
    as the plain-torch exchange (stable order inside each destination's block, dead and
    overflowing routes dropped), and the pick summation gives the same rows."""
    from keep_b200 import expert_parallel

    gen = torch.Generator().manual_seed(tokens * 31 + world)
    experts = torch.randint(0, world * per_rank, (tokens, k), generator=gen, dtype=torch.int32)
    experts[torch.rand((tokens, k), generator=gen) < 0.15] = -1                       # dead picks
    weights = torch.rand((tokens, k), generator=gen)
    x = torch.randn((tokens, 512), generator=gen).to(torch.bfloat16)
    ex = expert_parallel.RouteExchange(per_rank, capacity=capacity)
    ex.world = world                                                                   # no process group: pack only
    want_x, want_slot, want_weight, want_pos = ex.pack_torch(x, experts, weights)
    got_x, got_meta, got_pos = ex.pack_cuda(x.to(cuda), experts.to(cuda), weights.to(cuda))
    np.testing.assert_array_equal(got_pos.cpu().numpy(), want_pos.numpy())
    np.testing.assert_array_equal(got_meta[:, 0].cpu().numpy(), want_slot.numpy())
    np.testing.assert_array_equal(got_meta[:, 1].contiguous().view(torch.float32).cpu().numpy(), want_weight.numpy())
    assert torch.equal(got_x.cpu(), want_x)
    if capacity is not None:
        assert int((want_pos == world * capacity).sum()) > int((experts < 0).sum())     # the small capacity did overflow

    back = torch.randn((int(want_x.shape[0]), 512), generator=gen).to(torch.bfloat16)   # stands for the returned expert outputs
    ex.world = 1                                                                       # combine without an all-to-all
    want = ex.combine(back, want_pos, torch.bfloat16)
    got = ex.combine(back.to(cuda), got_pos, torch.bfloat16)
    assert torch.equal(got.cpu(), want)
