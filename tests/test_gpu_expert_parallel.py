"""Expert parallelism on two GPUs (NCCL): the sharded layer gives what one GPU holding every
expert gives.  Needs two devices; on a single-GPU box the test reports itself as skipped."""

import os
import socket

import numpy as np
import pytest
import torch

import synthetic

pytestmark = pytest.mark.gpu
EXPERTS, HIDDEN, INTER, TOP_K = 8, 512, 256, 3


def worker(rank, world, port, results, kind="nccl", tokens=6):
    import torch.distributed as dist

    # no NVLink multicast objects anywhere: plain peer mappings and plain NCCL rings
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
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
        exchange = None
        if kind == "peer":
            exchange = expert_parallel.PeerExchange(per_rank, tokens=tokens, top_k=TOP_K, hidden=HIDDEN, dtype=torch.bfloat16, device=device)
        layer = expert_parallel.ExpertParallelLayer(cfg["router"].to(device), local, experts_per_rank=per_rank, top_k=TOP_K, exchange=exchange)
        worst = 0.0
        for call in range(3):  # the buffers and barrier counts are reused from call to call
            x = synthetic.tokens(60 + rank + 10 * call, tokens, HIDDEN).to(device)
            got = layer.forward(x)
            want, _ = full.decode(x)
            torch.cuda.synchronize()
            ref = want.float().cpu().numpy()
            worst = max(worst, float(np.abs(got.float().cpu().numpy() - ref).max() / np.abs(ref).max()))
        if exchange is not None:
            assert not exchange.wait_expired()
        results[rank] = worst
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind,tokens", [("nccl", 6), ("peer", 6), ("peer", 200)])
def test_two_gpu_expert_parallel_matches_one_gpu(kind, tokens):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=worker, args=(rank, 2, port, results, kind, tokens)) for rank in range(2)]
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
    from ep_reference import TorchRouteExchange

    ex = expert_parallel.RouteExchange(per_rank, capacity=capacity)
    ref = TorchRouteExchange(per_rank, capacity=capacity)
    ex.world = ref.world = world                                                       # no process group: pack only
    want_x, want_slot, want_weight, want_pos = ref.pack(x, experts, weights)
    got_x, got_meta, got_pos = ex.pack_cuda(x.to(cuda), experts.to(cuda), weights.to(cuda))
    np.testing.assert_array_equal(got_pos.cpu().numpy(), want_pos.numpy())
    np.testing.assert_array_equal(got_meta[:, 0].cpu().numpy(), want_slot.numpy())
    np.testing.assert_array_equal(got_meta[:, 1].contiguous().view(torch.float32).cpu().numpy(), want_weight.numpy())
    assert torch.equal(got_x.cpu(), want_x)
    if capacity is not None:
        assert int((want_pos == world * capacity).sum()) > int((experts < 0).sum())     # the small capacity did overflow

    back = torch.randn((int(want_x.shape[0]), 512), generator=gen).to(torch.bfloat16)   # stands for the returned expert outputs
    ex.world = ref.world = 1                                                           # combine without an all-to-all
    want = ref.combine(back, want_pos, torch.bfloat16)
    got = ex.combine(back.to(cuda), got_pos, torch.bfloat16)
    assert torch.equal(got.cpu(), want)


def test_peer_barrier_gives_up_when_a_peer_never_arrives(cuda):
    """Failure detection without a fault: one GPU plays rank 0 of two, the buffers of "rank 1" are
    plain local tensors whose arrival word nothing ever sets.  The barrier polls 2000 times, sets
    the status word and returns; the context stays usable and the rows still landed."""
    from keep_b200 import _lib

    tokens, k, hidden, per_rank, world = 4, 2, 64, 3, 2
    capacity, rows = tokens * k, world * tokens * k
    gen = torch.Generator().manual_seed(5)
    x = torch.randn((tokens, hidden), generator=gen).to(torch.bfloat16).to(cuda)
    experts = torch.randint(0, world * per_rank, (tokens, k), generator=gen, dtype=torch.int32).to(cuda)
    weights = torch.rand((tokens, k), generator=gen).to(cuda)
    make = lambda shape, dt: [torch.zeros(shape, dtype=dt, device=cuda) for _ in range(world)]  # noqa: E731
    recv_x, recv_meta, back, flags = make((rows, hidden), torch.bfloat16), make((2, rows), torch.int32), make((rows, hidden), torch.bfloat16), make((32,), torch.int32)
    table = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=cuda)  # noqa: E731
    tables = [table(ts) for ts in (recv_x, recv_meta, back, flags)]
    epoch, status = torch.zeros(1, dtype=torch.int32, device=cuda), torch.zeros(1, dtype=torch.int32, device=cuda)
    position = torch.empty((tokens, k), dtype=torch.int32, device=cuda)
    arrivals = torch.zeros(1, dtype=torch.int32, device=cuda)
    peer = _lib.EpPeerArgs(world=world, rank=0, capacity=capacity, row_bytes=hidden * 2, recv_x=_lib.ptr(tables[0]), recv_meta=_lib.ptr(tables[1]),
                           back=_lib.ptr(tables[2]), flags=_lib.ptr(tables[3]), epoch=_lib.ptr(epoch), status=_lib.ptr(status), wait_spins=2000,
                           arrivals=_lib.ptr(arrivals))
    pack = _lib.EpPackArgs(x=_lib.ptr(x), row_bytes=hidden * 2, served_expert=_lib.ptr(experts), served_weight=_lib.ptr(weights), tokens=tokens,
                           top_k=k, world=world, experts_per_rank=per_rank, capacity=capacity, send_x=None, send_meta=None, position=_lib.ptr(position))
    _lib.check(_lib.load().keepvq_ep_dispatch_peer(pack, peer, _lib.stream_handle(cuda)), "keepvq_ep_dispatch_peer")
    torch.cuda.synchronize()
    assert int(status.item()) == 1 and int(epoch.item()) == 1            # gave up on rank 1, and said so
    assert int(flags[1][0].item()) == 1 and int(flags[0][0].item()) == 1  # its own arrival was announced to both
    pos = position.cpu().reshape(-1)
    for r in range(tokens * k):                                          # the rows did land where the plan says
        dest, slot = divmod(int(pos[r]), capacity)
        assert torch.equal(recv_x[dest][slot].cpu(), x[r // k].cpu())    # rank 0's block is the first of each table
        assert int(recv_meta[dest][0][slot]) == int(experts.reshape(-1)[r]) % per_rank
    assert torch.equal((x.float() * 2).cpu(), x.float().cpu() * 2)        # the context still answers
