"""Size-independent properties at the benchmark's full layer size (384 experts, hidden 4096,
inter 2048, top-6): the CPU oracle would need minutes per token there, so the full-size runs are
checked through exact identities instead, and a few tokens of them against the oracle."""

import numpy as np
import pytest
import torch

from oracle import e8, router as oracle_router

pytestmark = pytest.mark.gpu
EXPERTS, HIDDEN, INTER, TOP_K = 384, 4096, 2048, 6


@pytest.fixture(scope="module")
def full_layer(cuda):
    from keep_b200 import moe

    gen = torch.Generator(device=cuda)
    gen.manual_seed(0)

    def proj(out, inp):
        codes = torch.randint(0, 1 << 16, (EXPERTS, out, inp // 8), generator=gen, device=cuda, dtype=torch.int32).to(torch.uint16)
        scales = (0.02 * (0.5 + torch.rand((EXPERTS, out, 1), generator=gen, device=cuda))).to(torch.float16)
        return moe.Projection(codes, scales)

    router = (0.02 * torch.randn((EXPERTS, HIDDEN), generator=gen, device=cuda)).to(torch.bfloat16)
    return moe.RoutedMoELayer(router, proj(INTER, HIDDEN), proj(INTER, HIDDEN), proj(HIDDEN, INTER), top_k=TOP_K)


def tokens(cuda, count, seed):
    gen = torch.Generator().manual_seed(seed)
    return torch.randn((count, HIDDEN), generator=gen).to(torch.bfloat16).to(cuda)


def test_token_order_and_batch_split_do_not_change_a_token(cuda, full_layer):
    """A token's output depends on nothing but the token: permuting the batch permutes the outputs
    bit for bit, and two half batches give the same rows as the whole batch (route grouping, item
    order and activation staging differ between those calls; the arithmetic per route may not)."""
    x = tokens(cuda, 64, 1)
    whole = full_layer.decode(x)[0].clone()
    perm = torch.randperm(64, generator=torch.Generator().manual_seed(2)).to(cuda)
    assert torch.equal(full_layer.decode(x[perm])[0], whole[perm])
    halves = torch.cat([full_layer.decode(x[:32].contiguous())[0].clone(), full_layer.decode(x[32:].contiguous())[0].clone()])
    assert torch.equal(halves, whole)


def test_prefill_and_decode_kernels_agree_on_every_token(cuda, full_layer):
    """4096 tokens run the tcgen05 kernels, 64 of them alone the mma.sync kernels: both compute
    exact integer products of the same quantised activations, so the rows match to the last bit
    that the different summation of the two fp32 partials per row leaves (at most one bf16 step)."""
    x = tokens(cuda, 4096, 3)
    big, routing = full_layer.decode(x)
    big = big.clone()
    assert not full_layer.wait_expired(4096, x.dtype)
    picks = routing.served_expert.cpu().numpy().astype(np.int64)
    assert (picks >= 0).all() and np.bincount(picks.reshape(-1), minlength=EXPERTS).max() >= 64
    small = full_layer.decode(x[:64].contiguous())[0]
    a, b = big[:64].float(), small.float()
    assert e8.relative_gap(a.cpu().numpy(), b.cpu().numpy()) <= 2 ** -7
    assert (a - b).abs().max() <= 2 ** -7 * b.abs().max()


def test_sorted_route_operator_is_linear_in_the_activations(cuda, full_layer):
    """Doubling the activations doubles every output exactly (the activation step is a power of
    two, everything after it is integer arithmetic and one scaling), and the sum of two calls on
    orthogonal halves of the hidden dimension equals the call on the whole vector up to fp32 rounding."""
    from keep_b200 import prefill, vq

    rng = np.random.default_rng(4)
    routes = 2048
    rhs = torch.from_numpy(np.sort(rng.integers(0, 16, routes)).astype(np.int32)).to(cuda)  # 128 routes per expert: tcgen05
    x = torch.randn((routes, HIDDEN), generator=torch.Generator().manual_seed(5)).to(cuda)
    table = vq.table_on(cuda, "e8p")
    w1 = full_layer.w1
    f = lambda rows: prefill.tensor_core_projection(rows, w1.codes, w1.scales, table, rhs).clone()  # noqa: E731
    y = f(x)
    assert y is not None and torch.equal(f(2.0 * x), 2.0 * y)
    lo, hi = x.clone(), x.clone()
    lo[:, HIDDEN // 2:] = 0
    hi[:, : HIDDEN // 2] = 0
    assert e8.relative_gap((f(lo) + f(hi)).cpu().numpy(), y.cpu().numpy()) <= 1e-4


def test_a_few_full_size_tokens_against_the_oracle(cuda, full_layer):
    """Three tokens of the 64-token call, checked against the CPU oracle (18 experts decoded)."""
    x = tokens(cuda, 64, 1)
    out, routing = full_layer.decode(x)
    rows = [0, 31, 63]
    router_w = full_layer.router_w.cpu()
    want = oracle_router.routed_topk(x[rows].cpu(), router_w, None, None, None, top_k=TOP_K)
    assert oracle_router.min_cut_gap(want["served_keys"], TOP_K) > 0
    np.testing.assert_array_equal(routing.served_expert[rows].cpu().numpy(), want["served_expert"].numpy())
    slots = want["served_slot"].numpy()
    dense = {}
    for name, p in (("w1", full_layer.w1), ("w3", full_layer.w3), ("w2", full_layer.w2)):
        wanted = sorted({int(v) for v in slots.reshape(-1)})
        codes = np.stack([p.codes[e].cpu().numpy() for e in wanted])
        scales = np.stack([p.scales[e].cpu().numpy() for e in wanted])
        dense[name] = {e: w for e, w in zip(wanted, oracle_router.dense_slots(codes, scales, range(len(wanted))).values())}
    ref = oracle_router.moe_layer(x[rows].cpu(), slots, want["served_weight"].numpy(), dense["w1"], dense["w3"], dense["w2"])
    gap = e8.relative_gap(out[rows].float().cpu().numpy(), ref.numpy())
    assert gap <= 1e-2, gap
