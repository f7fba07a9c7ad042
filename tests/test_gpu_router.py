"""The CUDA router against the oracle and the reference's gate_masked outputs: selections exact,
weights to fp32 rounding."""

import numpy as np
import pytest
import torch

from oracle import router as oracle_router

pytestmark = pytest.mark.gpu


def as_sets(t):
    return [frozenset(int(v) for v in row if v >= 0) for row in np.asarray(t)]


@pytest.mark.parametrize("func", ["softmax", "sigmoid", "sqrtsoftplus"])
@pytest.mark.parametrize("mask", ["all", "masked", "few"])
def test_golden_gate_masked(cuda, golden, func, mask):
    """Per-token candidate sets, as the reference's simulator uses them: one call per token."""
    from keep_b200 import router

    g = golden("router")
    allowed = {"all": np.ones_like(g["allowed"]), "masked": g["allowed"], "few": g["few"]}[mask]
    w = torch.from_numpy(g["weight"]).to(cuda)
    want_w, want_i = g[f"{func}_{mask}_weights"], g[f"{func}_{mask}_indices"]
    for t in range(g["x"].shape[0]):
        bias = np.where(allowed[t], g["bias"], -np.inf).astype(np.float32)
        r = router.routed_topk(torch.from_numpy(g["x"][t:t + 1]).to(cuda), w, bias, g["bias"], top_k=int(g["top_k"]),
                               score_func=func, route_scale=1.5, gate_temp=1.25)
        got_i, got_w = r.served_expert.cpu().numpy()[0], r.served_weight.cpu().numpy()[0]
        live = want_w[t] > 0
        np.testing.assert_array_equal(got_i[live], want_i[t][live])
        np.testing.assert_allclose(got_w, want_w[t], rtol=2e-6, atol=1e-7)
        assert (got_i[~live] == -1).all()


@pytest.mark.parametrize("tokens,pool,hidden,k", [(1, 384, 4096, 6), (16, 384, 4096, 6), (5, 1024, 512, 8),
                                                  # 24 to 255 bf16 tokens: the tensor-core tile with K split over a cluster of eight blocks
                                                  # (ragged tiles and one K block per rank; the benchmark shape; three token tiles)
                                                  (37, 100, 256, 3), (64, 384, 4096, 6), (130, 200, 1024, 4),
                                                  # the tiled logits kernels: tensor-core, fp32, tensor-core with ragged tiles
                                                  (256, 256, 4096, 6), (303, 100, 520, 3), (300, 100, 512, 3)])
@pytest.mark.parametrize("func", ["softmax", "sqrtsoftplus"])
def test_served_demand_and_admission_match_the_oracle_exactly(cuda, tokens, pool, hidden, k, func):
    from keep_b200 import router

    rng = np.random.default_rng(1000 + tokens + pool)
    w = torch.from_numpy(rng.normal(scale=0.02, size=(pool, hidden)).astype(np.float32)).to(torch.bfloat16)
    x = torch.from_numpy(rng.normal(size=(tokens, hidden)).astype(np.float32)).to(torch.bfloat16)
    pool_bias = (1e-3 * rng.normal(size=pool)).astype(np.float32)
    resident = np.zeros(pool, dtype=bool)
    resident[rng.choice(pool, pool // 2, replace=False)] = True
    served_bias = np.where(resident, pool_bias, oracle_router.OFF).astype(np.float32)
    slot_of = np.full(pool, 0xFFFFFFFF, dtype=np.uint32)
    slot_of[np.flatnonzero(resident)] = rng.permutation(pool // 2).astype(np.uint32)
    kw = dict(top_k=k, score_func=func, route_scale=2.5, tau=0.3)
    want = oracle_router.routed_topk(x, w, served_bias, pool_bias, slot_of, **kw)
    assert oracle_router.min_cut_gap(want["served_keys"], k) > 0 and oracle_router.min_cut_gap(want["demand_keys"], k) > 0
    got = router.routed_topk(x.to(cuda), w.to(cuda), served_bias, pool_bias, slot_of, return_scores=True, **kw)
    np.testing.assert_allclose(got.scores.cpu().numpy(), want["scores"].numpy(), rtol=2e-5, atol=1e-9)
    np.testing.assert_array_equal(got.served_expert.cpu().numpy(), want["served_expert"].numpy())
    np.testing.assert_array_equal(got.served_slot.cpu().numpy(), want["served_slot"].numpy())
    np.testing.assert_array_equal(got.want.cpu().numpy(), want["want"].numpy())
    np.testing.assert_array_equal(got.admit.cpu().numpy(), want["admit"].numpy())
    np.testing.assert_allclose(got.served_weight.cpu().numpy(), want["served_weight"].numpy(), rtol=2e-5)
    np.testing.assert_allclose(got.want_score.cpu().numpy(), want["want_score"].numpy(), rtol=2e-5)
    assert all(resident[list(s)].all() for s in as_sets(got.served_expert.cpu()))


def test_nothing_masked_means_served_equals_demand(cuda):
    from keep_b200 import router

    rng = np.random.default_rng(3)
    w = torch.from_numpy(rng.normal(scale=0.05, size=(64, 128)).astype(np.float32)).to(cuda)
    x = torch.from_numpy(rng.normal(size=(7, 128)).astype(np.float32)).to(cuda)
    r = router.routed_topk(x, w, top_k=6, route_scale=1.5)
    assert torch.equal(r.served_expert, r.want) and torch.equal(r.served_slot, r.want)
    assert torch.allclose(r.served_weight.sum(-1), torch.full((7,), 1.5, device=cuda))
    assert (r.admit == -1).all()
    with pytest.raises(ValueError, match="top_k"):
        router.routed_topk(x, w, top_k=17)


def test_ties_go_to_the_lowest_expert(cuda):
    from keep_b200 import router

    logits = torch.zeros((2, 40), device=cuda)
    logits[1, [7, 9, 30]] = 1.0
    r = router.routed_topk(None, None, top_k=4, logits=logits, score_func="sigmoid")
    assert r.served_expert.cpu().tolist() == [[0, 1, 2, 3], [7, 9, 30, 0]]
