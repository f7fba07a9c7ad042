"""The router oracle against outputs of the reference's own gate_masked (no GPU)."""

import numpy as np
import pytest
import torch

from oracle import router


@pytest.mark.parametrize("func", ["softmax", "sigmoid", "sqrtsoftplus"])
@pytest.mark.parametrize("mask", ["all", "masked", "few"])
def test_gate_masked_matches_the_reference(golden, func, mask):
    g = golden("router")
    allowed = {"all": np.ones_like(g["allowed"]), "masked": g["allowed"], "few": g["few"]}[mask]
    sc = router.scores(g["x"], g["weight"], score_func=func, gate_temp=1.25)
    w, idx = router.gate_masked(sc, g["bias"], allowed, top_k=int(g["top_k"]), route_scale=1.5)
    want_w, want_i = g[f"{func}_{mask}_weights"], g[f"{func}_{mask}_indices"]
    live = want_w > 0
    # picks that carry weight agree exactly (position by position); dead picks are unspecified
    np.testing.assert_array_equal(idx.numpy()[live], want_i[live])
    np.testing.assert_allclose(w.numpy(), want_w, rtol=1e-6, atol=1e-7)
    if mask == "few":
        assert ((w.numpy() > 0).sum(-1) == 2).all()


def test_nothing_masked_is_the_plain_router_and_weights_sum_to_route_scale(golden):
    g = golden("router")
    r = router.routed_topk(g["x"], g["weight"], g["bias"], g["bias"], top_k=4, score_func="sqrtsoftplus", route_scale=1.5, gate_temp=1.25)
    np.testing.assert_array_equal(r["served_expert"].numpy(), r["want"].numpy())
    np.testing.assert_allclose(r["served_weight"].sum(-1).numpy(), 1.5, rtol=1e-6)
    assert (r["admit"].numpy() == -1).all()  # nothing absent, nothing to admit


def test_admission_is_demanded_absent_and_strong():
    rng = np.random.default_rng(5)
    w = rng.normal(scale=0.6, size=(16, 32)).astype(np.float32)
    x = rng.normal(size=(12, 32)).astype(np.float32)
    bias = np.where(rng.random(16) < 0.5, 0.0, router.OFF).astype(np.float32)
    r = router.routed_topk(x, w, bias, None, top_k=3, tau=0.3)
    want, g, admit = r["want"].numpy(), r["demand_weight"].numpy(), r["admit"].numpy()
    absent = bias[want] <= -1e29
    np.testing.assert_array_equal(admit, np.where(absent & (g >= 0.3), want, -1))
    assert (r["served_expert"].numpy() >= 0).all() and (bias[r["served_expert"].numpy()] == 0).all()
    assert torch.allclose(r["served_weight"].sum(-1), torch.ones(12))
