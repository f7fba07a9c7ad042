"""The routed operators (gather_vqmm family) against the oracle and the golden fixtures.

Mirrors tests/test_gather_vqmm.py:40-337 of the reference: gather = per-route qmv; the sorted path
scatters back to the caller's order; explicit lhs; mixed-expert tile boundaries; traces."""

import numpy as np
import pytest
import torch

from oracle import ops

pytestmark = pytest.mark.gpu


def f32(t):
    return t.float().cpu().numpy()


def test_golden_reference_outputs(cuda, golden):
    from keep_b200 import vq_switch

    g = golden("operators")
    kw = dict(input_dims=128, output_dims=24, group_size=32, code_bits=16)
    x = torch.from_numpy(g["x"]).to(cuda)
    for impl in ("cuda", "reference"):
        got = vq_switch.gather_vqmm(x, g["codes"], g["scales"], None, g["rhs"], implementation=impl, **kw)
        np.testing.assert_allclose(f32(got), g["token"], rtol=1e-5, atol=1e-5)
        got = vq_switch.gather_vqmm(x, g["codes"], g["scales"], None, g["flat_rhs"], lhs_indices=g["lhs"], implementation=impl, **kw)
        np.testing.assert_allclose(f32(got), g["routed"], rtol=1e-5, atol=1e-5)
        got = vq_switch.vq_switch_qmv(torch.from_numpy(g["xr"]).to(cuda), g["codes"], g["scales"], None, g["rhs"], implementation=impl, **kw)
        np.testing.assert_allclose(f32(got), g["per_route"], rtol=1e-5, atol=1e-5)
    got = vq_switch.gather_vqmm(x, g["codes8"], g["scales"], None, g["rhs"], **{**kw, "code_bits": 8})
    np.testing.assert_allclose(f32(got), g["token8"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("strategy", ["direct", "sorted_tiled", "per_route_decoded", "auto"])
@pytest.mark.parametrize("tokens,top_k", [(4, 3), (50, 6)])
def test_every_strategy_returns_the_callers_order(cuda, strategy, tokens, top_k):
    from keep_b200 import vq_switch

    rng = np.random.default_rng(31)
    experts, out, inp, group = 7, 40, 256, 64
    codes = rng.integers(0, 1 << 16, (experts, out, inp // 8), dtype=np.uint16)
    scales = rng.uniform(0.01, 0.2, (experts, out, inp // group)).astype(np.float16)
    x = rng.normal(size=(tokens, inp)).astype(np.float32)
    rhs = np.stack([rng.choice(experts, top_k, replace=False) for _ in range(tokens)]).astype(np.int64)
    want = ops.gather_vqmm(x, codes, scales, None, rhs, code_bits=16)
    with vq_switch.trace_gather_vqmm_calls() as trace:
        got = vq_switch.gather_vqmm(torch.from_numpy(x).to(cuda), codes, scales, None, rhs, input_dims=inp, output_dims=out,
                                    group_size=group, code_bits=16, route_strategy=strategy)
    np.testing.assert_allclose(f32(got), want, rtol=1e-4, atol=1e-3)
    assert trace[0]["route_count"] == tokens * top_k
    if strategy == "auto":
        assert trace[0]["strategy"] == ("sorted_tiled" if tokens * top_k >= 128 else "direct")


def test_sorted_routes_with_explicit_descriptors_and_boundaries(cuda):
    from keep_b200 import vq_switch

    rng = np.random.default_rng(32)
    experts, out, inp, group = 5, 24, 128, 32
    codes = rng.integers(0, 1 << 16, (experts, out, inp // 8), dtype=np.uint16)
    scales = rng.uniform(0.01, 0.2, (experts, out, inp // group)).astype(np.float16)
    x = rng.normal(size=(9, inp)).astype(np.float32)
    sorted_rhs = np.array([0] * 3 + [2] * 37 + [4] * 2, dtype=np.int32)  # expert 1 and 3 unused; 2 spans tiles
    sorted_lhs = rng.integers(0, 9, sorted_rhs.shape[0]).astype(np.int32)
    want = ops.gather_vqmm(x, codes, scales, None, sorted_rhs, lhs_indices=sorted_lhs, code_bits=16)
    xt = torch.from_numpy(x).to(cuda)
    tiles = vq_switch.expert_block_tile_descriptors(torch.from_numpy(sorted_rhs).to(cuda), num_experts=experts, route_tile=32)
    te, to, tc = (t.cpu().numpy() for t in tiles)
    assert te.shape[0] == 2 + experts and tc.sum() == sorted_rhs.shape[0]
    assert [(int(e), int(o), int(c)) for e, o, c in zip(te, to, tc) if c] == [(0, 0, 3), (2, 3, 32), (2, 35, 5), (4, 40, 2)]
    got = vq_switch.gather_vqmm_sorted_routes(xt, codes, scales, None, sorted_rhs, sorted_lhs, input_dims=inp, output_dims=out,
                                              group_size=group, code_bits=16, validate_indices=True, tile_descriptors=tiles)
    np.testing.assert_allclose(f32(got), want, rtol=1e-4, atol=1e-3)
    with pytest.raises(ValueError, match="sorted nondecreasing"):
        vq_switch.gather_vqmm_sorted_routes(xt, codes, scales, None, sorted_rhs[::-1].copy(), sorted_lhs, input_dims=inp,
                                            output_dims=out, group_size=group, code_bits=16, validate_indices=True)
    empty = vq_switch.gather_vqmm_sorted_routes(xt, codes, scales, None, sorted_rhs[:0], sorted_lhs[:0], input_dims=inp,
                                                output_dims=out, group_size=group, code_bits=16)
    assert tuple(empty.shape) == (0, out)


def test_metadata_errors_match_the_reference_messages(cuda):
    from keep_b200 import vq_switch

    x = torch.zeros((2, 64), device=cuda)
    codes = torch.zeros((3, 8, 8), dtype=torch.uint16, device=cuda)
    scales = torch.ones((3, 8, 2), device=cuda)
    rhs = torch.zeros((2, 2), dtype=torch.int64, device=cuda)
    kw = dict(input_dims=64, output_dims=8, group_size=32, code_bits=16)
    with pytest.raises(ValueError, match="route_strategy must be"):
        vq_switch.gather_vqmm(x, codes, scales, None, rhs, route_strategy="tiled", **kw)
    with pytest.raises(ValueError, match="rhs_indices token dimension"):
        vq_switch.gather_vqmm(x, codes, scales, None, rhs[:1], **kw)
    with pytest.raises(ValueError, match="codes must have shape"):
        vq_switch.gather_vqmm(x, codes[:, :4], scales, None, rhs, **kw)
    with pytest.raises(ValueError, match="codes dtype must be uint16"):
        vq_switch.gather_vqmm(x, codes.to(torch.uint8), scales, None, rhs, **kw)
    with pytest.raises(ValueError, match=r"indices must be in \[0, 3\)"):
        vq_switch.gather_vqmm(x, codes, scales, None, rhs + 3, implementation="reference", **kw)
    with pytest.raises(ValueError, match="same flattened shape"):
        vq_switch.gather_vqmm(x, codes, scales, None, rhs.reshape(-1), lhs_indices=torch.zeros(3, dtype=torch.int32, device=cuda), **kw)


@pytest.mark.parametrize("routes,experts", [(300, 6), (1500, 6), (1200, 40)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sorted_routes_on_the_tensor_core_kernels(cuda, routes, experts, dtype):
    """Prefill-shaped sorted calls (16-bit codes, in_dim % 256 == 0, one scale group per row) with
    bf16 activations run keepvq_grouped_projection: the mma.sync kernel for 300 routes, the tcgen05
    kernel for 1500 routes over 6 experts, the mma.sync one again for 1200 routes spread over 40
    experts; the only rounding there is the 16-bit fixed-point step on the activations.  fp32
    activations are not narrowed: they take the general kernel (24-bit fixed point)."""
    from keep_b200 import prefill, vq, vq_switch

    rng = np.random.default_rng(90 + routes)
    out, inp, tokens = 136, 512, 64
    codes = rng.integers(0, 1 << 16, (experts, out, inp // 8), dtype=np.uint16)
    scales = (0.02 * rng.uniform(0.5, 1.5, (experts, out, 1))).astype(np.float16)
    x = torch.from_numpy(rng.normal(size=(tokens, inp)).astype(np.float32)).to(dtype)
    rhs = np.sort(rng.integers(0, experts - 1, routes)).astype(np.int64)  # the last expert gets no route
    lhs = rng.integers(0, tokens, routes).astype(np.int64)
    want = ops.gather_vqmm(x.float().numpy(), codes, scales, None, rhs, lhs_indices=lhs, code_bits=16)
    got = vq_switch.gather_vqmm_sorted_routes(x.to(cuda), codes, scales, None, rhs, lhs, input_dims=inp, output_dims=out,
                                              group_size=inp, code_bits=16, validate_indices=True)
    assert got.dtype == dtype and tuple(got.shape) == (routes, out)
    tol = dict(rtol=1e-4, atol=3e-4) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(f32(got), want, **tol)
    rows = x.to(cuda)[torch.from_numpy(lhs).to(cuda)]
    direct = prefill.tensor_core_projection(rows, torch.from_numpy(codes).to(cuda), torch.from_numpy(scales).to(cuda),
                                            vq.table_on(cuda, "e8p"), torch.from_numpy(rhs).to(cuda))
    if dtype == torch.float32:
        assert direct is None
    else:
        assert direct is not None and torch.equal(direct, got)  # the operator did take this entry point


def test_routes_without_an_expert_give_zero_rows_on_every_path(cuda):
    """A route whose index names no expert (0xFFFFFFFF, or any value past the last expert) returns
    a row of zeros from the tensor-core kernels and from the general kernel alike."""
    from keep_b200 import kernels, prefill, vq

    rng = np.random.default_rng(21)
    experts, out, inp = 4, 64, 256
    codes = rng.integers(0, 1 << 16, (experts, out, inp // 8), dtype=np.uint16)
    scales = (0.02 * rng.uniform(0.5, 1.5, (experts, out, 1))).astype(np.float16)
    table = vq.table_on(cuda, "e8p")
    for routes in (6, 64):  # the sweep kernel and the slab kernel
        rhs = rng.integers(0, experts, routes).astype(np.int64)
        rhs[1], rhs[routes - 2] = 0xFFFFFFFF, experts + 3
        x = torch.from_numpy(rng.normal(size=(routes, inp)).astype(np.float32)).to(cuda)
        dead = torch.tensor([1, routes - 2])
        rhs_t = torch.from_numpy(rhs.astype(np.uint32).view(np.int32)).to(cuda)
        fast = prefill.tensor_core_projection(x.to(torch.bfloat16), torch.from_numpy(codes).to(cuda), torch.from_numpy(scales).to(cuda), table, rhs_t)
        assert fast is not None and bool((fast[dead] == 0).all()) and bool((fast[0] != 0).any())
        general = kernels.e8p_m1_per_route(x, codes, scales, table, rhs.astype(np.uint32), output_dims=out)
        assert bool((general[dead] == 0).all()) and bool((general[0] != 0).any())


@pytest.mark.parametrize("factor", [300.0, 3000.0])
def test_one_outlier_channel_costs_what_the_header_says(cuda, factor):
    """fp16 / bf16 rows are held as 16-bit fixed point with one power-of-two step per row, so a
    channel far above the rest takes precision from the small channels.  Bounds stated beside
    ``keepvq_grouped_projection``: against the true output the gap stays near 1e-3 of its largest
    magnitude; against the output the row would give without the outlier channel it is below 1 %
    at 300 times the row's RMS and below 5 % at 3000 times.  fp32 rows go to the general kernel,
    which keeps 24 bits of a row: 256 times tighter."""
    from keep_b200 import kernels, prefill, vq

    rng = np.random.default_rng(22)
    experts, out, inp, routes = 2, 256, 4096, 64
    codes = rng.integers(0, 1 << 16, (experts, out, inp // 8), dtype=np.uint16)
    scales = (0.02 * rng.uniform(0.5, 1.5, (experts, out, 1))).astype(np.float16)
    dense = ops.dense_experts(codes, scales, dtype=np.float64)
    rhs = rng.integers(0, experts, routes).astype(np.uint32)
    x = rng.normal(size=(routes, inp)).astype(np.float32)
    x[:, 7] = factor
    xb = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    xn = xb.float().cpu().numpy().astype(np.float64)
    want = np.stack([xn[r] @ dense[e].T for r, e in enumerate(rhs)])
    quiet = xn.copy()
    quiet[:, 7] = 0.0
    want_quiet = np.stack([quiet[r] @ dense[e].T for r, e in enumerate(rhs)])
    table = vq.table_on(cuda, "e8p")
    got = prefill.tensor_core_projection(xb, torch.from_numpy(codes).to(cuda), torch.from_numpy(scales).to(cuda), table,
                                         torch.from_numpy(rhs.view(np.int32)).to(cuda)).float().cpu().numpy()
    # bf16 output rounding alone is 2^-9 relative; the activation step adds the rest
    assert np.abs(got - want).max() <= 6e-3 * np.abs(want).max()
    noise = np.abs((got - want)).max() / np.abs(want_quiet).max()
    assert noise <= (0.01 if factor == 300.0 else 0.05) + 2 ** -8 * np.abs(want).max() / np.abs(want_quiet).max(), noise
    # fp32 rows: 24-bit fixed point in the general kernel
    got32 = kernels.e8p_m1_per_route(torch.from_numpy(xn.astype(np.float32)).to(cuda), codes, scales, table, rhs, output_dims=out).cpu().numpy()
    assert np.abs(got32 - want).max() <= (5e-5 if factor == 300.0 else 4e-4) * np.abs(want_quiet).max()
