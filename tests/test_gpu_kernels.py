"""The kernel-level operators against a dense decode of the same codes.

Re-expresses the reference's Metal-only tests on the CUDA operators with the same shapes, index
patterns and tolerances: tests/test_e8p_m1.py:119-165, tests/test_e8_1bit_m1.py:42-66,
tests/test_e8p_nested_m1.py:40-74, tests/test_vq_qmv.py:74-155, tests/test_vq_qmm.py:20-87.
Codes are drawn uniformly (the reference fits them with its encoder, which is not part of this path).
"""

import numpy as np
import pytest
import torch

from oracle import e8, ops

pytestmark = pytest.mark.gpu
NONE = e8.NO_RESIDUAL
HOT_OF_SLOT = np.array([2, NONE, 0, NONE, NONE, 1], dtype=np.uint32)


def layer(experts=6, out=32, inp=64, seed=0, group_size=32, code_bits=16):
    rng = np.random.default_rng(seed)
    hi = 1 << code_bits
    codes = rng.integers(0, hi, (experts, out, inp // 8), dtype=np.uint16 if code_bits == 16 else np.uint8)
    scales = rng.uniform(0.01, 0.2, (experts, out, inp // group_size)).astype(np.float16)
    return codes, scales


def f32(t):
    return t.float().cpu().numpy()


@pytest.mark.parametrize("group_size,inp,out", [(32, 128, 96), (64, 768, 93), (512, 4096, 40), (24, 48, 7)])
def test_token_and_per_route_e8p_match_the_dense_decode(cuda, group_size, inp, out):
    from keep_b200 import kernels, vq

    codes, scales = layer(out=out, inp=inp, seed=3, group_size=group_size)
    dense = ops.dense_experts(codes, scales, dtype=np.float64)
    table = vq.e8p_packed_abs_grid()
    rng = np.random.default_rng(4)
    rhs = np.array([[5, 0, 3]], dtype=np.uint32)
    x = rng.normal(size=(1, inp)).astype(np.float32)
    if (inp // 8 // (inp // group_size)) % 4:
        with pytest.raises(ValueError, match="divisible by 4"):
            kernels.e8p_m1_token_layout(torch.from_numpy(x).to(cuda), codes, scales, table, rhs, output_dims=out)
        return
    got = kernels.e8p_m1_token_layout(torch.from_numpy(x).to(cuda), codes, scales, table, rhs, output_dims=out)
    assert got.dtype == torch.float32 and tuple(got.shape) == (1, 3, out)
    want = np.stack([x[0] @ dense[e].T for e in (5, 0, 3)])[None]
    np.testing.assert_allclose(f32(got), want, rtol=1e-4, atol=1e-3)
    xr = rng.normal(size=(3, inp)).astype(np.float32)
    got = kernels.e8p_m1_per_route(torch.from_numpy(xr).to(cuda), codes, scales, table, rhs.reshape(-1), output_dims=out)
    want = np.stack([xr[r] @ dense[e].T for r, e in enumerate((5, 0, 3))])
    np.testing.assert_allclose(f32(got), want, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("tokens", [2, 5, 32])
def test_multi_token_layouts_match_the_dense_decode(cuda, tokens):
    from keep_b200 import kernels, vq

    codes, scales = layer(out=64, inp=128, seed=5)
    dense = ops.dense_experts(codes, scales, dtype=np.float64)
    table = vq.e8p_packed_abs_grid()
    rng = np.random.default_rng(6)
    rhs = np.stack([rng.choice(6, 3, replace=False) for _ in range(tokens)]).astype(np.uint32)
    x = rng.normal(size=(tokens, 128)).astype(np.float32)
    got = kernels.e8p_m1_token_layout(torch.from_numpy(x).to(cuda), codes, scales, table, rhs, output_dims=64)
    want = np.stack([[x[t] @ dense[e].T for e in rhs[t]] for t in range(tokens)])
    np.testing.assert_allclose(f32(got), want, rtol=1e-4, atol=1e-3)
    xr = rng.normal(size=(tokens * 3, 128)).astype(np.float32)
    got = kernels.e8p_m1_per_route(torch.from_numpy(xr).to(cuda), codes, scales, table, rhs.reshape(-1), output_dims=64)
    want = np.stack([xr[r] @ dense[e].T for r, e in enumerate(rhs.reshape(-1))])
    np.testing.assert_allclose(f32(got), want, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2), (torch.float16, 2e-3)])
def test_e8_1bit_layouts_and_no_residual_routes(cuda, dtype, tol):
    from keep_b200 import kernels, vq

    codes, scales = layer(experts=4, out=40, inp=256, seed=8, group_size=64, code_bits=8)
    dense = ops.dense_experts(codes, scales, code_bits=8, dtype=np.float64)
    table = vq.pair_packed(vq.e8_1bit_packed())
    np.testing.assert_array_equal(table, e8.pair_packed(e8.e8_1bit_packed()))
    rng = np.random.default_rng(9)
    rhs = np.array([[3, NONE, 0], [NONE, NONE, 2]], dtype=np.uint32)
    x = torch.from_numpy(rng.normal(size=(2, 256)).astype(np.float32)).to(cuda).to(dtype)
    xn = x.float().cpu().numpy().astype(np.float64)
    got = kernels.e8_1bit_m1_token_layout(x, codes, scales, table, rhs, output_dims=40)
    assert got.dtype == dtype
    want = np.stack([[np.zeros(40) if e == NONE else xn[t] @ dense[e].T for e in rhs[t]] for t in range(2)])
    assert e8.relative_gap(f32(got), want) <= tol
    assert np.all(f32(got)[0, 1] == 0) and np.all(f32(got)[1, :2] == 0)
    xr = torch.from_numpy(rng.normal(size=(6, 256)).astype(np.float32)).to(cuda).to(dtype)
    xn = xr.float().cpu().numpy().astype(np.float64)
    got = kernels.e8_1bit_m1_per_route(xr, codes, scales, table, rhs.reshape(-1), output_dims=40)
    want = np.stack([np.zeros(40) if e == NONE else xn[r] @ dense[e].T for r, e in enumerate(rhs.reshape(-1))])
    assert e8.relative_gap(f32(got), want) <= tol


def nested_case(out, inp, group_size, res_group_size, seed):
    rng = np.random.default_rng(seed)
    slots, rows = len(HOT_OF_SLOT), int((HOT_OF_SLOT != NONE).sum())
    codes = rng.integers(0, 1 << 16, (slots, out, inp // 8), dtype=np.uint16)
    scales = rng.uniform(0.01, 0.2, (slots, out, inp // group_size)).astype(np.float16)
    res_codes = rng.integers(0, 256, (rows, out, inp // 8), dtype=np.uint8)
    res_scales = rng.uniform(0.005, 0.1, (rows, out, inp // res_group_size)).astype(np.float16)
    dense = ops.nested_dense(codes, scales, res_codes, res_scales, HOT_OF_SLOT)
    return (codes, scales), (res_codes, res_scales), dense


@pytest.mark.parametrize("group_size,res_group_size,inp,out", [(32, 32, 128, 96), (64, 128, 768, 93), (512, 64, 4096, 64)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_nested_layouts_match_dense_and_the_two_separate_kernels(cuda, group_size, res_group_size, inp, out, dtype, tol):
    from keep_b200 import kernels, vq

    (codes, scales), (res_codes, res_scales), dense = nested_case(out, inp, group_size, res_group_size, seed=3)
    base = (codes, scales, vq.e8p_packed_abs_grid())
    residual = (res_codes, res_scales, vq.half2_pairs(vq.e8_1bit_grid()))
    separate_table = vq.pair_packed(vq.e8_1bit_packed())
    rng = np.random.default_rng(4)
    rhs = np.array([[5, 0, 3], [1, 2, 2], [4, 5, 0]], dtype=np.uint32)

    def rows(n):
        x = torch.from_numpy(rng.normal(size=(n, inp)).astype(np.float32)).to(cuda).to(dtype)
        return x, x.float().cpu().numpy().astype(np.float64)

    def check(got, want, separate):
        assert got.dtype == dtype and tuple(got.shape) == want.shape
        assert e8.relative_gap(f32(got), want) <= tol
        if dtype == torch.float32:  # bit for bit the fp32 sum of the two kernels it replaces
            np.testing.assert_array_equal(f32(got), f32(separate))

    x, xn = rows(3)
    got = kernels.e8p_nested_m1_token_layout(x, base, rhs, residual, HOT_OF_SLOT, output_dims=out)
    separate = (kernels.e8p_m1_token_layout(x, *base, rhs, output_dims=out)
                + kernels.e8_1bit_m1_token_layout(x, res_codes, res_scales, separate_table, HOT_OF_SLOT[rhs], output_dims=out))
    check(got, np.stack([[xn[t] @ dense[s].T for s in rhs[t]] for t in range(3)]), separate)
    x, xn = rows(9)
    flat = rhs.reshape(-1)
    got = kernels.e8p_nested_m1_per_route(x, base, flat, residual, HOT_OF_SLOT, output_dims=out)
    separate = (kernels.e8p_m1_per_route(x, *base, flat, output_dims=out)
                + kernels.e8_1bit_m1_per_route(x, res_codes, res_scales, separate_table, HOT_OF_SLOT[flat], output_dims=out))
    check(got, np.stack([xn[r] @ dense[s].T for r, s in enumerate(flat)]), separate)


@pytest.mark.parametrize("code_bits", [8, 16])
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 1e-5), (torch.float16, 2 ** -5), (torch.bfloat16, 2 ** -2)])
def test_vq_qmv_and_vq_qmm_match_dense_dequant(cuda, code_bits, dtype, atol):
    from keep_b200 import kernels

    rng = np.random.default_rng(20)
    out, inp, group = 48, 256, 64
    codes = rng.integers(0, 1 << code_bits, (out, inp // 8), dtype=np.uint16 if code_bits == 16 else np.uint8)
    scales = rng.uniform(0.01, 0.2, (out, inp // group)).astype(np.float32)
    x = torch.from_numpy(rng.normal(size=(5, inp)).astype(np.float32)).to(cuda).to(dtype)
    xn = x.float().cpu().numpy()
    kw = dict(in_dim=inp, out_dim=out, group_size=group, code_bits=code_bits)
    y = kernels.vq_qmv(x[0], codes, scales, None, **kw)
    assert y.dtype == dtype and tuple(y.shape) == (out,)
    want = ops.vq_qmv_reference(xn[0], codes, scales, code_bits=code_bits)
    np.testing.assert_allclose(f32(y), want, rtol=1e-6 if dtype == torch.float32 else 2e-2, atol=atol)
    ref = kernels.vq_qmv(x[0], codes, scales, None, implementation="reference", **kw)
    np.testing.assert_allclose(f32(ref), want, rtol=1e-5, atol=1e-5)
    ym = kernels.vq_qmm(x, codes, scales, None, **kw)
    assert tuple(ym.shape) == (5, out)
    np.testing.assert_allclose(f32(ym), ops.vq_qmm_reference(xn, codes, scales, code_bits=code_bits),
                               rtol=1e-6 if dtype == torch.float32 else 2e-2, atol=atol)


def test_vq_qmv_shape_and_dtype_errors(cuda):
    from keep_b200 import kernels

    x = torch.zeros(64, device=cuda)
    codes = torch.zeros((8, 8), dtype=torch.uint16, device=cuda)
    scales = torch.ones((8, 1), device=cuda)
    kw = dict(in_dim=64, out_dim=8, group_size=64, code_bits=16)
    with pytest.raises(ValueError, match="x must have shape"):
        kernels.vq_qmv(x[:32], codes, scales, None, **kw)
    with pytest.raises(ValueError, match="codes dtype must be uint16"):
        kernels.vq_qmv(x, codes.to(torch.uint8), scales, None, **kw)
    with pytest.raises(ValueError, match="divisible by group_size"):
        kernels.vq_qmv(x, codes, scales, None, **{**kw, "group_size": 48})
    with pytest.raises(ValueError, match="code_bits must be 8 or 16"):
        kernels.vq_qmv(x, codes, scales, None, **{**kw, "code_bits": 4})
    with pytest.raises(ValueError, match="codebook_duplication"):
        kernels.vq_qmv(x, codes, scales, None, codebook_duplication=2, **kw)


def test_config1_single_expert_vq_qmv(cuda):
    """W [2048 x 4096] uniform codes, scale 0.02 U(0.5, 1.5) per row, x bf16 N(0,1), seed 0: output
    within the bf16 tolerance of the dense-decode oracle, cosine reported."""
    from keep_b200 import kernels

    rng = np.random.default_rng(0)
    codes = rng.integers(0, 65536, (2048, 512), dtype=np.uint16)
    scales = (0.02 * rng.uniform(0.5, 1.5, (2048, 1))).astype(np.float16)
    x = torch.from_numpy(rng.normal(size=4096).astype(np.float32)).to(cuda).to(torch.bfloat16)
    y = kernels.vq_qmv(x, codes, scales, None, in_dim=4096, out_dim=2048, group_size=4096, code_bits=16)
    want = ops.vq_qmv_reference(x, codes, scales, code_bits=16)
    assert y.dtype == torch.bfloat16
    gap, cos = e8.relative_gap(f32(y), want), e8.cosine_similarity(f32(y), want)
    print(f"config 1: relative gap {gap:.3e}, cosine {cos:.8f}")
    assert gap <= 1e-2 and cos >= 0.9999
