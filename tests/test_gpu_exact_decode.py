"""Code-to-weight decode INSIDE the projection kernels, bit for bit.

``test_gpu_decode.py`` checks the stand-alone decode kernel.  The projections decode through their
own paths (table and arithmetic decoders of the mma.sync kernels, the tcgen05 decoder, the
residual table, the general kernel's int8 form).  Those are exact integer arithmetic, so a one-hot
activation row with a power-of-two value must return ``scale * weight * value`` with no rounding at
all: every one of the 65,536 E8P codes (and the 256 residual codes) is pushed through every kernel
family that way and compared with the oracle's decode (src/keep/vq/e8.py:210-234,186-200 restated
in ``oracle/e8.py``)."""

import numpy as np
import pytest
import torch

from oracle import e8

pytestmark = pytest.mark.gpu
IN, CW = 256, 32           # one 256-input scale group: 32 codewords per row
ROWS = 512                 # rows per expert: 16,384 codewords; four experts hold every 16-bit code once
VALUE = 2.0 ** 14


def all_codes_experts(copies=1):
    """codes [4 * copies, ROWS, CW]: expert e holds codes (e % 4) * 16384 ... in row-major order."""
    block = np.arange(1 << 16, dtype=np.uint16).reshape(4, ROWS, CW)
    return np.tile(block, (copies, 1, 1))


def scales_for(experts, seed):
    rng = np.random.default_rng(seed)
    return (0.02 * rng.uniform(0.5, 1.5, (experts, ROWS, 1))).astype(np.float16)


def one_hot_rows(sign=1.0):
    """[256, IN]: row i is VALUE at input i, zero elsewhere."""
    return (sign * VALUE * np.eye(IN, dtype=np.float32))


def expected(codes, scales, value):
    """[experts, IN, ROWS] fp32: out[e, i, row] = scale * weight[row, i] * value, exact in fp32."""
    dense = e8.decode_weight_matrix(codes.reshape(-1, CW), scales.reshape(-1, 1).astype(np.float32), code_bits=16)
    dense = dense.reshape(codes.shape[0], ROWS, IN)
    return np.transpose(dense, (0, 2, 1)) * np.float32(value)


def run_grouped(cuda, x, codes, scales, rhs, **kw):
    from keep_b200 import prefill, vq

    out = prefill.tensor_core_projection(torch.from_numpy(x).to(cuda).to(torch.bfloat16), torch.from_numpy(codes).to(cuda),
                                         torch.from_numpy(scales).to(cuda), vq.table_on(cuda, "e8p"), torch.from_numpy(rhs).to(cuda), **kw)
    assert out is not None, "these shapes are meant for the tensor-core kernels"
    return out.float().cpu().numpy()


def check_rows(got, want_by_expert, rhs, which_input):
    """got [routes, ROWS] in bf16-rounded fp32; the exact value rounded to bf16 must match bit for bit."""
    want = want_by_expert[rhs, which_input]                      # [routes, ROWS]
    want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("family", ["few", "slab8", "slab4", "tcgen05"])
def test_single_projection_kernels_return_scale_times_weight_exactly(cuda, family):
    """The M = 1 (down-shaped) kernels through ``keepvq_grouped_projection``.  The route count and
    the expert count pick the kernel: under 48 routes the sweep kernel ("few" below), from there the
    slab kernel with eight routes per group (many routes per expert) or four (few), and from 1024
    routes with 24 per expert the tcgen05 kernel."""
    copies = {"few": 1, "slab8": 1, "slab4": 32, "tcgen05": 1}[family]
    codes, scales = all_codes_experts(copies), None
    scales = scales_for(codes.shape[0], 1)
    want = expected(codes[:4], scales[:4], VALUE) if copies == 1 else None
    x = one_hot_rows()
    if family == "few":
        for e in range(4):
            for first in range(0, IN, 32):   # 32 routes per call
                rhs = np.full(32, e, dtype=np.int32)
                got = run_grouped(cuda, x[first:first + 32], codes, scales, rhs)
                check_rows(got, want, rhs, np.arange(first, first + 32))
    elif family == "slab8":
        for e in range(4):                   # 256 routes on one expert: groups of eight
            rhs = np.full(IN, e, dtype=np.int32)
            check_rows(run_grouped(cuda, x, codes, scales, rhs), want, rhs, np.arange(IN))
    elif family == "slab4":
        want = expected(codes, scales, VALUE)
        for shift in range(4):               # 256 routes over 128 experts: at most two per expert
            rhs = ((np.arange(IN) % 32) * 4 + (np.arange(IN) // 32 + shift) % 4).astype(np.int32)
            check_rows(run_grouped(cuda, x, codes, scales, rhs), want, rhs, np.arange(IN))
    else:
        rhs = np.repeat(np.arange(4, dtype=np.int32), IN)   # 1024 routes, 256 per expert
        got = run_grouped(cuda, np.tile(x, (4, 1)), codes, scales, rhs)
        check_rows(got, want, rhs, np.tile(np.arange(IN), 4))


@pytest.mark.parametrize("family,in_dim,routes,rows", [("sweep", 2048, 6, ROWS), ("sweep", 4096, 40, ROWS), ("sweep", 2304, 7, ROWS), ("sweep", 8192, 6, ROWS),
                                                       ("sweep", 1024, 9, 200), ("split", 2048, 60, ROWS), ("split-residual", 2048, 5, ROWS)])
def test_few_route_kernels_over_wide_inputs_exactly(cuda, family, in_dim, routes, rows):
    """Calls with few routes run the sweep kernel: the sixteen warps of a CTA split the input
    dimension (evenly or not: 2304 inputs are nine chunks over eight warps), carry the partial sums
    of several 16-row units and add them up in shared memory.  With a residual tier the split form
    of the slab kernel does the same per item.  (The 256-input cases above give every warp the
    whole row.)  A one-hot row at a random input picks one weight per output row, so whichever warp
    owns that part of the row must deliver it, exactly.  200 output rows leave the last unit of an
    expert short (its row indices are clamped); 60 routes over 32 experts are few route groups of
    a call too large for the sweep kernel: the split slab kernel without a residual."""
    from keep_b200 import vq

    experts, cw = (32 if family == "split" else 4), in_dim // 8  # 60 routes over 32 experts: groups of four, and few of them
    rng = np.random.default_rng(in_dim + routes)
    codes = rng.integers(0, 1 << 16, (experts, rows, cw), dtype=np.uint16)
    scales = np.ascontiguousarray(scales_for(experts, 6)[:, :rows])
    dense = e8.decode_weight_matrix(codes.reshape(-1, cw), scales.reshape(-1, 1).astype(np.float32), code_bits=16).reshape(experts, rows, in_dim)
    kw = {}
    if family == "split-residual":
        res_codes = rng.integers(0, 256, (2, rows, cw), dtype=np.uint8)
        res_scales = np.full((2, rows, 1), 2.0 ** -8, dtype=np.float16)
        hot = np.array([1, e8.NO_RESIDUAL, e8.NO_RESIDUAL, 0], dtype=np.uint32)
        res = e8.decode_weight_matrix(res_codes.reshape(-1, cw), res_scales.reshape(-1, 1).astype(np.float32), code_bits=8).reshape(2, rows, in_dim)
        dense[0] += res[1]
        dense[3] += res[0]
        kw = dict(residual=(torch.from_numpy(res_codes).to(cuda), torch.from_numpy(res_scales).to(cuda), vq.table_on(cuda, "e8_1bit_half2")),
                  hot_of_slot=torch.from_numpy(hot.astype(np.int32)).to(cuda))
    for call in range(4):
        rhs = rng.integers(0, experts, routes).astype(np.int32)
        which = rng.integers(0, in_dim, routes)
        which[0], which[-1] = 0, in_dim - 1   # the first and the last warp's share
        x = np.zeros((routes, in_dim), dtype=np.float32)
        x[np.arange(routes), which] = VALUE
        got = run_grouped(cuda, x, codes, scales, rhs, **kw)
        want = dense[rhs, :, which] * np.float32(VALUE)           # [routes, ROWS]
        np.testing.assert_array_equal(got, torch.from_numpy(want).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("cols", [8, 4])
def test_residual_pass_returns_base_plus_residual_exactly(cuda, cols):
    """Slab kernel with a residual tier: base codes cover a quarter of the 16-bit codes per expert,
    the 8-bit residual rows cover all 256 residual codes; the sum of the two decodes times the
    one-hot value is exact in fp32 and rounded once to bf16."""
    from keep_b200 import vq

    experts = 4 if cols == 8 else 128
    codes = all_codes_experts(experts // 4)
    scales = scales_for(experts, 2)
    res_rows = 2
    res_codes = (np.arange(res_rows * ROWS * CW, dtype=np.int64) % 256).astype(np.uint8).reshape(res_rows, ROWS, CW)
    res_scales = np.full((res_rows, ROWS, 1), 2.0 ** -8, dtype=np.float16)  # a power of two keeps base + residual exact
    hot = np.full(experts, e8.NO_RESIDUAL, dtype=np.uint32)
    hot[0], hot[experts - 1] = 1, 0
    base = expected(codes, scales, VALUE)
    res = e8.decode_weight_matrix(res_codes.reshape(-1, CW), res_scales.reshape(-1, 1).astype(np.float32), code_bits=8).reshape(res_rows, ROWS, IN)
    want = base.copy()
    for slot in (0, experts - 1):
        want[slot] += np.transpose(res[hot[slot]], (1, 0)) * np.float32(VALUE)
    if cols == 8:
        rhs = np.repeat(np.array([0, 3], dtype=np.int32), IN)
        which = np.tile(np.arange(IN), 2)
        x = np.tile(one_hot_rows(), (2, 1))
    else:
        rhs = np.concatenate([np.zeros(3, np.int32), np.full(3, experts - 1, np.int32), np.arange(IN - 6, dtype=np.int32) % experts])
        which = np.arange(IN)
        x = one_hot_rows()
    residual = (torch.from_numpy(res_codes).to(cuda), torch.from_numpy(res_scales).to(cuda), vq.table_on(cuda, "e8_1bit_half2"))
    got = run_grouped(cuda, x, codes, scales, rhs, residual=residual, hot_of_slot=torch.from_numpy(hot.astype(np.int32)).to(cuda))
    check_rows(got, want, rhs, which)


@pytest.mark.parametrize("family", ["few", "slab4", "slab8", "tcgen05"])
def test_gate_up_kernels_decode_both_matrices_exactly(cuda, family):
    """The M = 2 kernels fuse gate, up and SwiGLU, so G and U are not visible on their own.  With
    a one-hot activation of +-2^14 and a gate weight that is positive, G is at least 41 and
    silu(G) = G exactly in fp32 (exp(-G) is below half an ulp of 1), so
    h = round(round(G) * round(U)) is a closed form of the two decodes.  One matrix holds every
    16-bit code, the other a code whose eight weights are all positive; then the roles swap, with
    the activation's sign chosen per output so that G stays positive."""
    from keep_b200 import _lib, moe, vq

    tokens = {"few": 6, "slab4": 256, "slab8": 256, "tcgen05": 1024}[family]
    experts = {"few": 4, "slab4": 128, "slab8": 4, "tcgen05": 4}[family]
    every = all_codes_experts(experts // 4)
    # a codeword whose eight weights are all positive (the first one there is)
    grid = e8.decode_e8p(np.arange(1 << 16, dtype=np.uint16))
    positive_code = int(np.flatnonzero((grid > 0).all(axis=-1))[0])
    positive = np.full_like(every, positive_code)
    table = vq.table_on(cuda, "e8p")
    scales = scales_for(experts, 3)
    down = moe.Projection(torch.zeros((experts, IN, ROWS // 8), dtype=torch.uint16, device=cuda), torch.ones((experts, IN, 1), dtype=torch.float16, device=cuda))
    dev = lambda a: torch.from_numpy(a).to(cuda)  # noqa: E731
    w_every = expected(every, scales, 1.0)          # [experts, IN, ROWS] scale * weight
    w_pos = expected(positive, scales, 1.0)

    def run(gate_codes, up_codes, x, slots):
        layer = moe.RoutedMoELayer(torch.zeros((experts, IN), dtype=torch.bfloat16, device=cuda), moe.Projection(dev(gate_codes), dev(scales)),
                                   moe.Projection(dev(up_codes), dev(scales)), down, top_k=1, codebook=table)
        assert layer.kernel_path == "tensor"
        xt = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
        r = layer._buffers_for(int(xt.shape[0]), xt.dtype)["routing"]
        r.served_slot.copy_(torch.from_numpy(slots.reshape(-1, 1)).to(cuda))
        r.served_weight.fill_(1.0)
        layer.decode(xt, stages=_lib.STAGE_PREPARE | _lib.STAGE_GATE_UP)
        return layer.route_hidden(int(xt.shape[0]), xt.dtype).float().cpu().numpy()

    def closed_form(g, u):  # h = round(round(G) * round(U) * 1)
        g16 = torch.from_numpy(g).to(torch.bfloat16).float()
        u16 = torch.from_numpy(u).to(torch.bfloat16).float()
        return (g16 * u16).to(torch.bfloat16).float().numpy()

    rng = np.random.default_rng(7)
    for call in range(8 if family == "few" else 2):
        which = rng.integers(0, IN, tokens) if family in ("few",) else np.arange(tokens) % IN
        if family == "slab4":
            slots = (np.arange(tokens) % experts).astype(np.int32)
        elif family == "slab8" or family == "tcgen05":
            slots = ((np.arange(tokens) // IN + call) % 4).astype(np.int32)
        else:
            slots = rng.integers(0, experts, tokens).astype(np.int32)
        x = np.zeros((tokens, IN), dtype=np.float32)
        x[np.arange(tokens), which] = VALUE
        # up holds every code, gate is positive everywhere: G > 0 for all outputs
        got = run(positive, every, x, slots)
        np.testing.assert_array_equal(got, closed_form(w_pos[slots, which] * np.float32(VALUE), w_every[slots, which] * np.float32(VALUE)))
        # gate holds every code: outputs whose gate weight has the activation's sign are exact
        for sign in (1.0, -1.0):
            got = run(every, positive, sign * x, slots)
            g = w_every[slots, which] * np.float32(sign * VALUE)
            want = closed_form(g, w_pos[slots, which] * np.float32(sign * VALUE))
            ok = g >= 40.0
            assert ok.mean() > 0.3
            np.testing.assert_array_equal(got[ok], want[ok])


def test_general_kernel_returns_scale_times_weight_exactly(cuda):
    """``keepvq_routed_matvec`` (int8 dp4a form), fp32 activations and outputs, 16-bit and 8-bit codes."""
    from keep_b200 import kernels, vq

    codes = all_codes_experts()
    scales = scales_for(4, 4)
    want = expected(codes, scales, VALUE)
    x = torch.from_numpy(one_hot_rows()).to(cuda)
    table = vq.table_on(cuda, "e8p")
    for e in range(4):
        rhs = np.full(IN, e, dtype=np.uint32)
        got = kernels.e8p_m1_per_route(x, codes, scales, table, rhs, output_dims=ROWS)
        assert got.dtype == torch.float32
        np.testing.assert_array_equal(got.cpu().numpy(), want[e])
    res_codes = (np.arange(ROWS * CW, dtype=np.int64) % 256).astype(np.uint8).reshape(1, ROWS, CW)
    res_scales = scales_for(1, 5)
    dense = e8.decode_weight_matrix(res_codes[0], res_scales[0].astype(np.float32), code_bits=8)
    got = kernels.e8_1bit_m1_per_route(x, res_codes, res_scales, vq.pair_packed(vq.e8_1bit_packed()), np.zeros(IN, dtype=np.uint32), output_dims=ROWS)
    np.testing.assert_array_equal(got.cpu().numpy(), dense.T * np.float32(VALUE))
