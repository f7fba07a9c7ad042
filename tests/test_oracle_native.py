"""The C restatement of the decode against the numpy one and the reference's own outputs."""

import numpy as np

from oracle import e8, native, ops


def test_every_e8p_codeword_matches_numpy_and_the_reference(golden):
    table = e8.e8p_packed_abs_grid()
    codes = np.arange(65536, dtype=np.uint16)
    got = native.decode_e8p(codes, table)
    assert np.array_equal(got, e8.decode_e8p(codes))
    g = golden("codebooks")  # decoded by the reference itself: all 65,536 codewords in quarter units, and its golden vectors
    assert np.array_equal(np.round(got * 4).astype(np.int8), g["full_grid_quarter_units"]) and np.array_equal(got * 4, np.round(got * 4))
    assert np.array_equal(native.decode_e8p(g["e8p_codes"], g["e8p_packed_abs"]), g["e8p_decoded"])
    assert np.array_equal(native.decode_e8_1bit(g["res_codes"], g["e8_1bit_packed"]), g["res_decoded"])


def test_every_residual_codeword_matches_numpy():
    codes = np.arange(256, dtype=np.uint8)
    assert np.array_equal(native.decode_e8_1bit(codes, e8.e8_1bit_packed()), e8.decode_e8_1bit(codes))


def test_matvec_matches_the_numpy_reference_path():
    rng = np.random.default_rng(5)
    codes = rng.integers(0, 1 << 16, (48, 64), dtype=np.uint16)
    scales = (0.02 * rng.uniform(0.5, 1.5, (48, 4))).astype(np.float16)
    x = rng.normal(size=512).astype(np.float32)
    want = ops.vq_qmv_reference(x, codes, scales, None, code_bits=16)
    got = native.vq_qmv(x, codes, scales.astype(np.float32), e8.e8p_packed_abs_grid())
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
