"""The CPU oracle against the reference's golden vectors (no GPU)."""

import numpy as np

from oracle import e8, ops


def test_tables_match_the_pinned_digests_and_words(golden):
    g = golden("codebooks")
    assert e8.sha256_u32(e8.e8p_packed_abs_grid()) == e8.E8P_PACKED_ABS_SHA256
    assert e8.sha256_u32(e8.e8_1bit_packed()) == e8.E8_1BIT_PACKED_SHA256
    np.testing.assert_array_equal(e8.e8p_packed_abs_grid(), g["e8p_packed_abs"])
    np.testing.assert_array_equal(e8.e8_1bit_packed(), g["e8_1bit_packed"])
    # first and last packed words, as tests/test_e8_reference.py:33-34 of the reference pins them
    assert e8.e8p_packed_abs_grid()[:2].tolist() == g["e8p_packed_abs"][:2].tolist() == [2576980377, 1503238553]
    assert int(e8.e8p_packed_abs_grid()[-1]) == 2073803675


def test_decoders_match_the_reference_golden_codewords(golden):
    g = golden("codebooks")
    np.testing.assert_array_equal(e8.decode_e8p(g["e8p_codes"]), g["e8p_decoded"])
    np.testing.assert_array_equal(e8.e8p_full_grid()[g["e8p_codes"]], g["e8p_decoded"])
    np.testing.assert_array_equal(e8.decode_e8_1bit(g["res_codes"]), g["res_decoded"])
    np.testing.assert_array_equal(np.round(e8.e8p_full_grid() * 4).astype(np.int8), g["full_grid_quarter_units"])
    # code 0 is all +3/4; an odd sign byte shifts down by 1/4 (tests/test_e8_reference.py:40-42)
    np.testing.assert_array_equal(e8.decode_e8p(np.array([0, 1], np.uint16)), [[0.75] * 8, [0.25] * 8])


def test_full_grid_values_are_quarter_multiples_within_range():
    grid = e8.e8p_full_grid()
    assert grid.shape == (65536, 8)
    assert np.array_equal(grid * 4, np.round(grid * 4)) and np.abs(grid).max() == 2.75


def test_decode_weight_matrix_matches_the_reference(golden):
    g = golden("codebooks")
    np.testing.assert_array_equal(e8.decode_weight_matrix(g["codes16"], g["scales16"], code_bits=16), g["weights16"])
    np.testing.assert_array_equal(e8.decode_weight_matrix(g["codes8"], g["scales8"], code_bits=8), g["weights8"])


def test_table_layout_helpers_match_the_reference(golden):
    g = golden("operators")
    np.testing.assert_array_equal(e8.pair_packed(e8.e8_1bit_packed()), g["pair_packed"])
    np.testing.assert_array_equal(e8.half2_pairs(e8.e8_1bit_grid()), g["half2_pairs"])


def test_operator_oracle_matches_the_reference_reference_path(golden):
    g = golden("operators")
    kw = dict(code_bits=16)
    np.testing.assert_allclose(ops.gather_vqmm(g["x"], g["codes"], g["scales"], None, g["rhs"], **kw), g["token"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(ops.gather_vqmm(g["x"], g["codes"], g["scales"], None, g["flat_rhs"], lhs_indices=g["lhs"], **kw),
                               g["routed"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(ops.vq_switch_qmv(g["xr"], g["codes"], g["scales"], None, g["rhs"], **kw), g["per_route"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(ops.vq_qmv_reference(g["x"][0], g["codes"][2], g["scales"][2], code_bits=16), g["qmv"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(ops.gather_vqmm(g["x"], g["codes8"], g["scales"], None, g["rhs"], code_bits=8), g["token8"], rtol=1e-6, atol=1e-6)


def test_projection_byte_accounting():
    # 2048 x 4096 at group 512: 2,129,920 B of codes + fp16 scales (tests/test_e8p_m1.py:187-195)
    assert 2048 * 512 * 2 + 2048 * 8 * 2 == 2_129_920
