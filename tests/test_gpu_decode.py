"""Code-to-weight decode on the GPU: bit-exact against the oracle and the golden fixtures."""

import numpy as np
import pytest
import torch

from oracle import e8

pytestmark = pytest.mark.gpu


def test_all_65536_codewords_decode_bit_exactly(cuda, golden):
    from keep_b200 import vq

    grid = vq.e8p_full_grid(cuda).cpu().numpy()
    np.testing.assert_array_equal(grid, e8.e8p_full_grid())
    np.testing.assert_array_equal(np.round(grid * 4).astype(np.int8), golden("codebooks")["full_grid_quarter_units"])


def test_residual_table_decodes_bit_exactly(cuda):
    from keep_b200 import vq

    codes = torch.arange(256, dtype=torch.int32, device=cuda).to(torch.uint8)
    np.testing.assert_array_equal(vq.decode_e8_1bit(codes).cpu().numpy(), e8.e8_1bit_grid())


def test_golden_weight_matrices(cuda, golden):
    from keep_b200 import vq

    g = golden("codebooks")
    got = vq.decode_weight_matrix(g["codes16"], g["scales16"], code_bits=16)
    np.testing.assert_array_equal(got.cpu().numpy(), g["weights16"])
    got = vq.decode_weight_matrix(g["codes8"], g["scales8"], code_bits=8)
    np.testing.assert_array_equal(got.cpu().numpy(), g["weights8"])


@pytest.mark.parametrize("groups", [1, 8, 64])
def test_scaled_decode_is_exact_for_every_codeword_and_a_scale_sweep(cuda, groups):
    """Every codeword under fp16 scales drawn as the benchmark draws them: exact in fp32."""
    from keep_b200 import vq

    rng = np.random.default_rng(11)
    codes = rng.permutation(1 << 16).astype(np.uint16).reshape(128, 512)
    scales = (0.02 * rng.uniform(0.5, 1.5, size=(128, groups))).astype(np.float16)
    got = vq.decode_weight_matrix(codes, scales, code_bits=16).cpu().numpy()
    np.testing.assert_array_equal(got, e8.decode_weight_matrix(codes, scales, code_bits=16))


def test_custom_codebook_and_bf16_output(cuda):
    from keep_b200 import vq

    rng = np.random.default_rng(12)
    table = rng.integers(0, 1 << 32, size=256, dtype=np.uint64).astype(np.uint32)
    codes = rng.integers(0, 1 << 16, size=(9, 24), dtype=np.uint16)
    got = vq.decode_weight_matrix(codes, None, code_bits=16, codebook=table).cpu().numpy()
    np.testing.assert_array_equal(got, e8.decode_weight_matrix(codes, None, code_bits=16, codebook=table))
    got = vq.decode_weight_matrix(codes, None, code_bits=16, out_dtype=torch.bfloat16).float().cpu().numpy()
    np.testing.assert_array_equal(got, e8.decode_weight_matrix(codes, None, code_bits=16))  # grid values are exact in bf16


def test_empty_and_bad_shapes(cuda):
    from keep_b200 import vq

    empty = torch.zeros((0, 16), dtype=torch.uint16, device=cuda)
    assert tuple(vq.decode_weight_matrix(empty, None, code_bits=16).shape) == (0, 128)
    with pytest.raises(ValueError, match="divisible"):
        vq.decode_weight_matrix(torch.zeros((2, 6), dtype=torch.uint16, device=cuda), torch.ones((2, 4), device=cuda), code_bits=16)
    with pytest.raises(ValueError, match="uint16"):
        vq.decode_weight_matrix(torch.zeros((2, 8), dtype=torch.uint8, device=cuda), None, code_bits=16)
