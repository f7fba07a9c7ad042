"""Expert-grouped products over routes sorted by expert (the prefill side of ``gather_vqmm``).

Stands in for the reference's sorted-route kernels: ``gather_vqmm_tiled_down`` /
``gather_vqmm_mma*_blocks`` (``src/ramp/kernels/gather_vqmm.py:597-928``) and the native
``nax_e8p_fp16_sorted_matmul_steel[_m32n64]`` (``src/ramp/kernels/nax.py:330-366,3601-3632``).
"""

from __future__ import annotations

import torch

from .kernels import routed_matvec


def grouped_matmul_sorted(x, codes, scales, table, sorted_rhs, sorted_lhs, *, code_bits: int, tile_descriptors=None):
    """``out[r] = W[sorted_rhs[r]] @ x[sorted_lhs[r]]`` (``x[r]`` when ``sorted_lhs`` is None),
    ``[routes, out]`` in the given order.  ``tile_descriptors`` is accepted for callers that
    pre-build it; the CUDA kernels derive their own tiling from ``sorted_rhs``."""
    del tile_descriptors
    return routed_matvec(x, codes, scales, table, sorted_rhs, lhs=sorted_lhs, x_div=1, code_bits=code_bits)
