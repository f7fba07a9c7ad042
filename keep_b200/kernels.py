"""Kernel-level operators with the names, argument order and error behaviour of ``ramp.kernels``.

* ``vq_qmv``                         ``src/ramp/kernels/vq_qmv.py:163-232``
* ``vq_qmm``                         ``src/ramp/kernels/vq_qmm.py:93-152``
* ``e8p_m1_token_layout/per_route``  ``src/ramp/kernels/e8p_m1.py:134-183``
* ``e8_1bit_m1_token_layout/per_route``  ``src/ramp/kernels/e8_1bit_m1.py:76-97``
* ``e8p_nested_m1_token_layout/per_route``  ``src/ramp/kernels/e8p_nested_m1.py:90-112``

Tensors are torch CUDA tensors (numpy inputs are uploaded).  Output dtype follows the activations:
fp16 -> fp16, bf16 -> bf16, anything else -> fp32 (``vq_qmv.py:40-46``).  Calls enqueue on the
current stream and do not synchronise.  16-bit E8P codes with fp16 / bf16 activations and shapes
that fit (inputs and scale groups in multiples of 256) run on the layer's int8 tensor-core kernels
(``keepvq_grouped_projection``); everything else is one launch of the general kernel
(``keepvq_routed_matvec``), which keeps fp32 rows at 24 bits.
"""

from __future__ import annotations

import torch

from . import _lib
from .vq import (CODEWORD_DIM, NO_RESIDUAL, _code_tensor, _codebook_tensor, as_device, half2_pairs,  # noqa: F401
                 pair_packed)

__all__ = [
    "E8P_MAX_TOKENS", "NO_RESIDUAL", "e8_1bit_m1_per_route", "e8_1bit_m1_token_layout", "e8p_m1_per_route",
    "e8p_m1_token_layout", "e8p_nested_m1_per_route", "e8p_nested_m1_token_layout", "half2_pairs", "pair_packed",
    "routed_matvec", "should_use_e8p_m1", "vq_qmm", "vq_qmv",
]

#: Token rows the few-token kernels are meant for (``e8p_m1.py:40-42``).
E8P_MAX_TOKENS = 32


def qmv_output_dtype(x_dtype: torch.dtype) -> torch.dtype:
    return x_dtype if x_dtype in (torch.float16, torch.bfloat16) else torch.float32


def _activations(x, device=None) -> torch.Tensor:
    x = as_device(x, device)
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        x = x.to(torch.float32)
    return x.contiguous()


def _index_tensor(indices, device, dtype=torch.int32) -> torch.Tensor:
    idx = as_device(indices, device)
    if idx.dtype.is_floating_point or idx.dtype == torch.bool:
        raise ValueError(f"indices must use an integer dtype, found {idx.dtype}")
    if idx.dtype in (torch.uint32, torch.int32):
        return idx.contiguous().view(dtype) if idx.dtype != dtype else idx.contiguous()
    return idx.to(torch.int64).to(dtype).contiguous()  # 0xFFFFFFFF wraps to -1: same bits


def chunk_for(codewords: int, groups: int) -> int:
    """Codewords per wide load; a chunk must not straddle a row or scale group (``e8p_m1.py:98-104``)."""
    for chunk in (8, 4):
        if codewords % groups == 0 and (codewords // groups) % chunk == 0:
            return chunk
    raise ValueError(f"E8P M=1 needs codewords per scale group divisible by 4, got {codewords}/{groups}")


def should_use_e8p_m1(*, code_bits: int, tokens: int, sorted_indices: bool, route_strategy: str) -> bool:
    """The few-token dispatch predicate (``e8p_m1.py:72-83``); there is no opt-out flag here."""
    return code_bits == 16 and 1 <= tokens <= E8P_MAX_TOKENS and not sorted_indices and route_strategy in ("auto", "direct")


def routed_matvec(x, codes, scales, codebook, rhs, *, lhs=None, x_div=1, code_bits, layout=_lib.TABLE_PACKED,
                  residual=None, hot_of_slot=None, out_dtype=None) -> torch.Tensor:
    """One launch of the general routed kernel.  ``x`` [rows, in]; ``codes`` [E, out, in/8];
    ``rhs`` flat uint32/int32 [routes]; returns [routes, out]."""
    device = _lib.require_cuda(x, codes, scales, codebook, rhs)
    experts, out_dim, cw = (int(s) for s in codes.shape)
    groups = int(scales.shape[2])
    routes = int(rhs.numel())
    out_dtype = qmv_output_dtype(x.dtype) if out_dtype is None else out_dtype
    out = torch.empty((routes, out_dim), dtype=out_dtype, device=device)
    args = _lib.MatvecArgs(
        x=_lib.ptr(x), x_dtype=_lib.dtype_tag(x.dtype), x_rows=int(x.shape[0]),
        codes=_lib.ptr(codes), code_bits=code_bits,
        scales=_lib.ptr(scales), scales_dtype=_lib.dtype_tag(scales.dtype),
        experts=experts, out_dim=out_dim, in_dim=cw * 8, groups=groups,
        codebook=_lib.ptr(codebook), codebook_layout=layout,
        rhs=_lib.ptr(rhs), lhs=_lib.ptr(lhs), x_div=int(x_div), routes=routes,
        out=_lib.ptr(out), out_dtype=_lib.dtype_tag(out_dtype),
    )
    keep = [x, codes, scales, codebook, rhs, lhs]
    if residual is not None:
        res_codes, res_scales, res_table = residual
        args.res_codes, args.res_scales = _lib.ptr(res_codes), _lib.ptr(res_scales)
        args.res_scales_dtype = _lib.dtype_tag(res_scales.dtype)
        args.res_rows, args.res_groups = int(res_codes.shape[0]), int(res_scales.shape[2])
        args.res_table, args.hot_of_slot = _lib.ptr(res_table), _lib.ptr(hot_of_slot)
        keep += [res_codes, res_scales, res_table, hot_of_slot]
    with torch.cuda.device(device):
        _lib.check(_lib.load().keepvq_routed_matvec(args, _lib.stream_handle(device)), "keepvq_routed_matvec")
    del keep
    return out


# --- vq_qmv / vq_qmm --------------------------------------------------------------------------

def _validate_qmv(x_shape, codes, scales, codebook, *, in_dim, out_dim, group_size, code_bits, codebook_duplication, rows):
    if code_bits not in (8, 16):
        raise ValueError("code_bits must be 8 or 16")
    if in_dim <= 0 or out_dim <= 0:
        raise ValueError("in_dim and out_dim must be positive")
    if in_dim % CODEWORD_DIM != 0:
        raise ValueError("in_dim must be divisible by 8")
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    if in_dim % group_size != 0:
        raise ValueError("in_dim must be divisible by group_size")
    want_x = (in_dim,) if rows is None else (rows, in_dim)
    if tuple(x_shape) != want_x:
        raise ValueError(f"x must have shape {want_x}, found {tuple(x_shape)}")
    if tuple(codes.shape) != (out_dim, in_dim // CODEWORD_DIM):
        raise ValueError(f"codes must have shape ({out_dim}, {in_dim // CODEWORD_DIM}), found {tuple(codes.shape)}")
    if tuple(scales.shape) != (out_dim, in_dim // group_size):
        raise ValueError(f"scales must have shape ({out_dim}, {in_dim // group_size}), found {tuple(scales.shape)}")
    if codebook_duplication not in (1, 4, 8):
        raise ValueError("codebook_duplication must be 1, 4, or 8")


def _dense_reference(x2d, codes, scales, codebook, code_bits):
    """``implementation="reference"``: materialise the dense matrix with the decode kernel and
    multiply in fp32 on the device (``vq_qmv.py:126-160`` does the same on the host)."""
    from .vq import decode_weight_matrix

    weights = decode_weight_matrix(codes, scales, code_bits=code_bits, codebook=codebook)
    return x2d.to(torch.float32) @ weights.T


def _one_matrix(rows, codes, scales, table, rhs, code_bits):
    """Every row of ``rows`` against the one matrix ``codes``: the int8 tensor-core kernels for
    16-bit codes with fp16 / bf16 rows when the shapes fit them, else the general kernel."""
    out = None
    if code_bits == 16 and rows.dtype in (torch.float16, torch.bfloat16):
        from .prefill import tensor_core_projection

        out = tensor_core_projection(rows, codes[None], scales.contiguous()[None], table, rhs)
    if out is None:
        out = routed_matvec(rows, codes[None], scales.contiguous()[None], table, rhs, x_div=1, code_bits=code_bits)
    return out


def vq_qmv(x, codes, scales, codebook=None, *, in_dim: int, out_dim: int, group_size: int = 512, code_bits: int = 8,
           implementation: str = "cuda", codebook_duplication: int = 1) -> torch.Tensor:
    """``y[n] = sum_k W[n, k] x[k]`` with ``W`` decoded inside the kernel.  ``x`` [in] -> [out].

    ``implementation``: ``"cuda"`` (``"metal"`` is accepted as the same thing, for callers
    written against the reference) or ``"reference"`` (dense decode then fp32 matmul, on the GPU).
    ``codebook_duplication`` is validated and ignored.
    """
    if implementation not in ("cuda", "metal", "reference"):
        raise ValueError("implementation must be 'cuda' ('metal') or 'reference'")
    x_t = _activations(x)
    device = _lib.require_cuda(x_t)
    if code_bits not in (8, 16):
        raise ValueError("code_bits must be 8 or 16")
    codes_t = as_device(codes, device)
    scales_t = as_device(scales, device)
    _validate_qmv(x_t.shape, codes_t, scales_t, codebook, in_dim=in_dim, out_dim=out_dim, group_size=group_size,
                  code_bits=code_bits, codebook_duplication=codebook_duplication, rows=None)
    codes_t = _code_tensor(codes_t, code_bits, device)
    table = _codebook_tensor(codebook, code_bits, device)
    if implementation == "reference":
        return _dense_reference(x_t[None], codes_t, scales_t, table, code_bits)[0]
    rhs = torch.zeros(1, dtype=torch.int32, device=device)
    return _one_matrix(x_t[None], codes_t, scales_t, table, rhs, code_bits)[0]


def vq_qmm(x, codes, scales, codebook=None, *, in_dim: int, out_dim: int, group_size: int = 512, code_bits: int = 8,
           implementation: str = "cuda", codebook_duplication: int = 1) -> torch.Tensor:
    """``Y = X W^T`` for ``X`` [M, in] -> [M, out]; one route per activation row."""
    if implementation not in ("cuda", "metal", "reference"):
        raise ValueError("implementation must be 'cuda' ('metal') or 'reference'")
    x_t = _activations(x)
    device = _lib.require_cuda(x_t)
    if x_t.ndim != 2:
        raise ValueError(f"x must be 2D [batch, in_dim], found {tuple(x_t.shape)}")
    if code_bits not in (8, 16):
        raise ValueError("code_bits must be 8 or 16")
    codes_t = as_device(codes, device)
    scales_t = as_device(scales, device)
    _validate_qmv(x_t.shape, codes_t, scales_t, codebook, in_dim=in_dim, out_dim=out_dim, group_size=group_size,
                  code_bits=code_bits, codebook_duplication=codebook_duplication, rows=int(x_t.shape[0]))
    codes_t = _code_tensor(codes_t, code_bits, device)
    table = _codebook_tensor(codebook, code_bits, device)
    if implementation == "reference":
        return _dense_reference(x_t, codes_t, scales_t, table, code_bits)
    rhs = torch.zeros(int(x_t.shape[0]), dtype=torch.int32, device=device)
    return _one_matrix(x_t, codes_t, scales_t, table, rhs, code_bits)


# --- few-token kernels -------------------------------------------------------------------------

def _check_launch_shape(rows_per_simdgroup: int, simdgroups: int) -> None:
    # Accepted for source compatibility; the CUDA kernel picks its own tiling.
    if rows_per_simdgroup < 1 or simdgroups < 1 or simdgroups > 32:
        raise ValueError("rows_per_simdgroup must be >= 1 and simdgroups in 1..32")


def _few_token(x, codes, scales, codebook, rhs_indices, *, output_dims, code_bits, layout, token_layout, what,
               rows_per_simdgroup, simdgroups, residual=None, hot_of_slot=None):
    x_t = _activations(x)
    device = _lib.require_cuda(x_t)
    rhs_t = as_device(rhs_indices, device)
    if token_layout:
        if x_t.ndim != 2 or rhs_t.ndim != 2 or rhs_t.shape[0] != x_t.shape[0]:
            raise ValueError(f"token-layout {what} needs x [tokens, in] and rhs_indices [tokens, top_k]")
        x_div = int(rhs_t.shape[1])
    else:
        routes = int(rhs_t.numel())
        if x_t.ndim != 2 or x_t.shape[0] != routes:
            raise ValueError(f"per-route {what} needs x [{routes}, in], got {tuple(x_t.shape)}")
        x_div = 1
    _check_launch_shape(rows_per_simdgroup, simdgroups)
    codes_t = as_device(codes, device)
    want = torch.uint8 if code_bits == 8 else torch.uint16
    if codes_t.dtype != want:
        raise ValueError(f"{code_bits}-bit codes must be {'uint8' if code_bits == 8 else 'uint16'}, got {codes_t.dtype}")
    scales_t = as_device(scales, device).contiguous()
    chunk_for(int(codes_t.shape[2]), int(scales_t.shape[2]))
    table = as_device(codebook, device).contiguous()
    flat = _index_tensor(rhs_t.reshape(-1), device)
    out = None
    if code_bits == 16 and x_t.dtype in (torch.float16, torch.bfloat16):
        # 16-bit activations: the layer's own tensor-core kernels when the shapes fit them
        from .prefill import tensor_core_projection

        out = tensor_core_projection(x_t, codes_t.contiguous(), scales_t, table, flat, x_div=x_div, residual=residual, hot_of_slot=hot_of_slot)
    if out is None:
        out = routed_matvec(x_t, codes_t.contiguous(), scales_t, table, flat, x_div=x_div, code_bits=code_bits,
                            layout=layout, residual=residual, hot_of_slot=hot_of_slot)
    if token_layout:
        return out.reshape(int(rhs_t.shape[0]), int(rhs_t.shape[1]), output_dims)
    return out.reshape(int(rhs_t.numel()), output_dims)


def e8p_m1_token_layout(x, codes, scales, codebook, rhs_indices, *, output_dims: int, rows_per_simdgroup: int = 4,
                        simdgroups: int = 1) -> torch.Tensor:
    """Token ``t``'s row against its ``top_k`` experts: ``[tokens, top_k, out]``."""
    return _few_token(x, codes, scales, codebook, rhs_indices, output_dims=output_dims, code_bits=16,
                      layout=_lib.TABLE_PACKED, token_layout=True, what="E8P",
                      rows_per_simdgroup=rows_per_simdgroup, simdgroups=simdgroups)


def e8p_m1_per_route(x, codes, scales, codebook, rhs_indices, *, output_dims: int, rows_per_simdgroup: int = 4,
                     simdgroups: int = 1) -> torch.Tensor:
    """Route ``r``'s activation row against expert ``rhs_indices[r]``: ``[routes, out]``."""
    return _few_token(x, codes, scales, codebook, rhs_indices, output_dims=output_dims, code_bits=16,
                      layout=_lib.TABLE_PACKED, token_layout=False, what="E8P M=1",
                      rows_per_simdgroup=rows_per_simdgroup, simdgroups=simdgroups)


def e8_1bit_m1_token_layout(x, codes, scales, codebook, rhs_indices, *, output_dims: int, rows_per_simdgroup: int = 4,
                            simdgroups: int = 1) -> torch.Tensor:
    """8-bit residual codes, token layout.  ``codebook`` is ``pair_packed(e8_1bit_packed())``;
    a route whose index is ``NO_RESIDUAL`` writes zeros."""
    return _few_token(x, codes, scales, codebook, rhs_indices, output_dims=output_dims, code_bits=8,
                      layout=_lib.TABLE_PAIR_PACKED, token_layout=True, what="E8",
                      rows_per_simdgroup=rows_per_simdgroup, simdgroups=simdgroups)


def e8_1bit_m1_per_route(x, codes, scales, codebook, rhs_indices, *, output_dims: int, rows_per_simdgroup: int = 4,
                         simdgroups: int = 1) -> torch.Tensor:
    """8-bit residual codes, one activation row per route."""
    return _few_token(x, codes, scales, codebook, rhs_indices, output_dims=output_dims, code_bits=8,
                      layout=_lib.TABLE_PAIR_PACKED, token_layout=False, what="E8",
                      rows_per_simdgroup=rows_per_simdgroup, simdgroups=simdgroups)


def _nested(x, base, rhs_indices, residual, hot_of_slot, *, output_dims, token_layout, rows_per_simdgroup, simdgroups):
    (codes, scales, codebook), (res_codes, res_scales, res_table) = base, residual
    x_t = _activations(x)
    device = _lib.require_cuda(x_t)
    codes_t, res_codes_t = as_device(codes, device), as_device(res_codes, device)
    if codes_t.dtype != torch.uint16 or res_codes_t.dtype != torch.uint8:
        raise ValueError(f"nested codes must be uint16 base and uint8 residual, got {codes_t.dtype} and {res_codes_t.dtype}")
    if tuple(codes_t.shape[1:]) != tuple(res_codes_t.shape[1:]):
        raise ValueError(f"base and residual rows differ: {tuple(codes_t.shape[1:])} and {tuple(res_codes_t.shape[1:])}")
    res_table_t = as_device(res_table, device)
    if tuple(res_table_t.shape) != (256, 4) or res_table_t.dtype not in (torch.uint32, torch.int32):
        raise ValueError("the residual table must be half2_pairs(grid): [256, 4] uint32")
    hot_t = as_device(hot_of_slot, device)
    if hot_t.numel() != codes_t.shape[0]:
        raise ValueError(f"hot_of_slot needs one entry per slot, got {hot_t.numel()} for {codes_t.shape[0]}")
    res_scales_t = as_device(res_scales, device).contiguous()
    chunk_for(int(codes_t.shape[2]), int(res_scales_t.shape[2]))
    hot_t = _index_tensor(hot_t.reshape(-1), device)
    return _few_token(x_t, codes_t, scales, codebook, rhs_indices, output_dims=output_dims, code_bits=16,
                      layout=_lib.TABLE_PACKED, token_layout=token_layout, what="nested E8P",
                      rows_per_simdgroup=rows_per_simdgroup, simdgroups=simdgroups,
                      residual=(res_codes_t.contiguous(), res_scales_t, res_table_t.contiguous()), hot_of_slot=hot_t)


def e8p_nested_m1_token_layout(x, base, rhs_indices, residual, hot_of_slot, *, output_dims: int,
                               rows_per_simdgroup: int = 4, simdgroups: int = 1) -> torch.Tensor:
    """Base + residual in one pass, token layout.  ``base`` = (codes, scales, packed abs grid);
    ``residual`` = (uint8 codes, scales, ``half2_pairs`` table); ``hot_of_slot[slot]`` is the
    slot's residual row or ``NO_RESIDUAL``."""
    return _nested(x, base, rhs_indices, residual, hot_of_slot, output_dims=output_dims, token_layout=True,
                   rows_per_simdgroup=rows_per_simdgroup, simdgroups=simdgroups)


def e8p_nested_m1_per_route(x, base, rhs_indices, residual, hot_of_slot, *, output_dims: int,
                            rows_per_simdgroup: int = 4, simdgroups: int = 1) -> torch.Tensor:
    """Base + residual in one pass, one activation row per route."""
    return _nested(x, base, rhs_indices, residual, hot_of_slot, output_dims=output_dims, token_layout=False,
                   rows_per_simdgroup=rows_per_simdgroup, simdgroups=simdgroups)
