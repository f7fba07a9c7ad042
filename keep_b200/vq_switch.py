"""Routed-expert operators: the drop-in boundary.  Names, keywords, shapes and errors follow
``src/ramp/ops/vq_switch.py`` of the reference:

* ``gather_vqmm``                ``vq_switch.py:916-1221``
* ``gather_vqmm_sorted_routes``  ``vq_switch.py:620-913``
* ``vq_switch_qmv``              ``vq_switch.py:547-617``
* ``trace_gather_vqmm_calls``    ``vq_switch.py:75-84``
* ``expert_block_tile_descriptors``  ``vq_switch.py:117-152``

Differences a caller can see: tensors are torch CUDA tensors; ``implementation`` takes ``"cuda"``
(``"metal"`` is an alias) or ``"reference"`` (dense decode + fp32 matmul, still on the GPU);
``codebook_duplication`` is validated and ignored.  Hot kernels do not range-check indices
(``vq_switch.py:637,646-648``); the ``"reference"`` path and ``validate_indices=True`` do.
"""

from __future__ import annotations

from contextlib import contextmanager
from contextvars import ContextVar
from typing import Any, Iterator

import torch

from . import _lib
from .kernels import _activations, _index_tensor, qmv_output_dtype, routed_matvec
from .vq import CODEWORD_DIM, _codebook_tensor, as_device, decode_weight_matrix

__all__ = [
    "expert_block_tile_descriptors", "gather_vqmm", "gather_vqmm_sorted_routes", "trace_gather_vqmm_calls",
    "vq_switch_qmv",
]

#: Routes at or above this go to the expert-sorted path under ``route_strategy="auto"``
#: (``vq_switch.py:44``).
SORTED_TILED_ROUTE_THRESHOLD = 128
_ROUTE_STRATEGIES = ("auto", "direct", "sorted_tiled", "per_route_decoded")
_IMPLEMENTATIONS = ("cuda", "metal", "reference")
_TRACE: ContextVar[list[dict[str, Any]] | None] = ContextVar("gather_vqmm_trace", default=None)


@contextmanager
def trace_gather_vqmm_calls() -> Iterator[list[dict[str, Any]]]:
    """Record each dispatch made inside the block: token rows, routes, dims, code width,
    the strategy chosen and the implementation."""
    records: list[dict[str, Any]] = []
    token = _TRACE.set(records)
    try:
        yield records
    finally:
        _TRACE.reset(token)


def _record(**fields) -> None:
    records = _TRACE.get()
    if records is not None:
        records.append(fields)


def _validate_switch_metadata(x, codes, scales, codebook, indices, *, input_dims, output_dims, group_size, code_bits):
    """Same checks, same order, same messages as ``vq_switch.py:491-544``."""
    if code_bits not in (8, 16):
        raise ValueError("code_bits must be 8 or 16")
    if input_dims <= 0 or output_dims <= 0:
        raise ValueError("input_dims and output_dims must be positive")
    if input_dims % CODEWORD_DIM != 0:
        raise ValueError("input_dims must be divisible by 8")
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    if input_dims % group_size != 0:
        raise ValueError("input_dims must be divisible by group_size")
    if x.shape[-1] != input_dims:
        raise ValueError(f"x trailing dimension must be {input_dims}, found {x.shape[-1]}")
    if indices.ndim < 1:
        raise ValueError("indices must have at least one dimension")
    if tuple(x.shape[:-1]) != tuple(indices.shape[:-1]) and tuple(x.shape[:-1]) != tuple(indices.shape):
        raise ValueError(
            "x leading shape must either match indices leading shape for "
            f"token routing or the full indices shape for per-route routing; found x {tuple(x.shape)} and indices {tuple(indices.shape)}"
        )
    want = torch.uint8 if code_bits == 8 else torch.uint16
    if codes.dtype != want:
        raise ValueError(f"codes dtype must be {'uint8' if code_bits == 8 else 'uint16'}, found {codes.dtype}")
    if codebook.dtype not in (torch.uint32, torch.int32):
        raise ValueError(f"codebook dtype must be uint32, found {codebook.dtype}")
    if tuple(codebook.shape) != (256,):
        raise ValueError(f"codebook must have shape (256,), found {tuple(codebook.shape)}")
    if codes.ndim != 3:
        raise ValueError(f"codes must be 3D [experts, out, in/8], found {tuple(codes.shape)}")
    if scales.ndim != 3:
        raise ValueError(f"scales must be 3D [experts, out, in/group], found {tuple(scales.shape)}")
    experts = int(codes.shape[0])
    want_codes = (experts, output_dims, input_dims // CODEWORD_DIM)
    want_scales = (experts, output_dims, input_dims // group_size)
    if tuple(codes.shape) != want_codes:
        raise ValueError(f"codes must have shape {want_codes}, found {tuple(codes.shape)}")
    if tuple(scales.shape) != want_scales:
        raise ValueError(f"scales must have shape {want_scales}, found {tuple(scales.shape)}")
    return experts, int(indices.shape[-1])


def _prepare(x, codes, scales, codebook, code_bits):
    x_t = _activations(x)
    device = _lib.require_cuda(x_t)
    codes_t = as_device(codes, device)
    scales_t = as_device(scales, device)
    if code_bits not in (8, 16):
        raise ValueError("code_bits must be 8 or 16")
    table = _codebook_tensor(codebook, code_bits, device)
    return x_t, codes_t, scales_t, table, device


def _check_range(values: torch.Tensor, bound: int, what: str) -> None:
    if values.numel():
        lo, hi = int(values.min()), int(values.max())  # host read: only on the checked paths
        if lo < 0 or hi >= bound:
            raise ValueError(f"{what} must be in [0, {bound}), found range [{lo}, {hi}]")


def _dense_routes(x_rows, codes, scales, table, rhs, code_bits):
    """fp32 routes against dense-decoded experts, on the GPU: the ``"reference"`` arm."""
    weights = decode_weight_matrix(codes, scales, code_bits=code_bits, codebook=table)  # [E, out, in]
    return torch.einsum("rk,rnk->rn", x_rows.to(torch.float32), weights[rhs.long()])


def vq_switch_qmv(x, codes, scales, codebook, indices, *, input_dims: int, output_dims: int, group_size: int = 512,
                  code_bits: int = 8, codebook_duplication: int = 1, implementation: str = "cuda",
                  sorted_indices: bool = False) -> torch.Tensor:
    """Selected experts per token/route.  ``x`` leading shape equals ``indices.shape[:-1]`` (token
    routing, result ``[..., top_k, out]``) or ``indices.shape`` (per-route, result ``[..., out]``)."""
    del sorted_indices
    if implementation not in _IMPLEMENTATIONS:
        raise ValueError("implementation must be 'cuda' ('metal') or 'reference'")
    x_t, codes_t, scales_t, table, device = _prepare(x, codes, scales, codebook, code_bits)
    idx = as_device(indices, device)
    experts, top_k = _validate_switch_metadata(x_t, codes_t, scales_t, table, idx, input_dims=input_dims,
                                               output_dims=output_dims, group_size=group_size, code_bits=code_bits)
    per_route = tuple(x_t.shape[:-1]) == tuple(idx.shape)
    flat_x = x_t.reshape(-1, input_dims)
    flat_idx = _index_tensor(idx.reshape(-1), device)
    _check_range(flat_idx, experts, "indices")
    x_div = 1 if per_route else top_k
    if implementation == "reference":
        rows = torch.arange(flat_idx.numel(), device=device) // x_div
        out = _dense_routes(flat_x[rows], codes_t, scales_t, table, flat_idx, code_bits)
    else:
        out = routed_matvec(flat_x, codes_t.contiguous(), scales_t.contiguous(), table, flat_idx, x_div=x_div,
                            code_bits=code_bits)
    if per_route:
        return out.reshape(tuple(x_t.shape[:-1]) + (output_dims,))
    return out.reshape(tuple(x_t.shape[:-1]) + (top_k, output_dims))


def expert_block_tile_descriptors(sorted_rhs: torch.Tensor, *, num_experts: int, route_tile: int = 32):
    """(tile_experts, tile_offsets, tile_counts), int32, for routes sorted by expert: tiles of at
    most ``route_tile`` routes that never span two experts; ``ceil(R / tile) + E`` slots, the
    unused ones with count 0 (``vq_switch.py:117-152``).  Built on the device, no host read."""
    rhs = sorted_rhs.reshape(-1).long()
    routes = int(rhs.numel())
    counts = torch.bincount(rhs, minlength=num_experts)[:num_experts]
    offsets = torch.cumsum(counts, 0) - counts
    tiles_per_expert = (counts + route_tile - 1) // route_tile
    tile_end = torch.cumsum(tiles_per_expert, 0)
    max_tiles = (routes + route_tile - 1) // route_tile + num_experts
    pos = torch.arange(max_tiles, device=rhs.device)
    expert = torch.searchsorted(tile_end, pos, right=True)
    active = expert < num_experts
    expert = torch.where(active, expert, torch.zeros_like(expert))
    local = pos - (tile_end - tiles_per_expert)[expert]
    remaining = counts[expert] - local * route_tile
    tile_counts = torch.where(active, remaining.clamp(0, route_tile), torch.zeros_like(remaining))
    tile_offsets = offsets[expert] + local * route_tile
    return expert.to(torch.int32), tile_offsets.to(torch.int32), tile_counts.to(torch.int32)


def gather_vqmm_sorted_routes(x, codes, scales, codebook, sorted_rhs, sorted_lhs, *, input_dims: int, output_dims: int,
                              group_size: int = 512, code_bits: int = 8, codebook_duplication: int = 8,
                              implementation: str = "cuda", projection: str = "auto", validate_indices: bool = False,
                              tile_descriptors=None, x_pre_sorted: bool = False) -> torch.Tensor:
    """Routes already sorted by expert: ``[routes, out]`` in that same order, no sort, no scatter.

    ``sorted_lhs[r]`` is route ``r``'s activation row in ``x``.  ``x_pre_sorted=True`` declares
    that ``x`` already has one row per route in sorted order, which lets the down projection skip
    the activation gather (``vq_switch.py:687-694``).
    """
    if projection not in ("auto", "gate_up", "down"):
        raise ValueError("projection must be 'auto', 'gate_up', or 'down'")
    if implementation not in _IMPLEMENTATIONS + ("nax_e8", "nax_e8p", "nax_e8p_m32n64"):
        raise ValueError("implementation must be 'cuda' ('metal') or 'reference'")
    x_t, codes_t, scales_t, table, device = _prepare(x, codes, scales, codebook, code_bits)
    rhs = _index_tensor(as_device(sorted_rhs, device).reshape(-1), device)
    lhs = _index_tensor(as_device(sorted_lhs, device).reshape(-1), device)
    if x_t.ndim != 2:
        raise ValueError(f"x must be 2D [tokens_or_routes, input_dims], found {tuple(x_t.shape)}")
    if x_t.shape[1] != input_dims:
        raise ValueError(f"x trailing dimension must be {input_dims}, found {x_t.shape[1]}")
    if rhs.shape != lhs.shape:
        raise ValueError("sorted_rhs and sorted_lhs must have the same flattened shape")
    if codebook_duplication not in (1, 4, 8):
        raise ValueError("codebook_duplication must be 1, 4, or 8")
    routes = int(rhs.numel())
    if routes == 0:
        return torch.zeros((0, output_dims), dtype=x_t.dtype, device=device)
    experts = int(codes_t.shape[0])
    if validate_indices:
        _check_range(rhs, experts, "sorted_rhs")
        _check_range(lhs, int(x_t.shape[0]), "sorted_lhs")
        if routes > 1 and bool((rhs[1:] < rhs[:-1]).any()):
            raise ValueError("sorted_rhs must be sorted nondecreasing by expert id")
    role = ("down" if output_dims >= input_dims else "gate_up") if projection == "auto" else projection
    skip_gather = role == "down" and x_pre_sorted and int(x_t.shape[0]) == routes
    _record(token_rows=int(x_t.shape[0]), route_count=routes, input_dims=input_dims, output_dims=output_dims,
            code_bits=code_bits, strategy="sorted_tiled", implementation=implementation, projection=role)
    if implementation == "reference":
        rows = x_t if skip_gather else x_t[lhs.long()]
        return _dense_routes(rows, codes_t, scales_t, table, rhs, code_bits).to(qmv_output_dtype(x_t.dtype))
    from .prefill import grouped_matmul_sorted

    return grouped_matmul_sorted(x_t, codes_t.contiguous(), scales_t.contiguous(), table, rhs,
                                 None if skip_gather else lhs, code_bits=code_bits, tile_descriptors=tile_descriptors)


def gather_vqmm(x, codes, scales, codebook, rhs_indices, *, lhs_indices=None, input_dims: int, output_dims: int,
                group_size: int = 512, code_bits: int = 8, codebook_duplication: int = 1, implementation: str = "cuda",
                sorted_indices: bool = False, route_strategy: str = "auto") -> torch.Tensor:
    """The routed operator.  ``x`` [tokens, in], ``rhs_indices`` [tokens, top_k] -> [tokens, top_k, out];
    or with ``lhs_indices`` [routes] and flat ``rhs_indices`` -> [routes, out].

    ``route_strategy="auto"``: expert-sorted grouped kernel when ``sorted_indices`` or at least
    128 routes, otherwise the direct few-row kernel.  ``"per_route_decoded"`` names a Metal
    variant of the direct kernel and is served by the same CUDA kernel as ``"direct"``.
    """
    if route_strategy not in _ROUTE_STRATEGIES:
        raise ValueError("route_strategy must be 'auto', 'direct', 'sorted_tiled', or 'per_route_decoded'")
    if implementation not in _IMPLEMENTATIONS:
        raise ValueError("implementation must be 'cuda' ('metal') or 'reference'")
    x_t, codes_t, scales_t, table, device = _prepare(x, codes, scales, codebook, code_bits)
    rhs_t = as_device(rhs_indices, device)
    if x_t.ndim != 2:
        raise ValueError(f"x must be 2D [tokens, hidden], found {tuple(x_t.shape)}")
    if rhs_t.ndim not in (1, 2):
        raise ValueError(f"rhs_indices must be 1D or 2D, found {tuple(rhs_t.shape)}")
    flat_rhs = _index_tensor(rhs_t.reshape(-1), device)
    if lhs_indices is not None:
        flat_lhs = _index_tensor(as_device(lhs_indices, device).reshape(-1), device)
        if flat_lhs.shape != flat_rhs.shape:
            raise ValueError("lhs_indices and rhs_indices must have the same flattened shape")
        output_shape, x_div = (int(flat_rhs.numel()), output_dims), 1
    else:
        if rhs_t.ndim != 2:
            raise ValueError("rhs_indices must be 2D [tokens, top_k] when lhs_indices is not provided")
        if rhs_t.shape[0] != x_t.shape[0]:
            raise ValueError(f"rhs_indices token dimension {rhs_t.shape[0]} must match x token dimension {x_t.shape[0]}")
        flat_lhs, x_div = None, int(rhs_t.shape[1])
        output_shape = (int(x_t.shape[0]), x_div, output_dims)
    if lhs_indices is None:
        _validate_switch_metadata(x_t, codes_t, scales_t, table, rhs_t, input_dims=input_dims, output_dims=output_dims,
                                  group_size=group_size, code_bits=code_bits)
    else:
        _validate_lhs_metadata(x_t, codes_t, scales_t, table, input_dims=input_dims, output_dims=output_dims,
                               group_size=group_size, code_bits=code_bits)
    routes = int(flat_rhs.numel())
    strategy = route_strategy
    if strategy == "auto":
        strategy = "sorted_tiled" if (sorted_indices or routes >= SORTED_TILED_ROUTE_THRESHOLD) else "direct"
    if strategy == "per_route_decoded":
        strategy = "direct"
    _record(token_rows=int(x_t.shape[0]), route_count=routes, input_dims=input_dims, output_dims=output_dims,
            code_bits=code_bits, strategy=strategy, implementation=implementation)
    if routes == 0:
        return torch.zeros(output_shape, dtype=qmv_output_dtype(x_t.dtype), device=device)

    if implementation == "reference":
        _check_range(flat_rhs, int(codes_t.shape[0]), "indices")
        rows = flat_lhs.long() if flat_lhs is not None else torch.arange(routes, device=device) // x_div
        if flat_lhs is not None:
            _check_range(flat_lhs, int(x_t.shape[0]), "lhs_indices")
        return _dense_routes(x_t[rows], codes_t, scales_t, table, flat_rhs, code_bits).reshape(output_shape)

    if strategy == "direct":
        out = None
        if code_bits == 16 and flat_lhs is None and x_t.dtype in (torch.float16, torch.bfloat16):
            # token layout with 16-bit rows: the int8 tensor-core kernels, which group the routes by
            # expert on the device and read each touched expert's codes once
            from .prefill import tensor_core_projection

            out = tensor_core_projection(x_t, codes_t.contiguous(), scales_t.contiguous(), table, flat_rhs, x_div=x_div)
        if out is None:
            out = routed_matvec(x_t, codes_t.contiguous(), scales_t.contiguous(), table, flat_rhs, lhs=flat_lhs,
                                x_div=x_div, code_bits=code_bits)
        return out.reshape(output_shape)

    # sorted_tiled: sort routes by expert on the device, run the grouped kernel, undo the sort.
    lhs_rows = flat_lhs if flat_lhs is not None else (torch.arange(routes, device=device, dtype=torch.int32) // x_div)
    if sorted_indices:  # the caller vouches that rhs is already nondecreasing
        order, sorted_rhs, sorted_lhs = None, flat_rhs, lhs_rows
    else:
        order = torch.argsort(flat_rhs.long(), stable=True)
        sorted_rhs, sorted_lhs = flat_rhs[order], lhs_rows[order]
    routed = gather_vqmm_sorted_routes(x_t, codes_t, scales_t, table, sorted_rhs, sorted_lhs, input_dims=input_dims,
                                       output_dims=output_dims, group_size=group_size, code_bits=code_bits,
                                       implementation=implementation)
    if order is not None:
        unsorted = torch.empty_like(routed)
        unsorted[order] = routed
        routed = unsorted
    return routed.reshape(output_shape)


def _validate_lhs_metadata(x, codes, scales, codebook, *, input_dims, output_dims, group_size, code_bits):
    """The shape checks of ``_validate_switch_metadata`` that still apply when activation rows
    are named by ``lhs_indices`` (x's leading shape is then unrelated to the index shape)."""
    if input_dims <= 0 or output_dims <= 0:
        raise ValueError("input_dims and output_dims must be positive")
    if input_dims % CODEWORD_DIM != 0:
        raise ValueError("input_dims must be divisible by 8")
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    if input_dims % group_size != 0:
        raise ValueError("input_dims must be divisible by group_size")
    if x.shape[-1] != input_dims:
        raise ValueError(f"x trailing dimension must be {input_dims}, found {x.shape[-1]}")
    want = torch.uint8 if code_bits == 8 else torch.uint16
    if codes.dtype != want:
        raise ValueError(f"codes dtype must be {'uint8' if code_bits == 8 else 'uint16'}, found {codes.dtype}")
    if codes.ndim != 3 or tuple(codes.shape[1:]) != (output_dims, input_dims // CODEWORD_DIM):
        raise ValueError(f"codes must have shape (experts, {output_dims}, {input_dims // CODEWORD_DIM}), found {tuple(codes.shape)}")
    if scales.ndim != 3 or tuple(scales.shape) != (int(codes.shape[0]), output_dims, input_dims // group_size):
        raise ValueError(f"scales must have shape ({int(codes.shape[0])}, {output_dims}, {input_dims // group_size}), found {tuple(scales.shape)}")
