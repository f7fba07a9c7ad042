"""Expert-grouped products over routes sorted by expert (the prefill side of ``gather_vqmm``).

Stands in for the reference's sorted-route kernels: ``gather_vqmm_tiled_down`` /
``gather_vqmm_mma*_blocks`` (``src/ramp/kernels/gather_vqmm.py:597-928``) and the native
``nax_e8p_fp16_sorted_matmul_steel[_m32n64]`` (``src/ramp/kernels/nax.py:330-366,3601-3632``).

16-bit E8P codes with fp16 / bf16 activations whose shapes fit go to ``keepvq_grouped_projection``
(int8 tensor cores: the tcgen05 kernel from 24 routes per expert on, the mma.sync ones below);
everything else (fp32 activations, 8-bit codes, odd shapes, custom tables with even nibbles) to the
general routed kernel.
"""

from __future__ import annotations

import torch

from . import _lib
from .kernels import qmv_output_dtype, routed_matvec

_UNSUPPORTED = -5  # KEEPVQ_ERR_UNSUPPORTED
_all_odd: dict = {}     # table data_ptr -> (the tensor, its version, every nibble odd): read back once per table, never per call
_workspaces: dict = {}  # (device, routes, in_dim) -> scratch tensor; the most recent shapes only
_MAX_CACHED = 8


def _table_all_odd(table: torch.Tensor) -> bool:
    """Whether every nibble of the table is odd (what the int8 kernels need).  The cache holds the
    tensor itself, so its address cannot be handed to another table while the entry lives, and an
    in-place change of the table (a new version) is looked at again."""
    key = (table.data_ptr(), str(table.device))
    hit = _all_odd.get(key)
    if hit is None or hit[0] is not table or hit[1] != table._version:
        nibbles = (table.cpu().to(torch.int64) & 0xFFFFFFFF)[:, None] >> (4 * torch.arange(8))[None] & 1
        if len(_all_odd) >= _MAX_CACHED:
            _all_odd.pop(next(iter(_all_odd)))
        _all_odd[key] = (table, table._version, bool(nibbles.all()))
    return _all_odd[key][2]


def tensor_core_projection(rows, codes, scales, table, rhs, *, x_div: int = 1, residual=None, hot_of_slot=None):
    """``keepvq_grouped_projection``: route ``r`` against activation row ``r // x_div`` of ``rows``
    (fp16 / bf16), optionally with a nested residual ``(res_codes, res_scales, res_table)``.
    Returns None when the library says these shapes are not for the tensor-core kernels."""
    routes, in_dim = int(rhs.numel()), int(rows.shape[1])
    slots, out_dim, groups = int(codes.shape[0]), int(codes.shape[1]), int(scales.shape[2])
    if codes.dtype != torch.uint16 or in_dim % 256 or rows.dtype not in (torch.float16, torch.bfloat16):
        return None
    if int(rows.shape[0]) * x_div != routes:
        return None
    lib = _lib.load()
    device = rows.device
    key = (str(device), routes, in_dim)
    if key not in _workspaces:
        nbytes = int(lib.keepvq_grouped_projection_workspace_bytes(routes, in_dim))
        if nbytes < 0:
            _lib.check(nbytes, "keepvq_grouped_projection_workspace_bytes")
        if len(_workspaces) >= _MAX_CACHED:  # varying route counts must not pile up scratch
            _workspaces.pop(next(iter(_workspaces)))
        _workspaces[key] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    ws = _workspaces[key]
    out_dtype = qmv_output_dtype(rows.dtype)
    out = torch.empty((routes, out_dim), dtype=out_dtype, device=device)
    rows, rhs = rows.contiguous(), rhs.to(torch.int32).contiguous()
    args = _lib.GroupedProjectionArgs(
        x=_lib.ptr(rows), x_dtype=_lib.dtype_tag(rows.dtype), routes=routes, rhs=_lib.ptr(rhs), codes=_lib.ptr(codes), scales=_lib.ptr(scales),
        scales_dtype=_lib.dtype_tag(scales.dtype), slots=slots, out_dim=out_dim, in_dim=in_dim, groups=groups, codebook=_lib.ptr(table),
        codebook_all_odd=int(_table_all_odd(table)), out=_lib.ptr(out), out_dtype=_lib.dtype_tag(out_dtype),
        workspace=_lib.ptr(ws), workspace_bytes=int(ws.numel()), x_div=int(x_div))
    keep = [rows, rhs]
    if residual is not None:
        res_codes, res_scales, res_table = residual
        if res_scales.dtype != scales.dtype:
            return None
        args.res_codes, args.res_scales, args.res_table = _lib.ptr(res_codes), _lib.ptr(res_scales), _lib.ptr(res_table)
        args.res_rows, args.res_groups, args.hot_of_slot = int(res_codes.shape[0]), int(res_scales.shape[2]), _lib.ptr(hot_of_slot)
        keep += [res_codes, res_scales, res_table, hot_of_slot]
    with torch.cuda.device(device):
        status = lib.keepvq_grouped_projection(args, _lib.stream_handle(device))
    del keep
    if status == _UNSUPPORTED:
        return None
    _lib.check(status, "keepvq_grouped_projection")
    return out


def grouped_matmul_sorted(x, codes, scales, table, sorted_rhs, sorted_lhs, *, code_bits: int, tile_descriptors=None):
    """``out[r] = W[sorted_rhs[r]] @ x[sorted_lhs[r]]`` (``x[r]`` when ``sorted_lhs`` is None),
    ``[routes, out]`` in the given order.  ``tile_descriptors`` is accepted for callers that
    pre-build it; the CUDA kernels derive their own grouping from ``sorted_rhs``."""
    del tile_descriptors
    if code_bits == 16 and x.dtype in (torch.float16, torch.bfloat16) and scales.dtype in (torch.float32, torch.float16, torch.bfloat16):
        rows = x if sorted_lhs is None else x[sorted_lhs.long()]  # the gather the reference does before its kernels
        out = tensor_core_projection(rows, codes, scales, table, sorted_rhs)
        if out is not None:
            return out
    return routed_matvec(x, codes, scales, table, sorted_rhs, lhs=sorted_lhs, x_div=1, code_bits=code_bits)
