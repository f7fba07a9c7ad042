"""KEEP's E8 codebooks and the code-to-weight decode, on the GPU.

Mirrors the public names of the reference's ``keep.vq`` (``src/keep/vq/__init__.py:3-33``):
``e8p_packed_abs_grid``, ``e8_1bit_packed``, ``e8_1bit_grid``, ``e8p_full_grid``, ``decode_e8p``,
``decode_e8_1bit``, ``decode_weight_matrix``; plus the two table layouts the few-token kernels
take, ``pair_packed`` (``src/ramp/kernels/e8_1bit_m1.py:25-33``) and ``half2_pairs``
(``src/ramp/kernels/e8p_nested_m1.py:29-36``).

The two 256-word tables ship as files (``data/*.u32``) and are verified against the digests the
reference pins.  Decoding runs in ``libkeepvq.so``; tensors in and out are CUDA tensors.
"""

from __future__ import annotations

import hashlib
from functools import lru_cache
from pathlib import Path

import numpy as np
import torch

from . import _lib

CODEWORD_DIM = 8
NO_RESIDUAL = _lib.NO_RESIDUAL
E8P_PACKED_ABS_SHA256 = "efc2c03c60acd955dc812ff2bade9ec6cc31259807e48473506161f3a9a230ce"
E8_1BIT_PACKED_SHA256 = "b78586631069e239d29c146538722d763f4a0040d59a800e8c918ecef03e2180"
_DATA = Path(__file__).resolve().parent / "data"


def _load_table(name: str, digest: str) -> np.ndarray:
    raw = (_DATA / name).read_bytes()
    if hashlib.sha256(raw).hexdigest() != digest:
        raise RuntimeError(f"{name} does not match the pinned codebook digest")
    table = np.frombuffer(raw, dtype="<u4").astype(np.uint32)
    table.setflags(write=False)
    return table


@lru_cache(maxsize=None)
def e8p_packed_abs_grid() -> np.ndarray:
    """uint32[256]: the E8P abs table, eight ``2*value + 8`` nibbles per word (host array)."""
    return _load_table("e8p_packed_abs.u32", E8P_PACKED_ABS_SHA256)


@lru_cache(maxsize=None)
def e8_1bit_packed() -> np.ndarray:
    """uint32[256]: the 8-bit residual table, nibble d = dim d (host array)."""
    return _load_table("e8_1bit_packed.u32", E8_1BIT_PACKED_SHA256)


@lru_cache(maxsize=None)
def e8_1bit_grid() -> np.ndarray:
    """float32[256, 8]: the residual table unpacked (host array; 256 rows, built once)."""
    t = e8_1bit_packed()
    cols = [(((t >> np.uint32(4 * d)) & np.uint32(0xF)).astype(np.int16) - 8) for d in range(8)]
    grid = np.stack(cols, axis=-1).astype(np.float32) * np.float32(0.5)
    grid.setflags(write=False)
    return grid


def pair_packed(packed) -> np.ndarray:
    """Residual table with dims 2k, 2k+1 moved to nibbles k, k+4 (host array, uint32[256])."""
    p = np.asarray(packed, dtype=np.uint32)
    out = np.zeros(256, dtype=np.uint32)
    for k in range(4):
        out |= ((p >> np.uint32(8 * k)) & np.uint32(0xF)) << np.uint32(4 * k)
        out |= ((p >> np.uint32(8 * k + 4)) & np.uint32(0xF)) << np.uint32(16 + 4 * k)
    return out


def half2_pairs(grid) -> np.ndarray:
    """[256, 8] codebook -> uint32[256, 4]: word k = fp16 bits of dim 2k | dim 2k+1 << 16."""
    g = np.asarray(grid)
    h = g.astype(np.float16)
    if h.shape != (256, 8) or not np.array_equal(h.astype(np.float64), g.astype(np.float64)):
        raise ValueError("codebook not exact in float16")
    bits = h.view(np.uint16).astype(np.uint32)
    return np.ascontiguousarray(bits[:, 0::2] | (bits[:, 1::2] << 16))


def default_codebook(code_bits: int) -> np.ndarray:
    """The table a ``codebook=None`` argument stands for (``src/ramp/ops/vq_switch.py:105-108``)."""
    return e8_1bit_packed() if code_bits == 8 else e8p_packed_abs_grid()


_device_tables: dict[tuple, torch.Tensor] = {}


def table_on(device: torch.device, which: str) -> torch.Tensor:
    """A default table as a device tensor, uploaded once per device.  ``which``: ``e8p``,
    ``e8_1bit``, ``e8_1bit_pairs`` (pair-packed) or ``e8_1bit_half2`` ([256, 4])."""
    key = (str(device), which)
    if key not in _device_tables:
        host = {
            "e8p": e8p_packed_abs_grid,
            "e8_1bit": e8_1bit_packed,
            "e8_1bit_pairs": lambda: pair_packed(e8_1bit_packed()),
            "e8_1bit_half2": lambda: half2_pairs(e8_1bit_grid()),
        }[which]()
        _device_tables[key] = as_device(host, device)
    return _device_tables[key]


def as_device(array, device: torch.device | None = None) -> torch.Tensor:
    """A torch CUDA tensor for ``array`` (a torch tensor or anything numpy accepts).  uint16 and
    uint32 keep their dtype."""
    if isinstance(array, torch.Tensor):
        if device is not None and array.device != device:
            return array.to(device)
        return array
    host = np.ascontiguousarray(np.asarray(array))
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return torch.from_numpy(host.copy() if not host.flags.writeable else host).to(device)


def _code_tensor(codes, code_bits: int, device) -> torch.Tensor:
    codes = as_device(codes, device)
    want = torch.uint8 if code_bits == 8 else torch.uint16
    if codes.dtype != want:
        name = "uint8" if code_bits == 8 else "uint16"
        raise ValueError(f"codes dtype must be {name}, found {codes.dtype}")
    return codes.contiguous()


def _codebook_tensor(codebook, code_bits: int, device) -> torch.Tensor:
    if codebook is None:
        return table_on(device, "e8_1bit" if code_bits == 8 else "e8p")
    table = as_device(codebook, device)
    if table.dtype not in (torch.uint32, torch.int32):
        raise ValueError(f"codebook dtype must be uint32, found {table.dtype}")
    if tuple(table.shape) != (256,):
        raise ValueError(f"codebook must have shape (256,), found {tuple(table.shape)}")
    return table.contiguous()


def decode_weight_matrix(codes, scales=None, *, code_bits: int = 8, codebook=None,
                         out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """codes [..., in/8] (+ scales [..., groups]) -> weights [..., in] on the GPU.

    Same contract as ``keep.vq.e8.decode_weight_matrix`` (``src/keep/vq/e8.py:542-571``); an
    fp32 result is bit-identical to it.
    """
    if code_bits not in (8, 16):
        raise ValueError("code_bits must be 8 or 16")
    device = codes.device if isinstance(codes, torch.Tensor) else None
    codes_t = _code_tensor(codes, code_bits, device)
    device = _lib.require_cuda(codes_t)
    table = _codebook_tensor(codebook, code_bits, device)
    lead, cw = tuple(codes_t.shape[:-1]), int(codes_t.shape[-1])
    rows = int(np.prod(lead)) if lead else 1
    groups, scales_t = 1, None
    if scales is not None:
        scales_t = as_device(scales, device).contiguous()
        if tuple(scales_t.shape[:-1]) != lead:
            raise ValueError("scales leading shape must match codes")
        groups = int(scales_t.shape[-1])
        if groups == 0 or cw % groups != 0:
            raise ValueError("codeword count must be divisible by scale count")
    out = torch.empty(lead + (cw * 8,), dtype=out_dtype, device=device)
    args = _lib.DecodeArgs(
        codes=_lib.ptr(codes_t), code_bits=code_bits,
        scales=_lib.ptr(scales_t), scales_dtype=_lib.dtype_tag(scales_t.dtype) if scales_t is not None else 0,
        codebook=_lib.ptr(table), rows=rows, codewords=cw, groups=groups,
        out=_lib.ptr(out), out_dtype=_lib.dtype_tag(out_dtype),
    )
    with torch.cuda.device(device):
        _lib.check(_lib.load().keepvq_decode_weights(args, _lib.stream_handle(device)), "keepvq_decode_weights")
    return out


def decode_e8p(codewords, packed_abs_grid=None) -> torch.Tensor:
    """uint16 codes [...] -> float32 [..., 8] (``src/keep/vq/e8.py:210-234``)."""
    codes_t = _code_tensor(codewords, 16, codewords.device if isinstance(codewords, torch.Tensor) else None)
    flat = decode_weight_matrix(codes_t.reshape(-1, 1), None, code_bits=16, codebook=packed_abs_grid)
    return flat.reshape(tuple(codes_t.shape) + (8,))


def decode_e8_1bit(codes, packed_codebook=None) -> torch.Tensor:
    """uint8 codes [...] -> float32 [..., 8] (``src/keep/vq/e8.py:186-200``)."""
    codes_t = _code_tensor(codes, 8, codes.device if isinstance(codes, torch.Tensor) else None)
    flat = decode_weight_matrix(codes_t.reshape(-1, 1), None, code_bits=8, codebook=packed_codebook)
    return flat.reshape(tuple(codes_t.shape) + (8,))


def e8p_full_grid(device=None) -> torch.Tensor:
    """All 65,536 E8P codewords decoded on the GPU: float32 [65536, 8] (``e8.py:237-241``)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    codes = torch.arange(1 << 16, dtype=torch.int32, device=device).to(torch.uint16)
    return decode_e8p(codes)
