"""E8P (16-bit) and E8 1-bit (8-bit) codebooks and decoders, restated in numpy.

TEST INFRASTRUCTURE: the checker for the CUDA kernels, never the thing shipped or measured.

Follows ``src/keep/vq/e8.py`` of the reference (QuIP# lattice codebooks):

* table construction   ``e8.py:88-100`` (nibble packing), ``:111-139`` (E8P abs table),
  ``:145-183`` (1-bit residual table)
* decoders             ``e8.py:186-200`` (8-bit), ``:203-234`` (16-bit), ``:542-571`` (matrix)
* table layouts the few-token kernels take: ``src/ramp/kernels/e8_1bit_m1.py:25-33``
  (``pair_packed``) and ``src/ramp/kernels/e8p_nested_m1.py:29-36`` (``half2_pairs``)

All values are held in "half units" (twice the real value) as small integers, so decode is exact.
"""

from __future__ import annotations

import hashlib
import itertools
from functools import lru_cache

import numpy as np

CODEWORD_DIM = 8
#: Digests pinned by the reference, ``tests/test_e8_reference.py:25-26``.
E8P_PACKED_ABS_SHA256 = "efc2c03c60acd955dc812ff2bade9ec6cc31259807e48473506161f3a9a230ce"
E8_1BIT_PACKED_SHA256 = "b78586631069e239d29c146538722d763f4a0040d59a800e8c918ecef03e2180"
#: Output dimension d of a 16-bit codeword reads nibble SHUFFLE[d] of its table word (``e8.py:22``).
E8P_SHUFFLE = (0, 4, 1, 5, 2, 6, 3, 7)
NO_RESIDUAL = 0xFFFFFFFF

# The 29 norm-12 padding rows of the E8P table (``e8.py:25-58``, QuIP# appendix C.1) have five
# components of 3/2 and three of 1/2.  Bit i of each byte marks a 1/2 at component i.
_E8P_PAD_HALF_POSITIONS = bytes([
    0x0E, 0x0D, 0x0B, 0x07, 0xC8, 0xA8, 0x98, 0x68, 0x58, 0x38, 0xC4, 0xA4, 0x94, 0x64, 0x54,
    0x34, 0xC2, 0xA2, 0x92, 0x62, 0x52, 0x31, 0xC1, 0xA1, 0x91, 0x61, 0x51, 0x13, 0x8C,
])


def sha256_u32(words: np.ndarray) -> str:
    """Digest of a uint32 table over its little-endian bytes (``e8.py:84-85``)."""
    return hashlib.sha256(np.asarray(words, dtype="<u4").tobytes()).hexdigest()


def pack_nibbles(half_units: np.ndarray) -> np.ndarray:
    """[n, 8] integers in half units -> uint32[n]; nibble d holds ``value + 8`` (``e8.py:88-100``)."""
    v = np.asarray(half_units, dtype=np.int64)
    assert v.ndim == 2 and v.shape[1] == CODEWORD_DIM
    nib = v + 8
    if nib.min() < 0 or nib.max() > 15:
        raise ValueError("half-unit values must lie in [-8, 7]")
    out = np.zeros(v.shape[0], dtype=np.uint32)
    for d in range(CODEWORD_DIM):
        out |= (nib[:, d].astype(np.uint32) << np.uint32(4 * d))
    return out


def unpack_nibbles(words: np.ndarray) -> np.ndarray:
    """uint32[...] -> int16[..., 8] half-unit values (``e8.py:103-108``)."""
    w = np.asarray(words, dtype=np.uint32)
    out = np.empty(w.shape + (CODEWORD_DIM,), dtype=np.int16)
    for d in range(CODEWORD_DIM):
        out[..., d] = ((w >> np.uint32(4 * d)) & np.uint32(0xF)).astype(np.int16) - 8
    return out


@lru_cache(maxsize=None)
def e8p_packed_abs_grid() -> np.ndarray:
    """The 256-word E8P table (``e8.py:111-139``).

    227 rows of odd half-unit magnitudes {1,3,5,7}^8 with squared sum <= 40, in lexicographic
    order, then the 29 padding rows; columns reordered to [0,2,4,6,1,3,5,7]; a row whose sum is
    2 mod 4 has its last stored column negated; packed as nibbles.
    """
    rows = [r for r in itertools.product((1, 3, 5, 7), repeat=8) if sum(c * c for c in r) <= 40]
    assert len(rows) == 227
    for mask in _E8P_PAD_HALF_POSITIONS:
        rows.append(tuple(1 if (mask >> i) & 1 else 3 for i in range(8)))
    table = np.array(rows, dtype=np.int64)[:, [0, 2, 4, 6, 1, 3, 5, 7]]
    flip = (table.sum(axis=1) % 4) == 2
    table[flip, 7] *= -1
    packed = pack_nibbles(table)
    packed.setflags(write=False)
    return packed


@lru_cache(maxsize=None)
def e8_1bit_packed() -> np.ndarray:
    """The 256-word residual table (``e8.py:145-183``).

    E8 points of norm <= 2: integer rows in {-1,0,1}^8 with at most two non-zeros and an even
    sum (doubled into half units), then the all-(+-1/2) rows whose half-unit sum is 0 mod 4,
    then 15 of the 16 axis points of length 2 (the -2 on the last axis does not fit).
    """
    rows: list[tuple[int, ...]] = []
    for r in itertools.product((-1, 0, 1), repeat=8):
        if sum(c * c for c in r) <= 2 and sum(r) % 2 == 0:
            rows.append(tuple(2 * c for c in r))
    for r in itertools.product((-1, 1), repeat=8):
        if sum(r) % 4 == 0:
            rows.append(r)
    for sign in (4, -4):
        for axis in range(8):
            if sign < 0 and axis == 7:
                continue
            rows.append(tuple(sign if i == axis else 0 for i in range(8)))
    table = np.array(rows, dtype=np.int64)
    assert table.shape == (256, 8), table.shape
    packed = pack_nibbles(table)
    packed.setflags(write=False)
    return packed


def _as_table(table, default) -> np.ndarray:
    t = default() if table is None else np.asarray(table, dtype=np.uint32)
    if t.shape != (256,):
        raise ValueError("a packed codebook must have shape [256]")
    return t


def decode_e8_1bit(codes, packed_codebook=None) -> np.ndarray:
    """uint8 codes [...] -> float32 [..., 8]: nibble d of the table word, minus 8, halved
    (``e8.py:186-200``).  No shuffle, no parity, no shift."""
    table = _as_table(packed_codebook, e8_1bit_packed)
    c = np.asarray(codes, dtype=np.uint8)
    return unpack_nibbles(table[c]).astype(np.float32) * np.float32(0.5)


def decode_e8p(codewords, packed_abs_grid=None) -> np.ndarray:
    """uint16 codes [...] -> float32 [..., 8] (``e8.py:210-234``).

    Low byte: sign bits.  High byte: row of the abs table.  The parity of the sign byte flips
    sign bit 0 and picks the shift: +1/4 for even, -1/4 for odd.  Output dimension d takes
    nibble SHUFFLE[d] and sign bit SHUFFLE[d].
    """
    table = _as_table(packed_abs_grid, e8p_packed_abs_grid)
    c = np.asarray(codewords, dtype=np.uint16)
    flat = c.reshape(-1).astype(np.uint32)
    signs = flat & 0xFF
    parity = np.zeros_like(signs)
    for b in range(8):
        parity ^= (signs >> b) & 1
    eff = signs ^ parity
    word = table[flat >> 8]
    quarter = np.empty((flat.shape[0], 8), dtype=np.int32)  # values in quarter units, exact
    for d, p in enumerate(E8P_SHUFFLE):
        half = ((word >> np.uint32(4 * p)) & 0xF).astype(np.int32) - 8
        neg = ((eff >> np.uint32(p)) & 1).astype(bool)
        half = np.where(neg, -half, half)
        quarter[:, d] = 2 * half + np.where(parity.astype(bool), -1, 1)
    out = quarter.astype(np.float32) * np.float32(0.25)
    return out.reshape(c.shape + (8,))


@lru_cache(maxsize=None)
def e8p_full_grid() -> np.ndarray:
    """All 65,536 codewords decoded, [65536, 8] float32 (``e8.py:237-241``)."""
    g = decode_e8p(np.arange(1 << 16, dtype=np.uint32).astype(np.uint16))
    g.setflags(write=False)
    return g


@lru_cache(maxsize=None)
def e8_1bit_grid() -> np.ndarray:
    """The residual table unpacked, [256, 8] float32 (``e8.py:176-180``)."""
    g = unpack_nibbles(e8_1bit_packed()).astype(np.float32) * np.float32(0.5)
    g.setflags(write=False)
    return g


def decode_weight_matrix(codes, scales=None, *, code_bits=8, codebook=None) -> np.ndarray:
    """codes [..., in/8] (+ scales [..., groups]) -> float32 weights [..., in] (``e8.py:542-571``).

    Each scale covers ``codewords / groups`` consecutive codewords of its row.  The product of a
    grid value (4 significant bits) and a float16 scale is exact in float32.
    """
    if code_bits == 8:
        dec = decode_e8_1bit(codes, codebook)
    elif code_bits == 16:
        dec = decode_e8p(codes, codebook)
    else:
        raise ValueError("code_bits must be 8 or 16")
    if scales is not None:
        s = np.asarray(scales).astype(np.float32)
        cw = dec.shape[-2]
        if cw % s.shape[-1] != 0:
            raise ValueError("codeword count must be divisible by scale count")
        dec = dec * np.repeat(s, cw // s.shape[-1], axis=-1)[..., None]
    return dec.reshape(dec.shape[:-2] + (dec.shape[-2] * 8,))


def pair_packed(packed) -> np.ndarray:
    """The residual table with dims 2k and 2k+1 moved to nibbles k and k+4, the order the
    few-token 8-bit kernel takes (``src/ramp/kernels/e8_1bit_m1.py:25-33``)."""
    p = np.asarray(packed, dtype=np.uint32)
    out = np.zeros(256, dtype=np.uint32)
    for k in range(4):
        out |= ((p >> np.uint32(8 * k)) & np.uint32(0xF)) << np.uint32(4 * k)
        out |= ((p >> np.uint32(8 * k + 4)) & np.uint32(0xF)) << np.uint32(16 + 4 * k)
    return out


def half2_pairs(grid) -> np.ndarray:
    """[256, 8] codebook -> uint32 [256, 4]; word k carries the float16 bits of dim 2k (low
    half) and dim 2k+1 (high half) (``src/ramp/kernels/e8p_nested_m1.py:29-36``)."""
    g = np.asarray(grid)
    h = g.astype(np.float16)
    if h.shape != (256, 8) or not np.array_equal(h.astype(np.float64), g.astype(np.float64)):
        raise ValueError("codebook must be [256, 8] and exact in float16")
    bits = h.view(np.uint16).astype(np.uint32)
    return np.ascontiguousarray(bits[:, 0::2] | (bits[:, 1::2] << 16))


def cosine_similarity(a, b) -> float:
    """Cosine in float64; two all-zero inputs count as equal (``e8.py:574-580``)."""
    x = np.asarray(a, dtype=np.float64).reshape(-1)
    y = np.asarray(b, dtype=np.float64).reshape(-1)
    d = np.linalg.norm(x) * np.linalg.norm(y)
    if d == 0:
        return 1.0 if np.array_equal(x, y) else 0.0
    return float(x @ y / d)


def relative_gap(got, want) -> float:
    """max|got - want| / max|want|: the reference's agreement measure
    (``scripts/v41_build/omlx_lattice.py:594-595``, ``tests/test_e8_1bit_m1.py:26-30``)."""
    g = np.asarray(got, dtype=np.float64)
    w = np.asarray(want, dtype=np.float64)
    top = float(np.max(np.abs(w))) if w.size else 0.0
    if top == 0.0:
        return float(np.max(np.abs(g))) if g.size else 0.0
    return float(np.max(np.abs(g - w)) / top)
