"""The arithmetic the CUDA decode kernels rest on, checked on the CPU over all 65,536 codewords.

The kernels never decode a codeword to floats.  They read two table words of eight 4-bit values
each (keep_b200/csrc/moe_fast.cuh: ``abs_table_entry`` / ``sign_table_entry`` packed by
``pack_nibbles``): ``E[abs byte] ^ 0x88888888`` and ``M[sign byte]``, XOR them, and hand the
nibbles ``u`` to the tensor cores as unsigned bytes.  The claim: ``4 w = 2 (u - 8) + 1`` for every
weight ``w`` the reference decodes (``oracle.e8.decode_e8p``, pinned to src/keep/vq/e8.py:210-234
by the golden vectors), with table nibble ``n`` of the word standing for output dimension ``d``
where ``n = SHUFFLE[d]``.  The table rules are restated here in numpy, line for line with the
device functions, so a change to either side shows up without a GPU.
"""

import numpy as np

from oracle import e8


def abs_entry_bytes(word: int, parity: int) -> np.ndarray:
    """q of the eight table nibbles of an abs row (``abs_table_entry``): nibble - 8, then on odd
    parity ^1 (nibble 0: ~)."""
    q = np.array([((word >> (4 * n)) & 0xF) - 8 for n in range(8)], dtype=np.int64)
    if parity:
        q = np.array([~q[0]] + [v ^ 1 for v in q[1:]], dtype=np.int64)
    return q & 0xFF


def sign_entry_bytes(sign_byte: int) -> np.ndarray:
    """XOR masks of a sign byte (``sign_table_entry``): 0xFE where the bit is set; on odd parity
    ^1 everywhere (^0xFF on nibble 0)."""
    parity = bin(sign_byte).count("1") & 1
    m = np.array([0xFE if (sign_byte >> n) & 1 else 0 for n in range(8)], dtype=np.int64)
    if parity:
        m ^= np.array([0xFF] + [0x01] * 7, dtype=np.int64)
    return m


def test_nibble_tables_reproduce_every_codeword():
    table = e8.e8p_packed_abs_grid().astype(np.int64)
    abs_nibbles = np.stack([(abs_entry_bytes(int(w), 0) & 0xF) ^ 0x8 for w in table])     # [256, 8] u = q + 8, even parity
    sign_nibbles = np.stack([sign_entry_bytes(s) & 0xF for s in range(256)])              # [256, 8]
    codes = np.arange(1 << 16, dtype=np.int64)
    u = abs_nibbles[codes >> 8] ^ sign_nibbles[codes & 0xFF]                              # [65536, 8] by table nibble
    assert u.min() >= 0 and u.max() <= 15
    quarter = np.round(e8.e8p_full_grid() * 4).astype(np.int64)                           # [65536, 8] by output dimension
    for d, n in enumerate(e8.E8P_SHUFFLE):
        np.testing.assert_array_equal(2 * (u[:, n] - 8) + 1, quarter[:, d])


def test_byte_and_nibble_forms_of_the_tables_agree():
    """The byte form (q as a signed byte, masks 0x00 / 0xFE / 0x01 / 0xFF) and its low nibbles give
    the same q: every q lies in [-8, 7], so four bits of two's complement hold it."""
    table = e8.e8p_packed_abs_grid().astype(np.int64)
    for w in table[:: 17]:
        for s in (0, 1, 0x80, 0x55, 0xFF, 0x7E):
            parity = bin(s).count("1") & 1
            q_bytes = (abs_entry_bytes(int(w), 0) ^ sign_entry_bytes(s)) & 0xFF
            q = np.where(q_bytes >= 128, q_bytes - 256, q_bytes)
            assert q.min() >= -8 and q.max() <= 7
            u = ((abs_entry_bytes(int(w), 0) & 0xF) ^ 0x8) ^ (sign_entry_bytes(s) & 0xF)
            np.testing.assert_array_equal(u - 8, q)
            # and the parity rule of the abs entry itself: the odd-parity entry is the even one with the parity masks applied
            if parity:
                flips = np.array([0xFF] + [0x01] * 7, dtype=np.int64)
                np.testing.assert_array_equal(abs_entry_bytes(int(w), 1), (abs_entry_bytes(int(w), 0) ^ flips) & 0xFF)


def test_the_offset_comes_off_in_wrapping_arithmetic():
    """sum(u x') - 8 sum(x') = sum(q x') even when 256 * high + low overflows 32 bits on the way."""
    rng = np.random.default_rng(3)
    u = rng.integers(10, 14, size=8192)
    x = rng.integers(20000, 32640, size=8192)                       # one-sided rows: the worst case for the intermediate
    hi = (x + 128) >> 8
    lo = x - 256 * hi
    d_hi, d_lo = int((u * hi).sum()), int((u * lo).sum())           # what the two accumulators hold
    wrapped = (d_hi * 256 + d_lo - 8 * int(x.sum())) & 0xFFFFFFFF
    want = int(((u - 8) * x).sum())
    assert abs(want) < 2 ** 31 and d_hi * 256 >= 2 ** 31             # the true value fits, the intermediate does not
    assert (wrapped - (1 << 32) if wrapped >= 1 << 31 else wrapped) == want
