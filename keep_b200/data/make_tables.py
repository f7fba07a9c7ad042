"""Writes the two 1 KiB codebook files shipped with the package.

    python keep_b200/data/make_tables.py /path/to/keep/checkout

Imports ``keep.vq.e8`` from a checkout of the reference project (its ``src`` directory) and
dumps ``e8p_packed_abs_grid()`` and ``e8_1bit_packed()`` as little-endian uint32[256].  The
package verifies both files against the SHA-256 digests the reference pins
(``tests/test_e8_reference.py:25-26``) each time it loads them.
"""

import sys
from pathlib import Path

import numpy as np


def main() -> None:
    checkout = Path(sys.argv[1])
    sys.path.insert(0, str(checkout / "src"))
    from keep.vq import e8

    here = Path(__file__).resolve().parent
    for name, table in (("e8p_packed_abs.u32", e8.e8p_packed_abs_grid()), ("e8_1bit_packed.u32", e8.e8_1bit_packed())):
        data = np.asarray(table, dtype="<u4")
        assert data.shape == (256,)
        (here / name).write_bytes(data.tobytes())
        print(name, e8._sha256_u32(data))


if __name__ == "__main__":
    main()
