"""The C-ABI library loads and exports every symbol the header declares (no GPU, no compute)."""

import ctypes
import re

from conftest import ROOT


def declared_entry_points():
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names += re.findall(r"^\s*(?:const\s+char\s*\*|int64_t|int)\s+(keepvq_\w+)\s*\(", text, flags=re.M)
    return names


def test_header_declares_entry_points():
    names = declared_entry_points()
    assert "keepvq_routed_matvec" in names and "keepvq_decode_weights" in names


def test_library_exports_every_declared_symbol():
    from keep_b200 import _lib

    lib = _lib.load()
    for name in declared_entry_points():
        assert hasattr(lib, name), f"libkeepvq.so lacks {name}"
    assert sorted(declared_entry_points()) == _lib.exported_names(), "ctypes table and header disagree"
    assert lib.keepvq_abi_version() == 3
    assert lib.keepvq_status_string(-2).decode() == "inconsistent sizes"


def test_struct_sizes_match_the_compiler():
    """ctypes mirrors of the argument structs have the layout gcc gives the header."""
    import subprocess
    import tempfile

    from keep_b200 import _lib

    structs = {"keepvq_decode_args": _lib.DecodeArgs, "keepvq_matvec_args": _lib.MatvecArgs}
    structs.update(getattr(_lib, "EXTRA_STRUCTS", {}))
    body = "".join(f'printf("{n} %zu\\n", sizeof({n}));' for n in structs)
    src = f'#include <stdio.h>\n#include "keepvq.h"\nint main(void){{{body}return 0;}}'
    with tempfile.TemporaryDirectory() as tmp:
        (c := __import__("pathlib").Path(tmp) / "s.c").write_text(src)
        exe = c.with_suffix("")
        subprocess.run(["gcc", "-I", str(ROOT / "include"), str(c), "-o", str(exe)], check=True)
        out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    for line in out.splitlines():
        name, size = line.split()
        assert ctypes.sizeof(structs[name]) == int(size), name


def test_operators_refuse_cpu_tensors():
    import pytest
    import torch

    from keep_b200 import _lib, kernels

    x = torch.zeros(64)
    with pytest.raises(_lib.KeepVQError):
        kernels.vq_qmv(x, torch.zeros(8, 8, dtype=torch.uint16), torch.ones(8, 1), None, in_dim=64, out_dim=8,
                       group_size=64, code_bits=16)


def test_custom_ops_register_without_a_gpu():
    """Importing ``keep_b200.torch_ops`` defines every operator under ``torch.ops.keepvq`` with a
    schema (no compute happens without a device)."""
    import torch

    from keep_b200 import torch_ops

    for name in torch_ops.OPS:
        schema = getattr(torch.ops.keepvq, name).default._schema
        assert schema.name == f"keepvq::{name}" and len(schema.returns) >= 1
