"""Readers for the layer files the routed path is served from.

The reference writes one ``layer-NN.npz`` per MoE layer: an uncompressed zip of
``{w1,w2,w3}_codes`` (uint16 ``[E, out, in/8]``, uint8 for 1-bit codes), ``{w1,w2,w3}_scales``
(fp16 ``[E, out, in/g]``) and ``code_bits`` (``scripts/runpod/v41_reap/keep_quant.py:16-19,131-133``),
and serves from it with positional reads of one expert's slab at a time
(``scripts/v41_build/omlx_lattice.py:115-150``).

``PoolFile`` reads the JSON that describes a pool wider than the loaded checkpoint
(``scripts/v41_build/omlx_lattice.py:22-30,461-480``): which directory and which position in its
layer files holds each expert of the pool, the pool's router rows, and the order in which the
residents start out.

``LayerFile`` finds each array inside the zip once and then hands out experts as views of a memory
map (no decompression, no whole-file read): the bytes an installer copies into a slot are the
file's own bytes.  ``store`` materialises the whole layer in (pinned) host memory for
``residency.SlotInstaller``; ``projection`` builds the device tensors of the resident slots.
"""

from __future__ import annotations

import io
import struct
import zipfile
from pathlib import Path

import numpy as np
import torch

TENSOR_NAMES = tuple(f"{p}_{f}" for p in ("w1", "w3", "w2") for f in ("codes", "scales"))


class LayerFile:
    """One ``layer-NN.npz``.  ``members[name] = (byte offset of the array data, shape, dtype)``."""

    def __init__(self, path):
        self.path = Path(path)
        self.members: dict[str, tuple[int, tuple, np.dtype]] = {}
        with zipfile.ZipFile(self.path) as archive, open(self.path, "rb") as raw:
            for info in archive.infolist():
                if info.compress_type != zipfile.ZIP_STORED:
                    raise ValueError(f"{self.path}: member {info.filename} is compressed; the serving path needs stored arrays (np.savez)")
                # local file header: 30 fixed bytes, then the name and the extra field
                raw.seek(info.header_offset)
                fixed = raw.read(30)
                if fixed[:4] != b"PK\x03\x04":
                    raise ValueError(f"{self.path}: bad local header for {info.filename}")
                name_len, extra_len = struct.unpack("<HH", fixed[26:30])
                data_start = info.header_offset + 30 + name_len + extra_len
                raw.seek(data_start)
                head = io.BytesIO(raw.read(min(info.file_size, 4096)))
                version = np.lib.format.read_magic(head)
                reader = np.lib.format.read_array_header_1_0 if version[0] == 1 else np.lib.format.read_array_header_2_0
                shape, fortran, dtype = reader(head)
                if fortran:
                    raise ValueError(f"{self.path}: {info.filename} is stored in Fortran order")
                self.members[info.filename.removesuffix(".npy")] = (data_start + head.tell(), tuple(shape), np.dtype(dtype))
        missing = [n for n in TENSOR_NAMES if n not in self.members]
        if missing:
            raise ValueError(f"{self.path}: missing arrays {missing}")
        self.code_bits = int(self.array("code_bits")) if "code_bits" in self.members else (16 if self.members["w1_codes"][2] == np.uint16 else 8)
        self.experts = int(self.members["w1_codes"][1][0])

    def array(self, name: str) -> np.ndarray:
        """The whole array as a read-only memory map of the file."""
        offset, shape, dtype = self.members[name]
        if not shape:
            return np.fromfile(self.path, dtype=dtype, count=1, offset=offset)[0]
        return np.memmap(self.path, dtype=dtype, mode="r", offset=offset, shape=shape)

    def slab(self, name: str, expert: int) -> tuple[int, int]:
        """(byte offset in the file, byte count) of one expert's rows of ``name``."""
        offset, shape, dtype = self.members[name]
        if not 0 <= expert < shape[0]:
            raise IndexError(f"expert {expert} outside 0..{shape[0] - 1}")
        size = int(np.prod(shape[1:], dtype=np.int64)) * dtype.itemsize
        return offset + expert * size, size

    def read(self, name: str, experts) -> np.ndarray:
        """``[len(experts), ...]``: the named array's rows of those experts, copied out of the map."""
        view = self.array(name)
        return np.stack([np.asarray(view[int(e)]) for e in experts]) if len(experts) else np.empty((0,) + view.shape[1:], view.dtype)


def _torch_dtype(dtype: np.dtype) -> torch.dtype:
    return {np.dtype(np.uint16): torch.uint16, np.dtype(np.uint8): torch.uint8, np.dtype(np.float16): torch.float16,
            np.dtype(np.float32): torch.float32}[np.dtype(dtype)]


def store(layer: LayerFile, *, pin: bool = True) -> dict[str, torch.Tensor]:
    """Every expert of the layer in host memory, by tensor name: what ``SlotInstaller`` copies
    from.  ``pin=True`` (needs a CUDA runtime) makes the copies asynchronous."""
    out = {}
    for name in TENSOR_NAMES:
        view = layer.array(name)
        host = torch.empty(tuple(view.shape), dtype=_torch_dtype(view.dtype), pin_memory=pin)
        host.numpy()[...] = view
        out[name] = host
    return out


def projection(layer: LayerFile, which: str, experts, device):
    """``moe.Projection`` holding the given experts' rows of ``w1`` / ``w3`` / ``w2`` in slot order."""
    from .moe import Projection

    codes = torch.from_numpy(layer.read(f"{which}_codes", experts)).to(device)
    scales = torch.from_numpy(layer.read(f"{which}_scales", experts)).to(device)
    return Projection(codes, scales)


# ---- safetensors checkpoints ---------------------------------------------------------------
# KEEP's converted checkpoints store a switch projection as ``<prefix>.codes`` (uint8 / uint16
# [experts, out, in/8]) and ``<prefix>.scales`` ([experts, out, in/group]), optionally ``.bias``,
# an optional shared ``model.vq_codebook.e8`` table, and a ``quantization_config`` JSON in the
# file metadata that names the codebook by its SHA-256 (src/keep/io/schema.py:64-106,
# src/keep/io/load.py:109-122,154-181,236-262).


def switch_linear_dims(shapes: dict, dtypes: dict, prefix: str) -> tuple[int, int, int, int, int]:
    """(in_dim, out_dim, experts, group_size, code_bits) from the tensors' shapes and dtypes, with
    the reference's checks (``infer_vq_switch_linear_dims``, load.py:154-181)."""
    codes_name, scales_name = f"{prefix}.codes", f"{prefix}.scales"
    for name in (codes_name, scales_name):
        if name not in shapes:
            raise KeyError(f"missing tensor {name!r}")
    codes, scales = tuple(shapes[codes_name]), tuple(shapes[scales_name])
    if len(codes) != 3:
        raise ValueError(f"{codes_name} must be 3D [experts, out, in/8], found {codes}")
    if len(scales) != 3:
        raise ValueError(f"{scales_name} must be 3D [experts, out, in/group], found {scales}")
    if codes[:2] != scales[:2]:
        raise ValueError("switch codes and scales must have the same expert and out dimensions")
    code_bits = {"U8": 8, "UINT8": 8, "U16": 16, "UINT16": 16}.get(str(dtypes[codes_name]).upper())
    if code_bits is None:
        raise ValueError(f"{codes_name} must be uint8 or uint16, found {dtypes[codes_name]}")
    experts, out_dim, codewords = codes
    in_dim = codewords * 8
    if scales[2] <= 0 or in_dim % scales[2] != 0:
        raise ValueError("switch scale count must divide inferred in_dim")
    return in_dim, out_dim, experts, in_dim // scales[2], code_bits


def load_quantized_vq_switch_linear(path, prefix: str, device):
    """``<prefix>.codes`` / ``.scales`` (/ ``.bias``) of a KEEP safetensors file as a
    ``switch.QuantizedVQSwitchLinear`` on ``device``.  A codebook hash in the file's metadata must
    be one of the two tables this library carries, as in the reference."""
    import json

    from safetensors import safe_open

    from .switch import QuantizedVQSwitchLinear
    from .vq import E8_1BIT_PACKED_SHA256, E8P_PACKED_ABS_SHA256

    with safe_open(str(path), framework="pt", device="cpu") as f:
        meta = f.metadata() or {}
        config = json.loads(meta["quantization_config"]) if "quantization_config" in meta else {}
        expected = (config.get("codebook") or {}).get("sha256") if isinstance(config, dict) else None
        if expected is not None and expected not in (E8_1BIT_PACKED_SHA256, E8P_PACKED_ABS_SHA256):
            raise ValueError(f"checkpoint E8 codebook hash {expected!r} is not supported by this runtime")
        names = set(f.keys())
        # tensors the reference's loader would hand to the layer and its forward would apply
        # (src/keep/io/load.py:245-257, src/ramp/nn/linear.py:77-82): loading without them would
        # give wrong outputs silently, so a checkpoint that carries one is refused by name
        from .switch import _OUTSIDE

        for sidecar in _OUTSIDE:
            if f"{prefix}.{sidecar}" in names:
                raise NotImplementedError(f"{prefix}.{sidecar} is present: {sidecar} belongs to the conversion tooling and is not applied by the routed hot path")
        wanted = [n for n in (f"{prefix}.codes", f"{prefix}.scales") if n in names]
        shapes = {n: tuple(f.get_slice(n).get_shape()) for n in wanted}
        dtypes = {n: f.get_slice(n).get_dtype() for n in wanted}
        in_dim, out_dim, experts, group_size, code_bits = switch_linear_dims(shapes, dtypes, prefix)
        get = lambda n: f.get_tensor(n).to(device) if n in names else None  # noqa: E731
        codes, scales, bias = get(f"{prefix}.codes"), get(f"{prefix}.scales"), get(f"{prefix}.bias")
        codebook = get("model.vq_codebook.e8")
    return QuantizedVQSwitchLinear(input_dims=in_dim, output_dims=out_dim, num_experts=experts, codes=codes, scales=scales,
                                   codebook=codebook, bias=bias, group_size=group_size, code_bits=code_bits)


class PoolFile:
    """A pool wider than the loaded checkpoint, as the reference's ``wide_pool`` reads it
    (``scripts/v41_build/omlx_lattice.py:22-30,461-480``).  The file is JSON::

        {"codes": [[CODES_DIR, IDS.json], ...], "router": "router.safetensors", "mass": "reap-stats.npz",
         "residual": DIR, "hot": H}            # the last two are optional (the 8-bit residual tier)

    ``IDS.json`` (``{"survivors": {layer: [...]}}``) gives the pool number of each expert of its
    directory in file order; ``router`` holds ``layers.N.ffn.gate.weight`` / ``.bias`` for every
    expert of the pool; ``mass`` (``reap__gate_norm_sum`` ``[layers, pool]``) orders the starting
    residents.  Paths inside the file are relative to it.

    Attributes: ``directories`` (paths), ``where[layer][expert] = (directory index, position in
    that directory's layer file)``, ``order[layer]`` (experts by descending mass, ties to the lower
    number), ``residual`` (path or None) and ``hot`` (0 without a residual directory;
    ``OMLX_LATTICE_HOT`` overrides the file, as in the reference).
    """

    def __init__(self, path):
        import json
        import os

        self.path = Path(path)
        spec = json.loads(self.path.read_text())
        at = lambda p: self.path.parent / Path(p).expanduser()  # noqa: E731
        self.directories = [at(d) for d, _ in spec["codes"]]
        ids = [json.loads(at(f).read_text())["survivors"] for _, f in spec["codes"]]
        layers = len(ids[0])
        self.where = [{int(e): (d, j) for d, per in enumerate(ids) for j, e in enumerate(per[str(i)])} for i in range(layers)]
        self.first_directory = [[int(e) for e in ids[0][str(i)]] for i in range(layers)]  # the loaded checkpoint's experts, file order
        mass = np.load(at(spec["mass"]))["reap__gate_norm_sum"]
        self.pool = int(mass.shape[1])
        if mass.shape[0] < layers or any(sorted(w) != list(range(self.pool)) for w in self.where):
            raise ValueError(f"{self.path}: the directories do not cover the pool once")
        self.order = [np.argsort(-mass[i], kind="stable").tolist() for i in range(layers)]
        self._router_path = at(spec["router"])
        self.residual = at(spec["residual"]) if "residual" in spec else None
        self.hot = int(os.environ.get("OMLX_LATTICE_HOT", spec.get("hot", 0))) if self.residual is not None else 0
        if self.hot == 0:
            self.residual = None

    def router(self, layer: int, device="cpu") -> tuple[torch.Tensor, torch.Tensor | None]:
        """(weight ``[pool, hidden]``, bias ``[pool]`` or None) of the pool's router for one layer."""
        from safetensors import safe_open

        with safe_open(str(self._router_path), framework="pt", device="cpu") as f:
            names = set(f.keys())
            weight = f.get_tensor(f"layers.{layer}.ffn.gate.weight").to(device)
            bias = f.get_tensor(f"layers.{layer}.ffn.gate.bias").to(device) if f"layers.{layer}.ffn.gate.bias" in names else None
        if int(weight.shape[0]) != self.pool:
            raise ValueError(f"{self._router_path}: layer {layer} has {int(weight.shape[0])} router rows for a pool of {self.pool}")
        return weight, bias

    def check_loaded_router(self, layer: int, weight: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        """The loaded checkpoint's router rows must be the first directory's rows of the pool router."""
        full_w, full_b = self.router(layer)
        rows = torch.tensor(self.first_directory[layer], dtype=torch.long)
        if not torch.equal(full_w[rows], weight.cpu()):
            raise ValueError(f"layer {layer}: router weight differs from the pool file's")
        if bias is not None and full_b is not None and not torch.equal(full_b[rows], bias.cpu()):
            raise ValueError(f"layer {layer}: router bias differs from the pool file's")

    def layer_file(self, layer: int, expert: int) -> tuple[Path, int]:
        """(path of the ``layer-NN.npz`` that holds the expert, its position in that file)."""
        directory, position = self.where[layer][int(expert)]
        return self.directories[directory] / f"layer-{layer:02d}.npz", position

    def starting_residents(self, layer: int, slots: int) -> list[int]:
        """The ``slots`` experts a layer starts out with: the heaviest by ``mass``."""
        return self.order[layer][:slots]
