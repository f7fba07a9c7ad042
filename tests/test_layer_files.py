"""Layer files (layer-NN.npz): members found inside the stored zip, slabs at the right bytes,
compressed files refused.  CPU only."""

import os

import numpy as np
import pytest
import torch

from keep_b200 import io as layer_io


def write_layer(path, experts=5, out=6, inp=64, code_bits=16, compressed=False):
    rng = np.random.default_rng(3)
    arrays = {"code_bits": np.asarray(code_bits)}
    for p, (o, i) in (("w1", (out, inp)), ("w3", (out, inp)), ("w2", (inp, out * 8))):
        arrays[f"{p}_codes"] = rng.integers(0, 1 << code_bits, (experts, o, i // 8)).astype(np.uint16 if code_bits == 16 else np.uint8)
        arrays[f"{p}_scales"] = rng.uniform(0.01, 0.05, (experts, o, 1)).astype(np.float16)
    (np.savez_compressed if compressed else np.savez)(path, **arrays)
    return arrays


@pytest.mark.parametrize("code_bits", [16, 8])
def test_members_slabs_and_reads(tmp_path, code_bits):
    path = tmp_path / "layer-03.npz"
    arrays = write_layer(path, code_bits=code_bits)
    layer = layer_io.LayerFile(path)
    assert layer.code_bits == code_bits and layer.experts == 5
    fd = os.open(path, os.O_RDONLY)
    try:
        for name in layer_io.TENSOR_NAMES:
            np.testing.assert_array_equal(np.asarray(layer.array(name)), arrays[name])
            for expert in (0, 3, 4):  # a positional read of the slab gives exactly that expert's bytes
                offset, size = layer.slab(name, expert)
                assert os.pread(fd, size, offset) == arrays[name][expert].tobytes()
            np.testing.assert_array_equal(layer.read(name, [4, 1]), arrays[name][[4, 1]])
    finally:
        os.close(fd)
    with pytest.raises(IndexError):
        layer.slab("w1_codes", 5)
    host = layer_io.store(layer, pin=False)
    assert set(host) == set(layer_io.TENSOR_NAMES) and host["w2_codes"].dtype == (torch.uint16 if code_bits == 16 else torch.uint8)
    np.testing.assert_array_equal(host["w3_scales"].numpy(), arrays["w3_scales"])


def test_compressed_and_incomplete_files_are_refused(tmp_path):
    write_layer(tmp_path / "c.npz", compressed=True)
    with pytest.raises(ValueError, match="compressed"):
        layer_io.LayerFile(tmp_path / "c.npz")
    np.savez(tmp_path / "m.npz", w1_codes=np.zeros((2, 2, 2), np.uint16))
    with pytest.raises(ValueError, match="missing arrays"):
        layer_io.LayerFile(tmp_path / "m.npz")


def test_safetensors_switch_dims_and_checks():
    shapes = {"m.w.codes": (4, 6, 8), "m.w.scales": (4, 6, 2)}
    assert layer_io.switch_linear_dims(shapes, {"m.w.codes": "U16", "m.w.scales": "F16"}, "m.w") == (64, 6, 4, 32, 16)
    assert layer_io.switch_linear_dims(shapes, {"m.w.codes": "U8", "m.w.scales": "F16"}, "m.w")[4] == 8
    with pytest.raises(KeyError, match="missing tensor"):
        layer_io.switch_linear_dims(shapes, {}, "m.v")
    with pytest.raises(ValueError, match="uint8 or uint16"):
        layer_io.switch_linear_dims(shapes, {"m.w.codes": "I32", "m.w.scales": "F16"}, "m.w")
    with pytest.raises(ValueError, match="same expert and out"):
        layer_io.switch_linear_dims({"m.w.codes": (4, 6, 8), "m.w.scales": (4, 5, 2)}, {"m.w.codes": "U16"}, "m.w")
    with pytest.raises(ValueError, match="must divide"):
        layer_io.switch_linear_dims({"m.w.codes": (4, 6, 8), "m.w.scales": (4, 6, 3)}, {"m.w.codes": "U16"}, "m.w")


@pytest.mark.parametrize("sidecar", ["rht_signs", "rotation_matrix", "continuous_low_rank_left"])
def test_a_checkpoint_with_a_rotation_or_residual_sidecar_is_refused(tmp_path, sidecar):
    """The reference's loader hands ``<prefix>.rht_signs`` / ``.rotation_matrix`` (and the other
    conversion-side tensors) to the layer, whose forward applies them (src/keep/io/load.py:245-257,
    src/ramp/nn/linear.py:77-82).  This runtime does not apply them, so it must not load such a
    file as if they were absent: the refusal comes before any tensor reaches a device."""
    import torch
    from safetensors.torch import save_file

    tensors = {"m.w.codes": torch.zeros((2, 8, 4), dtype=torch.uint8), "m.w.scales": torch.ones((2, 8, 1), dtype=torch.float16),
               f"m.w.{sidecar}": torch.ones(32, dtype=torch.float16)}
    path = tmp_path / "layer.safetensors"
    save_file(tensors, str(path))
    with pytest.raises(NotImplementedError, match=sidecar):
        layer_io.load_quantized_vq_switch_linear(path, "m.w", "cpu")


def test_pool_file_maps_every_expert_and_orders_the_residents(tmp_path, monkeypatch):
    """The JSON of a pool wider than the loaded checkpoint (scripts/v41_build/omlx_lattice.py:22-30,461-480):
    two directories of experts, the pool's router, the mass that orders the starting residents."""
    import json

    from safetensors.torch import save_file

    layers, pool, hidden = 2, 6, 16
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    first = {"0": [4, 1, 5], "1": [0, 2, 3]}    # the loaded checkpoint's experts, in file order
    second = {"0": [0, 2, 3], "1": [5, 4, 1]}
    (tmp_path / "a" / "ids.json").write_text(json.dumps({"survivors": first}))
    (tmp_path / "b" / "ids.json").write_text(json.dumps({"survivors": second}))
    gen = torch.Generator().manual_seed(0)
    router = {f"layers.{i}.ffn.gate.weight": torch.randn((pool, hidden), generator=gen) for i in range(layers)}
    router.update({f"layers.{i}.ffn.gate.bias": torch.randn((pool,), generator=gen) for i in range(layers)})
    save_file(router, str(tmp_path / "router.safetensors"))
    mass = np.array([[1.0, 5.0, 2.0, 5.0, 0.5, 3.0], [6.0, 1.0, 2.0, 3.0, 4.0, 5.0]])
    np.savez(tmp_path / "stats.npz", reap__gate_norm_sum=mass)
    spec = {"codes": [["a", "a/ids.json"], ["b", "b/ids.json"]], "router": "router.safetensors", "mass": "stats.npz", "residual": "res", "hot": 2}
    (tmp_path / "pool.json").write_text(json.dumps(spec))
    monkeypatch.delenv("OMLX_LATTICE_HOT", raising=False)
    pool_file = layer_io.PoolFile(tmp_path / "pool.json")
    assert pool_file.pool == pool and pool_file.hot == 2 and pool_file.residual == tmp_path / "res"
    assert pool_file.where[0][5] == (0, 2) and pool_file.where[0][3] == (1, 2) and pool_file.where[1][4] == (1, 1)
    assert pool_file.layer_file(1, 4) == (tmp_path / "b" / "layer-01.npz", 1)
    assert pool_file.order[0] == [1, 3, 5, 2, 0, 4]            # descending mass, ties to the lower number
    assert pool_file.starting_residents(1, 3) == [0, 5, 4]
    weight, bias = pool_file.router(0)
    assert torch.equal(weight, router["layers.0.ffn.gate.weight"]) and torch.equal(bias, router["layers.0.ffn.gate.bias"])
    pool_file.check_loaded_router(0, weight[[4, 1, 5]], bias[[4, 1, 5]])
    with pytest.raises(ValueError, match="differs"):
        pool_file.check_loaded_router(0, weight[[4, 1, 0]])
    monkeypatch.setenv("OMLX_LATTICE_HOT", "1")
    assert layer_io.PoolFile(tmp_path / "pool.json").hot == 1
    # a pool the directories do not cover exactly once is refused
    (tmp_path / "b" / "ids.json").write_text(json.dumps({"survivors": {"0": [0, 2, 2], "1": [5, 4, 1]}}))
    with pytest.raises(ValueError, match="cover the pool once"):
        layer_io.PoolFile(tmp_path / "pool.json")


def test_pool_file_positions_lead_to_the_experts_own_bytes(tmp_path):
    """A pool of six experts in two directories of three: ``PoolFile.layer_file`` names the file
    and the position, and the ``LayerFile`` slab read there is that expert's codes."""
    import json

    from safetensors.torch import save_file

    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    ids = [{"0": [4, 1, 5]}, {"0": [0, 2, 3]}]
    written = []
    for name, per in zip("ab", ids):
        (tmp_path / name / "ids.json").write_text(json.dumps({"survivors": per}))
        rng_seed = 11 if name == "a" else 12
        arrays = write_layer(tmp_path / name / "layer-00.npz", experts=3)
        # make the two directories' contents differ
        arrays["w1_codes"] = (arrays["w1_codes"].astype(np.int64) + rng_seed).astype(np.uint16)
        np.savez(tmp_path / name / "layer-00.npz", **arrays)
        written.append(arrays)
    save_file({"layers.0.ffn.gate.weight": torch.zeros((6, 8))}, str(tmp_path / "router.safetensors"))
    np.savez(tmp_path / "stats.npz", reap__gate_norm_sum=np.arange(6, dtype=np.float64)[None])
    (tmp_path / "pool.json").write_text(json.dumps({"codes": [["a", "a/ids.json"], ["b", "b/ids.json"]], "router": "router.safetensors", "mass": "stats.npz"}))
    pool = layer_io.PoolFile(tmp_path / "pool.json")
    assert pool.residual is None and pool.hot == 0 and pool.starting_residents(0, 2) == [5, 4]
    for expert in range(6):
        directory, position = pool.where[0][expert]
        path, at = pool.layer_file(0, expert)
        assert at == position and path.parent.name == "ab"[directory]
        np.testing.assert_array_equal(layer_io.LayerFile(path).read("w1_codes", [at])[0], written[directory]["w1_codes"][position])
        assert ids[directory]["0"][position] == expert
