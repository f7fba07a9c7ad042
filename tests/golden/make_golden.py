"""Generates the golden fixtures in this directory by running the REFERENCE's own Python.

    python tests/golden/make_golden.py /path/to/keep/checkout

Run where a checkout of jackmaxwil/keep is available; the fixtures it writes are committed, and
the tests read only those.  Nothing here is imported by the package or by the tests.

The reference's routed operators import ``mlx.core`` at module top.  ``mlx`` does not exist
off Apple hardware, so this script installs a small numpy-backed stand-in for the handful of
``mlx.core`` names those modules touch at import time and on their ``implementation="reference"``
path (which is numpy underneath).  The Metal paths are never entered.
"""

from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def install_mlx_stand_in() -> None:
    import ml_dtypes

    core = types.ModuleType("mlx.core")

    class array(np.ndarray):  # noqa: N801 - mirrors mlx's name
        def __new__(cls, value, dtype=None):
            return np.asarray(value, dtype=dtype).view(cls)

        def astype(self, dtype, *a, **k):
            return np.asarray(self).astype(dtype, *a, **k).view(array)

    class Dtype:  # only used in annotations
        pass

    core.array, core.Dtype = array, Dtype
    core.float32, core.float16, core.bfloat16 = np.float32, np.float16, ml_dtypes.bfloat16
    core.int32, core.int64, core.uint8, core.uint16, core.uint32, core.bool_ = (
        np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.bool_)
    core.stack = lambda xs, axis=0: np.stack([np.asarray(x) for x in xs], axis=axis).view(array)
    core.arange = lambda *a, dtype=None: np.arange(*a, dtype=dtype).view(array)
    core.zeros = lambda shape, dtype=np.float32: np.zeros(shape, dtype).view(array)
    core.ones = lambda shape, dtype=np.float32: np.ones(shape, dtype).view(array)
    core.argsort = lambda x, axis=-1: np.argsort(np.asarray(x), axis=axis, kind="stable").view(array)
    core.contiguous = lambda x: x
    core.eval = lambda *a, **k: None
    core.device_info = lambda: {"architecture": "none"}

    def metal_kernel(**kw):
        def refuse(*a, **k):
            raise RuntimeError("Metal kernels cannot run here")
        return refuse

    core.fast = types.SimpleNamespace(metal_kernel=metal_kernel)
    core.metal = types.SimpleNamespace(is_available=lambda: False, device_info=lambda: {"architecture": "none"})
    pkg = types.ModuleType("mlx")
    pkg.core = core
    sys.modules["mlx"], sys.modules["mlx.core"] = pkg, core


def load_by_path(name: str, path: Path):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def codebook_fixture(e8) -> None:
    """Tables, the reference's own golden codewords (tests/test_e8_reference.py:37-83) and a
    seeded decode_weight_matrix case for both code widths."""
    rng = np.random.default_rng(20260623)
    e8p_codes = np.array([0, 1, 255, 256, 0x1234, 0xFFFF], dtype=np.uint16)
    res_codes = np.array([0, 1, 112, 113, 240, 241, 255], dtype=np.uint8)
    codes16 = rng.integers(0, 1 << 16, size=(6, 32), dtype=np.uint16)
    scales16 = (0.02 * rng.uniform(0.5, 1.5, size=(6, 4))).astype(np.float16)
    codes8 = rng.integers(0, 256, size=(4, 16), dtype=np.uint8)
    scales8 = rng.normal(loc=1.0, scale=0.05, size=(4, 2)).astype(np.float32)
    full = e8.e8p_full_grid()
    np.savez_compressed(
        HERE / "codebooks.npz",
        e8p_packed_abs=e8.e8p_packed_abs_grid(), e8_1bit_packed=e8.e8_1bit_packed(),
        e8p_codes=e8p_codes, e8p_decoded=e8.decode_e8p(e8p_codes),
        res_codes=res_codes, res_decoded=e8.decode_e8_1bit(res_codes),
        full_grid_quarter_units=np.round(full * 4).astype(np.int8),
        codes16=codes16, scales16=scales16,
        weights16=e8.decode_weight_matrix(codes16, scales16.astype(np.float32), code_bits=16),
        codes8=codes8, scales8=scales8, weights8=e8.decode_weight_matrix(codes8, scales8, code_bits=8),
    )


def operator_fixture(checkout: Path) -> None:
    """Outputs of the reference's ``vq_qmv`` / ``gather_vqmm`` with ``implementation="reference"``
    and of its table-layout helpers, on seeded inputs."""
    install_mlx_stand_in()
    import mlx.core as mx
    from ramp.kernels.e8_1bit_m1 import pair_packed
    from ramp.kernels.e8p_nested_m1 import half2_pairs
    from ramp.kernels.vq_qmv import vq_qmv_reference_np
    from ramp.ops.vq_switch import gather_vqmm, vq_switch_qmv
    from keep.vq import e8

    rng = np.random.default_rng(7)
    experts, out, inp, group = 5, 24, 128, 32
    codes = rng.integers(0, 1 << 16, size=(experts, out, inp // 8), dtype=np.uint16)
    scales = (0.02 * rng.uniform(0.5, 1.5, size=(experts, out, inp // group))).astype(np.float16)
    x = rng.normal(size=(4, inp)).astype(np.float32)
    rhs = np.stack([rng.choice(experts, 3, replace=False) for _ in range(4)]).astype(np.uint32)
    kw = dict(input_dims=inp, output_dims=out, group_size=group, code_bits=16, implementation="reference")
    token = np.asarray(gather_vqmm(mx.array(x), mx.array(codes), mx.array(scales), None, mx.array(rhs), **kw))
    lhs = np.array([3, 0, 2, 2, 1, 0, 3], dtype=np.int32)
    flat = np.array([4, 4, 0, 1, 3, 2, 0], dtype=np.uint32)
    routed = np.asarray(gather_vqmm(mx.array(x), mx.array(codes), mx.array(scales), None, mx.array(flat),
                                    lhs_indices=mx.array(lhs), **kw))
    xr = rng.normal(size=(4, 3, inp)).astype(np.float32)
    per_route = np.asarray(vq_switch_qmv(mx.array(xr), mx.array(codes), mx.array(scales), None, mx.array(rhs),
                                         input_dims=inp, output_dims=out, group_size=group, code_bits=16,
                                         implementation="reference"))
    qmv = vq_qmv_reference_np(x[0], codes[2], scales[2], None, in_dim=inp, out_dim=out, group_size=group, code_bits=16)
    codes8 = rng.integers(0, 256, size=(experts, out, inp // 8), dtype=np.uint8)
    token8 = np.asarray(gather_vqmm(mx.array(x), mx.array(codes8), mx.array(scales), None, mx.array(rhs),
                                    **{**kw, "code_bits": 8}))
    np.savez_compressed(
        HERE / "operators.npz",
        codes=codes, scales=scales, x=x, rhs=rhs, token=token, lhs=lhs, flat_rhs=flat, routed=routed,
        xr=xr, per_route=per_route, qmv=qmv, codes8=codes8, token8=token8,
        pair_packed=pair_packed(e8.e8_1bit_packed()), half2_pairs=half2_pairs(e8.e8_1bit_grid()),
    )


def router_fixture(checkout: Path) -> None:
    """Outputs of the reference's ``gate_masked`` (scripts/runpod/v41_reap/local_eval.py:69-90) on
    seeded inputs, for the three score functions, with and without a residency mask and with
    fewer allowed experts than top-k."""
    import types

    import torch

    sys.path.insert(0, str(checkout / "scripts" / "runpod" / "v41_reap"))
    local_eval = load_by_path("keep_reference_local_eval", checkout / "scripts" / "runpod" / "v41_reap" / "local_eval.py")
    rng = np.random.default_rng(41)
    pool, dim, tokens, k = 24, 64, 9, 4
    weight = rng.normal(scale=0.3, size=(pool, dim)).astype(np.float32)
    x = rng.normal(size=(tokens, dim)).astype(np.float32)
    bias = (0.01 * rng.normal(size=pool)).astype(np.float32)
    allowed = rng.random((tokens, pool)) < 0.5
    few = np.zeros((tokens, pool), dtype=bool)
    few[:, [3, 17]] = True
    out = dict(weight=weight, x=x, bias=bias, allowed=allowed, few=few, top_k=np.int64(k))
    for func in ("softmax", "sigmoid", "sqrtsoftplus"):
        gate = types.SimpleNamespace(weight=torch.from_numpy(weight), bias=torch.from_numpy(bias), gate_temp=1.25,
                                     score_func=func, topk=k, norm_topk_prob=True, route_scale=1.5)
        for name, mask in (("all", np.ones((tokens, pool), dtype=bool)), ("masked", allowed), ("few", few)):
            w, i = local_eval.gate_masked(gate, torch.from_numpy(x), torch.from_numpy(mask), torch.nn.functional.linear)
            out[f"{func}_{name}_weights"], out[f"{func}_{name}_indices"] = w.numpy(), i.numpy()
    np.savez_compressed(HERE / "router.npz", **out)


def residency_fixture(checkout: Path) -> None:
    """A step-by-step trace of the reference's ``Cache`` policy (scripts/v41_build/omlx_routed.py:
    167-247: begin -> harvest -> install / admit / evict) on a seeded demand stream, with reads that
    land on a scripted schedule.  The reference class runs unmodified; only its storage hooks
    (``slabs`` / ``route`` / ``unroute``) and its reader pool are stand-ins."""
    import json
    import os
    import types

    sys.path.insert(0, str(checkout / "scripts" / "v41_build"))
    os.environ.update(OMLX_ROUTED_TAU="0.3", OMLX_ROUTED_SPARE="2", OMLX_ROUTED_LAG="2")
    omlx_routed = load_by_path("keep_reference_omlx_routed", checkout / "scripts" / "v41_build" / "omlx_routed.py")

    landed: set[int] = set()

    class Future:
        def __init__(self, expert):
            self.expert = expert

        def done(self):
            return self.expert in landed

        def result(self):
            return 64

    class Pool:
        def submit(self, fn, expert):
            return Future(expert)

    class Layer:
        def __init__(self, index, hot, rank):
            self.index = index
            self.slot_expert = np.array(hot, dtype=np.int64)
            self.slot_of = {e: s for s, e in enumerate(hot)}
            self.last_use = -1.0 - np.array(rank, dtype=np.float64)
            self.cooling, self.free, self.reading = [], [], {}

        def views_current(self):
            return True

    log: list = []

    class Trace(omlx_routed.Cache):
        def slabs(self, layer, expert, slot):
            return [(expert,)]

        def route(self, layer, expert, slot):
            log.append(("route", layer.index, int(expert), int(slot)))

        def unroute(self, layer, expert, slot):
            log.append(("unroute", layer.index, int(expert), int(slot)))

    pool_size, slots, k, tokens, steps = 24, 10, 3, 4, 14
    config = types.SimpleNamespace(score_func="sqrtsoftplus", n_activated_experts=k, route_scale=1.5)
    cache = Trace(config, None)
    cache.pool = Pool()
    rng = np.random.default_rng(77)
    layers = []
    for index in range(2):
        hot = rng.permutation(pool_size)[:slots].tolist()
        layers.append(Layer(index, hot, rank=list(range(slots))))
    cache.layers = layers
    init = [dict(slot_expert=l.slot_expert.tolist(), last_use=l.last_use.tolist()) for l in layers]

    trace = []
    for step in range(1, steps + 1):
        demand = []
        for layer in layers:
            index = np.stack([rng.choice(pool_size, k, replace=False) for _ in range(tokens)]).astype(np.uint32)
            weight = rng.uniform(0.05, 1.0, size=(tokens, k)).astype(np.float32) ** 2
            demand.append((index, weight))
        cache.pending[cache.step + 1] = demand  # what observe() records while call step+1 is built
        # each outstanding read lands with probability 0.6 before this tick (same flag for both layers)
        for layer in layers:
            for expert in list(layer.reading):
                if rng.random() < 0.6:
                    landed.add(expert)
        before = len(log)
        landed_now = sorted(int(e) for e in landed)  # per layer: expert ids whose bytes are in
        cache.begin()
        landed.clear()  # a landed read is consumed by the install of this tick
        trace.append(dict(
            step=cache.step, landed=landed_now,
            demand=[dict(index=i.tolist(), weight=[[float(v) for v in row] for row in w]) for i, w in demand],
            layers=[dict(slot_expert=l.slot_expert.tolist(),
                         last_use=[None if not np.isfinite(v) else float(v) for v in l.last_use],
                         free=[int(s) for s in l.free], cooling=[[int(s), int(c)] for s, c in l.cooling],
                         reading={str(int(e)): int(s) for e, (s, _) in l.reading.items()}) for l in layers],
            stats={key: (float(v) if key == "policy_s" else int(v)) for key, v in cache.stats.items() if key != "policy_s"},
            actions=[list(a) for a in log[before:]]))
    (HERE / "residency_trace.json").write_text(json.dumps(dict(
        tau=cache.tau, spare=cache.spare, lag=cache.lag, route_scale=1.5, top_k=k, pool=pool_size, slots=slots,
        init=init, trace=trace), indent=0))


def main() -> None:
    checkout = Path(sys.argv[1]).resolve()
    sys.path.insert(0, str(checkout / "src"))
    from keep.vq import e8

    codebook_fixture(e8)
    operator_fixture(checkout)
    router_fixture(checkout)
    residency_fixture(checkout)
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
