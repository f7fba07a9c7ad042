"""The device-side residency policy replayed against the trace of the reference's own Cache and
against the CPU oracle: every list, table and counter identical after every step."""

import numpy as np
import pytest
import torch

from oracle import residency as oracle_residency
from test_oracle_residency import load_trace, replay

pytestmark = pytest.mark.gpu


def test_device_policy_reproduces_the_reference_trace(cuda):
    from keep_b200 import residency
    from keep_b200.router import OFF

    trace = load_trace()
    layers = [residency.LayerResidency(i["slot_expert"], i["last_use"], trace["pool"], device=cuda, tau=trace["tau"],
                                       spare=trace["spare"], route_scale=trace["route_scale"], top_k=trace["top_k"])
              for i in trace["init"]]

    def tick(layer, index, weight, landed, call, step):
        state = layers[layer]
        flags = np.zeros(trace["pool"], dtype=np.uint8)
        flags[list(landed)] = 1
        state.landed.copy_(torch.from_numpy(flags))
        state.tick(torch.from_numpy(index.astype(np.int32)).to(cuda), torch.from_numpy(weight).to(cuda), call=call, step=step,
                   first_layer=layer == 0)

    for record in replay(trace, tick):
        actions = []
        for layer, want in enumerate(record["layers"]):
            got = layers[layer].snapshot()
            for key in ("slot_expert", "last_use", "free", "cooling", "reading"):
                assert got[key] == want[key], (record["step"], layer, key)
            actions += [[kind, layer, e, s] for kind, e, s in layers[layer].drain_actions() if kind != "admit"]
            # router tables follow the slots
            slot_of = layers[layer].slot_of.cpu().numpy().astype(np.int64)
            bias = layers[layer].served_bias.cpu().numpy()
            for slot, expert in enumerate(want["slot_expert"]):
                if expert >= 0:
                    assert slot_of[expert] == slot and bias[expert] == 0.0
            absent = np.setdiff1d(np.arange(trace["pool"]), [e for e in want["slot_expert"] if e >= 0])
            assert (slot_of[absent] == 0xFFFFFFFF).all() and (bias[absent] == np.float32(OFF)).all()
        assert sorted(actions) == sorted(record["actions"]), record["step"]
        totals = {k: sum(layer.snapshot()["stats"][k] for layer in layers) for k in oracle_residency.STAT_NAMES}
        for key, value in record["stats"].items():
            if key != "bytes":
                assert totals[key] == value, (record["step"], key)


def test_tau_infinity_keeps_the_starting_set(cuda):
    """With tau = inf nothing is strong: no admission, no eviction beyond the spare slots
    (scripts/v41_build/omlx_routed.py:20-21)."""
    from keep_b200 import residency

    state = residency.LayerResidency(list(range(6)), [-1.0 - r for r in range(6)], 12, device=cuda, tau=float("inf"), spare=0, top_k=2)
    want = torch.tensor([[7, 8], [9, 1]], dtype=torch.int32, device=cuda)
    score = torch.tensor([[0.9, 0.1], [0.8, 0.2]], device=cuda)
    for step in range(3, 6):
        state.tick(want, score, call=step - 2, step=step, first_layer=True)
    snap = state.snapshot()
    assert snap["slot_expert"] == list(range(6)) and not snap["reading"] and not snap["cooling"]
    assert snap["stats"]["admitted"] == 0 and snap["stats"]["evicted"] == 0 and snap["stats"]["calls"] == 3
