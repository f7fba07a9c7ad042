"""The residency-policy oracle replayed against a trace of the reference's own Cache (no GPU)."""

import json

import numpy as np

from conftest import GOLDEN
from oracle import residency


def load_trace():
    return json.loads((GOLDEN / "residency_trace.json").read_text())


def replay(trace, tick):
    """Drive `tick(layer_index, index, weight, landed, call, step) -> None` over the trace the way
    Cache.begin does: the demand recorded for call s is harvested at step s + lag."""
    pending = {}
    for record in trace["trace"]:
        step = record["step"]
        pending[step] = record["demand"]
        ready = step - trace["lag"]
        if ready in pending:
            demand = pending.pop(ready)
            for layer, d in enumerate(demand):
                tick(layer, np.array(d["index"]), np.array(d["weight"], dtype=np.float32), set(record["landed"]), ready, step)
        yield record


def test_oracle_reproduces_the_reference_trace_step_for_step():
    trace = load_trace()
    states = [residency.LayerState.start(i["slot_expert"], i["last_use"]) for i in trace["init"]]
    stats, actions = residency.new_stats(), []

    def tick(layer, index, weight, landed, call, step):
        if layer == 0:
            stats["calls"] += 1
        residency.harvest_layer(states[layer], index, weight, landed, call=call, step=step, tau=trace["tau"], spare=trace["spare"],
                                route_scale=trace["route_scale"], stats=stats, actions=actions, layer=layer)

    for record in replay(trace, tick):
        for layer, want in enumerate(record["layers"]):
            s = states[layer]
            assert s.slot_expert.tolist() == want["slot_expert"], (record["step"], layer)
            assert [None if not np.isfinite(v) else float(v) for v in s.last_use] == want["last_use"]
            assert s.free == want["free"] and [list(c) for c in s.cooling] == want["cooling"]
            assert {str(e): int(sl) for e, sl in s.reading.items()} == want["reading"]
        assert actions == record["actions"], record["step"]
        actions.clear()
        for key, value in record["stats"].items():
            if key != "bytes":  # the stand-in reader reports a made-up byte count
                assert stats[key] == value, (record["step"], key)
    assert stats["admitted"] > 10 and stats["evicted"] > 10 and stats["no_slot"] > 10, "the trace should exercise every branch"
