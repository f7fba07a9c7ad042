"""Admission / eviction bookkeeping of the routed expert cache, restated on the CPU.

TEST INFRASTRUCTURE: the checker for the CUDA policy kernel, never shipped.

Follows ``scripts/v41_build/omlx_routed.py`` of the reference, one layer at a time:

* ``tick``      ``Cache.begin`` + ``Cache.harvest``   ``omlx_routed.py:167-216``
* ``install``   ``Cache.install``                     ``omlx_routed.py:218-229``
* ``evict``     ``Cache.evict``                       ``omlx_routed.py:231-247``

"Bytes landed" is an explicit input (a set of expert ids), so a trace can be replayed step for
step.  Pinned against a trace of the reference's own class (``tests/golden/residency_trace.json``).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

STAT_NAMES = ("calls", "tokens", "demand", "resident", "wanted", "admitted", "installed", "evicted", "bytes", "no_slot")


@dataclass
class LayerState:
    slot_expert: np.ndarray                       # int64 [slots], -1 = unrouted
    last_use: np.ndarray                          # float64 [slots]
    slot_of: dict = field(default_factory=dict)   # expert -> slot
    free: list = field(default_factory=list)
    cooling: list = field(default_factory=list)   # (slot, call that unrouted it)
    reading: dict = field(default_factory=dict)   # expert -> slot, insertion ordered

    @classmethod
    def start(cls, slot_expert, last_use):
        se = np.asarray(slot_expert, dtype=np.int64).copy()
        return cls(se, np.asarray(last_use, dtype=np.float64).copy(), {int(e): s for s, e in enumerate(se) if e >= 0})


def install(state: LayerState, landed, step: int, stats: dict, actions: list, layer: int) -> None:
    """Route every read whose bytes have landed (``omlx_routed.py:218-229``)."""
    for expert in [e for e in state.reading if e in landed]:
        slot = state.reading.pop(expert)
        actions.append(["route", layer, int(expert), int(slot)])
        state.slot_expert[slot], state.slot_of[expert] = expert, slot
        state.last_use[slot] = step
        stats["installed"] += 1


def evict(state: LayerState, protected: set, spare: int, step: int, stats: dict, actions: list, layer: int) -> None:
    """Unroute the least recently strongly demanded residents until ``spare`` slots are free or
    cooling (``omlx_routed.py:231-247``): stable order of ``last_use``, demanded experts spared."""
    short = spare - len(state.free) - len(state.cooling)
    if short <= 0:
        return
    order = np.argsort(state.last_use, kind="stable")
    victims = [int(s) for s in order if state.slot_expert[s] >= 0 and int(state.slot_expert[s]) not in protected]
    for slot in victims[:short]:
        expert = int(state.slot_expert[slot])
        del state.slot_of[expert]
        state.slot_expert[slot] = -1
        state.last_use[slot] = np.inf
        actions.append(["unroute", layer, expert, slot])
        state.cooling.append((slot, step))
        stats["evicted"] += 1


def harvest_layer(state: LayerState, index, weight, landed, *, call: int, step: int, tau: float, spare: int,
                  route_scale: float, stats: dict, actions: list, layer: int) -> list:
    """One layer of ``Cache.harvest`` (``omlx_routed.py:184-216``).  Returns the admissions made:
    [(expert, slot)]."""
    index = np.asarray(index).astype(np.int64)
    w = np.asarray(weight, dtype=np.float64).reshape(index.shape)
    w = w / (w.sum(-1, keepdims=True) + 1e-20) * route_scale
    if layer == 0:
        stats["tokens"] += index.shape[0]
    stats["demand"] += index.size
    strong = w >= tau
    wanted: dict[int, float] = {}
    for e, g in zip(index[strong].tolist(), w[strong].tolist()):
        wanted[e] = max(g, wanted.get(e, 0.0))
    stats["resident"] += sum(e in state.slot_of for e in index.reshape(-1).tolist())
    install(state, landed, step, stats, actions, layer)
    missing = []
    for e, g in wanted.items():
        slot = state.slot_of.get(e)
        if slot is not None:
            state.last_use[slot] = call
        elif e not in state.reading:
            missing.append((g, e))
    stats["wanted"] += len(missing)
    state.free += [slot for slot, since in state.cooling if since <= call]
    state.cooling = [(slot, since) for slot, since in state.cooling if since > call]
    admitted = []
    for _, e in sorted(missing, reverse=True):
        if not state.free:
            stats["no_slot"] += 1
            continue
        slot = state.free.pop()
        state.reading[e] = slot
        admitted.append((e, slot))
        stats["admitted"] += 1
    evict(state, set(wanted), spare, step, stats, actions, layer)
    return admitted


def new_stats() -> dict:
    return dict.fromkeys(STAT_NAMES, 0)
