"""Routed residency bookkeeping on the device: admit, install, evict, one kernel per layer tick.

The reference keeps this policy in host Python (``Cache.begin / harvest / install / evict``,
``scripts/v41_build/omlx_routed.py:167-247``) and reads the demand back two calls late.  Here the
state lives in device arrays and ``keepvq_residency_tick`` updates the router tables in place, so
a decode call is never followed by a host read.  The host only feeds ``landed`` flags (a read has
finished) and drains the action log (reads to start, slots that were unrouted).
"""

from __future__ import annotations

import numpy as np
import torch

from . import _lib
from .router import OFF

STAT_NAMES = ("calls", "tokens", "demand", "resident", "wanted", "admitted", "installed", "evicted", "bytes", "no_slot")
ACTION_NAMES = {1: "route", 2: "unroute", 3: "admit"}


class LayerResidency:
    """Residency state of one layer.

    ``slot_expert`` [slots]: the starting residents (slot -> expert); ``last_use`` [slots]: their
    starting recency (the reference starts colder experts lower, ``omlx_routed.py:77``).
    ``served_bias`` and ``slot_of`` are the tensors a ``RoutedMoELayer`` routes with: pass the
    layer's own so that ticks and decode calls share them.
    """

    def __init__(self, slot_expert, last_use, pool: int, *, device, pool_bias=None, served_bias=None, slot_of=None,
                 tau: float = 0.3, spare: int = 4, route_scale: float = 1.0, top_k: int = 6, max_actions: int = 4096):
        se = np.asarray(slot_expert, dtype=np.int64)
        self.slots, self.pool, self.device = int(se.shape[0]), int(pool), torch.device(device)
        self.tau, self.spare, self.route_scale, self.top_k = float(tau), int(spare), float(route_scale), int(top_k)
        dev = self.device
        self.slot_expert = torch.from_numpy(se.astype(np.int32)).to(dev)
        self.last_use = torch.from_numpy(np.asarray(last_use, dtype=np.float64).copy()).to(dev)
        self.pool_bias = None if pool_bias is None else torch.as_tensor(pool_bias, dtype=torch.float32).to(dev).contiguous()
        if slot_of is None:
            table = np.full(self.pool, 0xFFFFFFFF, dtype=np.uint32)
            table[se[se >= 0]] = np.flatnonzero(se >= 0).astype(np.uint32)
            slot_of = torch.from_numpy(table).to(dev)
        if served_bias is None:
            bias = np.full(self.pool, OFF, dtype=np.float32)
            bias[se[se >= 0]] = 0.0 if pool_bias is None else np.asarray(pool_bias, dtype=np.float32)[se[se >= 0]]
            served_bias = torch.from_numpy(bias).to(dev)
        self.slot_of, self.served_bias = slot_of, served_bias
        i32 = lambda *shape: torch.zeros(shape, dtype=torch.int32, device=dev)  # noqa: E731
        self.free_list, self.cooling, self.reading, self.counts = i32(self.slots), i32(self.slots, 2), i32(self.slots, 2), i32(3)
        self.stats = torch.zeros(len(STAT_NAMES), dtype=torch.int64, device=dev)
        self.landed = torch.zeros(self.pool, dtype=torch.uint8, device=dev)
        self.actions, self.action_count, self.max_actions = i32(max_actions, 3), i32(1), int(max_actions)

    def tick(self, want: torch.Tensor, want_score: torch.Tensor, *, call: int, step: int, first_layer: bool = False) -> None:
        """Harvest the demand of call ``call`` while call ``step`` is being built.  Enqueued on the
        current stream; reads nothing back."""
        _lib.require_cuda(want, want_score)
        tokens = int(want.shape[0])
        args = _lib.ResidencyArgs(
            slot_expert=_lib.ptr(self.slot_expert), slot_of=_lib.ptr(self.slot_of), served_bias=_lib.ptr(self.served_bias),
            pool_bias=_lib.ptr(self.pool_bias), last_use=_lib.ptr(self.last_use), free_list=_lib.ptr(self.free_list),
            cooling=_lib.ptr(self.cooling), reading=_lib.ptr(self.reading), counts=_lib.ptr(self.counts), stats=_lib.ptr(self.stats),
            pool=self.pool, slots=self.slots, want=_lib.ptr(want.contiguous()), want_score=_lib.ptr(want_score.contiguous()),
            tokens=tokens, top_k=self.top_k, landed=_lib.ptr(self.landed), call=int(call), step=int(step), tau=self.tau,
            route_scale=self.route_scale, spare=self.spare, first_layer=int(first_layer),
            actions=_lib.ptr(self.actions), action_count=_lib.ptr(self.action_count), max_actions=self.max_actions)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().keepvq_residency_tick(args, _lib.stream_handle(self.device)), "keepvq_residency_tick")

    # ---- host-side helpers (synchronise; for installers, logs and tests, not the token path) ----
    def drain_actions(self) -> list[tuple[str, int, int]]:
        n = min(int(self.action_count.item()), self.max_actions)
        rows = self.actions[:n].cpu().tolist()
        self.action_count.zero_()
        return [(ACTION_NAMES[k], e, s) for k, e, s in rows]

    def snapshot(self) -> dict:
        counts = self.counts.cpu().tolist()
        last = self.last_use.cpu().numpy()
        return dict(
            slot_expert=self.slot_expert.cpu().tolist(),
            last_use=[None if not np.isfinite(v) else float(v) for v in last],
            free=self.free_list[: counts[0]].cpu().tolist(), cooling=self.cooling[: counts[1]].cpu().tolist(),
            reading={str(e): s for e, s in self.reading[: counts[2]].cpu().tolist()},
            stats=dict(zip(STAT_NAMES, self.stats.cpu().tolist())))


class SlotInstaller:
    """Carries out the reads the policy admits: an expert's stored bytes go from pinned host
    memory into its slot's rows of the layer's weight tensors, on a copy stream of their own.

    The reference reads with ``preadv`` into unified memory from reader threads and checks the
    bytes afterwards (``scripts/v41_build/omlx_routed.py:114-145,218-229``).  Here a read is a
    handful of ``cudaMemcpyAsync`` calls (one per tensor of the slot) followed, on the same copy
    stream, by a one-byte store into the policy's ``landed`` flags.  The next policy tick that sees
    the flag routes the expert, so by stream order its bytes are in place before any kernel can be
    routed to the slot, and nobody waits for a copy: not the host, not the token path.  Slots are
    only ever written while unrouted and cooled (the policy hands out free slots, and frees an
    evicted slot only after the calls that could still read it).

    ``store`` maps a tensor name (``w1_codes``, ``w1_scales``, ... ``w2_scales``) to a pinned host
    tensor ``[pool, ...]``; ``weights`` maps the same names to the layer's device tensors
    ``[slots, ...]``.
    """

    NAMES = tuple(f"{p}_{f}" for p in ("w1", "w3", "w2") for f in ("codes", "scales"))

    def __init__(self, residency: LayerResidency, store: dict, weights: dict):
        self.residency, self.store, self.weights = residency, store, weights
        for name in self.NAMES:
            host, dev = store[name], weights[name]
            if not host.is_pinned():
                raise ValueError(f"store[{name!r}] must be pinned host memory")
            if tuple(host.shape[1:]) != tuple(dev.shape[1:]) or host.dtype != dev.dtype:
                raise ValueError(f"store[{name!r}] rows do not match the layer's {name}")
        self.stream = torch.cuda.Stream(device=residency.device)
        self._one = torch.ones(1, dtype=torch.uint8).pin_memory()
        self.bytes_copied = 0

    def execute(self, actions) -> int:
        """Start the read of every ``("admit", expert, slot)`` in ``actions`` (what
        ``LayerResidency.drain_actions`` returns).  Returns the number of reads started."""
        started = 0
        # the reads may only start once the tick that admitted them (and the kernels before it) has run
        self.stream.wait_stream(torch.cuda.current_stream(self.residency.device))
        with torch.cuda.stream(self.stream):
            for kind, expert, slot in actions:
                if kind != "admit":
                    continue
                for name in self.NAMES:
                    self.weights[name][slot].copy_(self.store[name][expert], non_blocking=True)
                    self.bytes_copied += self.store[name][expert].numel() * self.store[name].element_size()
                self.residency.landed[expert : expert + 1].copy_(self._one, non_blocking=True)
                started += 1
        return started

    def differing(self, slot: int) -> int:
        """Tensors of a routed slot whose bytes differ from its expert's stored bytes
        (``omlx_routed.py:138-145``).  Synchronises; for checks, not the token path."""
        expert = int(self.residency.slot_expert[slot].item())
        if expert < 0:
            return 0
        self.stream.synchronize()
        return sum(not torch.equal(self.weights[name][slot].cpu(), self.store[name][expert]) for name in self.NAMES)
