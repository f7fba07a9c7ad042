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


def test_decode_loop_with_admissions_and_installs(cuda):
    """The whole routed-residency cycle on one layer: decode calls serve the resident half of the
    pool, the policy kernel admits strongly demanded absent experts, the installer copies their
    bytes from pinned host memory into free slots on its own stream and raises the landed flag,
    a later tick routes them, and later calls serve them.  Every call's output must equal the
    oracle's for the experts that call actually served, every routed slot must hold its expert's
    stored bytes, and nothing but the action drain reads the device."""
    import synthetic
    from keep_b200 import moe, residency
    from keep_b200.router import OFF
    from oracle import e8, router as oracle_router

    pool, slots, hidden, inter, k, tokens = 16, 10, 512, 256, 2, 4
    cfg = synthetic.layer(seed=90, experts=pool, hidden=hidden, inter=inter)
    start = list(range(6))                                 # experts 0..5 resident in slots 0..5, slots 6..9 free
    names = residency.SlotInstaller.NAMES
    full = {f"{p}_{f}": torch.from_numpy(cfg[p][i]) for p in ("w1", "w3", "w2") for i, f in enumerate(("codes", "scales"))}
    store = {n: full[n].pin_memory() for n in names}
    weights = {n: torch.zeros((slots,) + tuple(full[n].shape[1:]), dtype=full[n].dtype, device=cuda) for n in names}
    for n in names:
        weights[n][: len(start)] = full[n][start].to(cuda)
    state = residency.LayerResidency(start + [-1] * (slots - len(start)), [-1.0 - r for r in range(slots)], pool, device=cuda,
                                     tau=0.3, spare=1, top_k=k)
    # the starting free list: slots 6..9
    state.free_list[: slots - len(start)] = torch.arange(len(start), slots, dtype=torch.int32, device=cuda)
    state.counts[0] = slots - len(start)
    layer = moe.RoutedMoELayer(cfg["router"].to(cuda), moe.Projection(weights["w1_codes"], weights["w1_scales"]),
                               moe.Projection(weights["w3_codes"], weights["w3_scales"]),
                               moe.Projection(weights["w2_codes"], weights["w2_scales"]), top_k=k, tau=0.3,
                               served_bias=state.served_bias, slot_of=state.slot_of)
    layer.served_bias, layer.slot_of = state.served_bias, state.slot_of  # the very tensors the policy updates
    installer = residency.SlotInstaller(state, store, weights)
    dense = {p: oracle_router.dense_slots(*cfg[p], range(pool)) for p in ("w1", "w3", "w2")}  # every expert, by expert id

    served_after_install, installed = 0, set()
    for step in range(1, 15):
        x = synthetic.tokens(900 + step, tokens, hidden)
        out, routing = layer.decode(x.to(cuda))
        served_expert = routing.served_expert.cpu().numpy().astype(np.int64)
        served_slot = routing.served_slot.cpu().numpy().astype(np.int64)
        weight = routing.served_weight.cpu().numpy()
        slot_expert = state.slot_expert.cpu().numpy()
        live = served_expert >= 0
        assert (slot_expert[served_slot[live]] == served_expert[live]).all()        # routed where the policy says
        served_after_install += int(np.isin(served_expert[live], list(installed)).sum())
        ref = oracle_router.moe_layer(x, np.where(live, served_expert, -1), weight, dense["w1"], dense["w3"], dense["w2"])
        assert e8.relative_gap(out.float().cpu().numpy(), ref.numpy()) <= 1e-2
        state.tick(routing.want, routing.want_score, call=step, step=step + 1, first_layer=True)
        actions = state.drain_actions()
        installed |= {e for kind, e, _ in actions if kind == "route"}
        installer.execute(actions)
        for slot in range(slots):                                                  # the reference's byte check
            assert installer.differing(slot) == 0
    snap = state.snapshot()
    assert snap["stats"]["admitted"] >= 2 and snap["stats"]["installed"] >= 2, snap["stats"]
    assert served_after_install > 0, "no installed expert was served afterwards"
    absent = np.setdiff1d(np.arange(pool), [e for e in snap["slot_expert"] if e >= 0])
    assert (state.served_bias.cpu().numpy()[absent] == np.float32(OFF)).all()


def test_layer_served_from_a_layer_file(cuda, tmp_path):
    """layer-NN.npz -> resident slots on the device and a pinned store for the installer: a decode
    call over tensors loaded that way equals the oracle on the file's arrays, and an install copies
    exactly the file's bytes of that expert."""
    import synthetic
    from keep_b200 import io as layer_io, moe, residency
    from oracle import e8, router as oracle_router

    pool, hidden, inter, k = 8, 512, 256, 2
    cfg = synthetic.layer(seed=95, experts=pool, hidden=hidden, inter=inter)
    path = tmp_path / "layer-00.npz"
    np.savez(path, code_bits=np.asarray(16), **{f"{p}_{f}": cfg[p][i] for p in ("w1", "w3", "w2") for i, f in enumerate(("codes", "scales"))})
    layer_file = layer_io.LayerFile(path)
    residents = [5, 2, 7, 0]                                    # slot s holds expert residents[s]; two more slots stay free
    slots = len(residents) + 2
    weights = {}
    for p in ("w1", "w3", "w2"):
        proj = layer_io.projection(layer_file, p, residents, cuda)
        for f, t in (("codes", proj.codes), ("scales", proj.scales)):
            weights[f"{p}_{f}"] = torch.cat([t, torch.zeros((2,) + tuple(t.shape[1:]), dtype=t.dtype, device=cuda)])
    state = residency.LayerResidency(residents + [-1, -1], [-1.0] * slots, pool, device=cuda, top_k=k)
    layer = moe.RoutedMoELayer(cfg["router"].to(cuda), *(moe.Projection(weights[f"{p}_codes"], weights[f"{p}_scales"]) for p in ("w1", "w3", "w2")),
                               top_k=k, served_bias=state.served_bias, slot_of=state.slot_of)
    x = synthetic.tokens(96, 5, hidden)
    out, routing = layer.decode(x.to(cuda))
    experts = routing.served_expert.cpu().numpy().astype(np.int64)
    assert np.isin(experts, residents).all()
    dense = {p: oracle_router.dense_slots(*cfg[p], range(pool)) for p in ("w1", "w3", "w2")}
    ref = oracle_router.moe_layer(x, experts, routing.served_weight.cpu().numpy(), dense["w1"], dense["w3"], dense["w2"])
    assert e8.relative_gap(out.float().cpu().numpy(), ref.numpy()) <= 1e-2
    installer = residency.SlotInstaller(state, layer_io.store(layer_file), weights)
    assert installer.execute([("admit", 3, 4)]) == 1
    installer.stream.synchronize()
    assert int(state.landed[3].item()) == 1
    for name in residency.SlotInstaller.NAMES:
        offset, size = layer_file.slab(name, 3)
        with open(path, "rb") as f:
            f.seek(offset)
            assert weights[name][4].cpu().numpy().tobytes() == f.read(size)
