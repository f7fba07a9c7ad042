"""Benchmark of the routed E8P MoE layer (decode) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

A step is one pass of one routed MoE layer (384 experts, hidden 4096, inter 2048, top-6, softmax
router, uniform-random E8P codes, per-row fp16 scales) over one batch of B decode tokens.  Token
batches rotate over 64 different seeded batches so that successive steps touch different experts
of the 2.4 GB pool (larger than L2).  Prints ONE JSON line on rank 0.

``value``      tokens/s with inputs resident in HBM, timed with CUDA events around a CUDA-graph
               replay of the K steps (no host launch gaps inside the timed region).
``e2e``        the same metric through ``RoutedMoELayer.decode`` from pinned host buffers: the
               H2D copy of the tokens and the D2H copy of the layer output are inside the region.
``roofline``   the dominant kernel (expert projections) timed alone with CUDA events: distinct
               served experts x code bytes per launch / launch time, against the measured HBM peak.
``cpu_baseline``  the CPU oracle (a port of the reference's CPU path) timed on the host cores on
               a bounded sample (one token through its six experts, decode included).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

EXPERTS, HIDDEN, INTER, TOP_K = 384, 4096, 2048, 6
CODE_BYTES_PER_PROJECTION = INTER * HIDDEN // 8 * 2          # 2,097,152
CODE_BYTES_PER_EXPERT = 3 * CODE_BYTES_PER_PROJECTION        # 6,291,456
ROTATION = 64
METRIC, UNIT = "routed VQ MoE layer tokens/s", "tokens/s"


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML every 5 ms (read
    only), or nvidia-smi every 200 ms when the NVML binding is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index: int):
        self.index, self.rows, self.stop_flag, self.thread = index, [], threading.Event(), None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            bus = torch.cuda.get_device_properties(self.index).pci_bus_id
            domain = getattr(torch.cuda.get_device_properties(self.index), "pci_domain_id", 0)
            device = getattr(torch.cuda.get_device_properties(self.index), "pci_device_id", 0)
            return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(f"{domain:08x}:{bus:02x}:{device:02x}.0".encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _run(self):
        try:
            nvml, handle = self._nvml_handle()
            top = nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM)
            while not self.stop_flag.is_set():
                mask = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.rows.append([str(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)), str(top)] +
                                 ["Active" if mask & bit else "Not Active" for _, bit in self.REASON_BITS])
                self.stop_flag.wait(0.005)
            return
        except Exception:
            pass
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop_flag.set()
        self.thread.join(timeout=6)

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in self.rows for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def build_layer(device, seed=0):
    """The benchmark layer with codes drawn on the device (uniform uint16), scales 0.02*U(0.5,1.5)."""
    from keep_b200 import moe

    gen = torch.Generator(device=device)
    gen.manual_seed(seed)

    def proj(out, inp):
        codes = torch.randint(0, 1 << 16, (EXPERTS, out, inp // 8), generator=gen, device=device, dtype=torch.int32).to(torch.uint16)
        scales = (0.02 * (0.5 + torch.rand((EXPERTS, out, 1), generator=gen, device=device))).to(torch.float16)
        return moe.Projection(codes, scales)

    router = (0.02 * torch.randn((EXPERTS, HIDDEN), generator=gen, device=device)).to(torch.bfloat16)
    return moe.RoutedMoELayer(router, proj(INTER, HIDDEN), proj(INTER, HIDDEN), proj(HIDDEN, INTER), top_k=TOP_K)


def token_batches(device, batch, count=ROTATION):
    gen = torch.Generator(device="cpu")
    gen.manual_seed(1 + batch)
    return [torch.randn((batch, HIDDEN), generator=gen).to(torch.bfloat16).to(device) for _ in range(count)]


REPLAYS = 7


def time_graph(fn, steps, warmup, replays=REPLAYS, every=False, warm_fn=None):
    """CUDA-event time of `steps` calls of fn(i) replayed from one CUDA graph, in ms: the median of
    `replays` timed replays (after one untimed replay).  With ``every`` the list of all replay
    times is returned as well.  ``warm_fn`` (default fn) runs the untimed eager warm-up calls."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for i in range(max(warmup, 3)):
            (warm_fn or fn)(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(steps):
                fn(i)
        graph.replay()  # one untimed replay
        torch.cuda.synchronize()
        times = []
        for _ in range(max(replays, 1)):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            graph.replay()
            end.record(stream)
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end))
    return (statistics.median(times), times) if every else statistics.median(times)


def distinct_experts(layer, xs):
    counts = []
    for x in xs:
        _, routing = layer.decode(x)
        served = routing.served_expert.cpu().numpy()
        counts.append(len({int(v) for v in served.reshape(-1) if v >= 0}))
    return counts


def projection_roofline(layer, xs, steps, hbm_gbs, peak_kind):
    """Times the dominant kernel alone: the gate/up projection stage (two of the three code streams
    of a layer).  Each rotating batch keeps its own scratch state, filled by one full call."""
    from keep_b200 import _lib

    uniq = []
    for j, x in enumerate(xs):
        _, r = layer.decode(x, state=1 + j)
        uniq.append(len({int(v) for v in r.served_expert.cpu().numpy().reshape(-1) if v >= 0}))

    def one(i):
        j = i % len(xs)
        layer.decode(xs[j], stages=_lib.STAGE_GATE_UP, state=1 + j)

    ms = time_graph(one, steps, 3)
    tensor = layer.kernel_path == "tensor"
    launches = 1 if tensor else 3  # general kernels: gate, up and the SwiGLU pass
    bytes_per_stage = statistics.fmean(uniq[i % len(xs)] for i in range(steps)) * 2 * CODE_BYTES_PER_PROJECTION
    achieved = bytes_per_stage / (ms / steps * 1e-3) / 1e9
    # DRAM bytes per launch are not measured in this run: they come from one ncu capture of this kernel
    # at batch 64 (dram__bytes_read.sum + dram__bytes_write.sum = 999.2 MB for 1025.4 MB of distinct code
    # bytes) and are scaled by the code bytes of the launch timed here.
    traffic = int(NCU_TRAFFIC_PER_CODE_BYTE * bytes_per_stage) if tensor else None
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s", "frac": round(achieved / hbm_gbs, 4),
            "traffic": traffic, "traffic_source": "one ncu capture of this kernel at batch 64 (dram__bytes_read.sum + dram__bytes_write.sum), scaled by this launch's code bytes; not measured in this run" if tensor else None,
            "peak_kind": peak_kind,
            "kernel": "projection_slab_kernel<2,1> (gate+up+SwiGLU, int8 tensor cores)" if tensor else "routed_rowdot_kernel x2 + swiglu",
            "launches_per_stage": launches, "algorithmic_bytes_per_launch": int(bytes_per_stage),
            "us_per_launch": round(ms / steps * 1e3, 2)}


NCU_TRAFFIC_PER_CODE_BYTE = 999.2 / 1025.4


def batch_sweep(layer, device, rotation, steps, hbm_gbs, batches=(1, 4, 16)):
    """The other decode batch sizes of config 2: layer tokens/s and the gate/up kernel's fraction
    of the HBM peak, measured the same way as the headline batch."""
    out = {}
    for b in batches:
        xs = token_batches(device, b, rotation)
        ms = time_graph(lambda i: layer.decode(xs[i % len(xs)]), steps, 3)
        roof = projection_roofline(layer, xs, steps, hbm_gbs, "")
        out[str(b)] = {"tokens_per_s": round(b * steps / (ms * 1e-3), 1), "layer_us": round(ms / steps * 1e3, 1),
                       "gate_up_us": roof["us_per_launch"], "gate_up_frac_of_hbm": roof["frac"]}
    return out


def residency_leg(layer, device, rotation, steps, hbm_gbs, batch=16, resident=192, hot=32):
    """Config 4: routed residency at batch 16.  Half the pool resident (seed 3), absent experts
    masked out of the served selection, the 32 resident experts a 4096-token warm-up routing
    selects most carry the nested 8-bit residual (scale 0.005), admissions at tau = 0.3.  Reports
    layer tokens/s and the GB/s of code bytes the served routes touch (base + residual)."""
    from keep_b200 import moe, router as router_ops

    cpu = torch.Generator().manual_seed(3)
    residents = torch.randperm(EXPERTS, generator=cpu)[:resident].sort().values
    slot_of = torch.full((EXPERTS,), 0xFFFFFFFF, dtype=torch.int64)
    slot_of[residents] = torch.arange(resident)
    served_bias = torch.full((EXPERTS,), -1e30)
    served_bias[residents] = 0.0
    gen = torch.Generator(device="cpu").manual_seed(4)
    warm = torch.randn((PREFILL_TOKENS, HIDDEN), generator=gen).to(torch.bfloat16).to(device)
    routed = router_ops.routed_topk(warm, layer.router_w, served_bias.numpy(), None, slot_of.numpy().astype(np.uint32), top_k=TOP_K)
    picks = routed.served_slot.reshape(-1).long()
    counts = torch.bincount(picks[picks < resident], minlength=resident)
    hot_slots = counts.topk(hot).indices.cpu()
    hot_of_slot = torch.full((resident,), 0xFFFFFFFF, dtype=torch.int64)
    hot_of_slot[hot_slots] = torch.arange(hot)
    dgen = torch.Generator(device=device).manual_seed(7)

    def with_residual(p, out, inp):
        res_codes = torch.randint(0, 256, (hot, out, inp // 8), generator=dgen, device=device, dtype=torch.int32).to(torch.uint8)
        res_scales = torch.full((hot, out, 1), 0.005, dtype=torch.float16, device=device)
        return moe.Projection(p.codes[:resident], p.scales[:resident], res_codes, res_scales)

    tiered = moe.RoutedMoELayer(layer.router_w, with_residual(layer.w1, INTER, HIDDEN), with_residual(layer.w3, INTER, HIDDEN),
                                with_residual(layer.w2, HIDDEN, INTER), top_k=TOP_K, tau=0.3, served_bias=served_bias.numpy(),
                                slot_of=slot_of.numpy().astype(np.uint32), hot_of_slot=hot_of_slot.numpy().astype(np.uint32))
    xs = token_batches(device, batch, rotation)
    base_u, hot_u, admitted = [], [], []
    for j, x in enumerate(xs):
        _, r = tiered.decode(x, state=1 + j)
        slots = {int(v) for v in r.served_slot.cpu().numpy().astype("int64").reshape(-1) if 0 <= v < resident}
        base_u.append(len(slots))
        hot_u.append(sum(1 for v in slots if int(hot_of_slot[v]) < hot))
        admitted.append(int((r.admit >= 0).sum()))
    ms = time_graph(lambda i: tiered.decode(xs[i % len(xs)]), steps, 3)
    code_bytes = statistics.fmean(base_u) * CODE_BYTES_PER_EXPERT + statistics.fmean(hot_u) * CODE_BYTES_PER_EXPERT / 2
    gbs = code_bytes / (ms / steps * 1e-3) / 1e9
    return {"batch": batch, "resident": resident, "hot": hot, "tokens_per_s": round(batch * steps / (ms * 1e-3), 1), "layer_us": round(ms / steps * 1e3, 1),
            "distinct_base_experts": round(statistics.fmean(base_u), 1), "distinct_hot_experts": round(statistics.fmean(hot_u), 1),
            "admissions_per_step": round(statistics.fmean(admitted), 1), "code_gbs": round(gbs, 1), "code_frac_of_hbm": round(gbs / hbm_gbs, 4),
            "kernel_path": tiered.kernel_path}


def stage_times(layer, xs, steps):
    """Microseconds per stage of the layer call, each stage replayed alone on the state the full
    calls of `projection_roofline` left behind (same rotation of token batches)."""
    from keep_b200 import _lib

    names = {"router": _lib.STAGE_ROUTER, "prepare": _lib.STAGE_PREPARE, "gate_up": _lib.STAGE_GATE_UP,
             "down": _lib.STAGE_DOWN, "combine": _lib.STAGE_COMBINE}
    return {k: round(time_graph(lambda i, m=m: layer.decode(xs[i % len(xs)], stages=m, state=1 + i % len(xs)), steps, 3) / steps * 1e3, 1)
            for k, m in names.items()}

PREFILL_TOKENS = 4096
PREFILL_FLOPS = 2.0 * PREFILL_TOKENS * TOP_K * (INTER * HIDDEN) * 3  # useful FLOPs of the three projections: 1.2369e12


def prefill_leg(layer, device, steps=6):
    """Config 3: 4096 tokens through the same layer (about 64 routes per expert; the skew variant
    shifts the router logits by a Zipf(1.1) per-expert bias).  Reports the whole layer and the
    expert projections alone (tcgen05 kernels), as TFLOP/s of useful bf16-equivalent work."""
    from keep_b200 import _lib

    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("bf16_tflops", 1590.0))
    gen = torch.Generator(device="cpu")
    gen.manual_seed(2)
    xs = [torch.randn((PREFILL_TOKENS, HIDDEN), generator=gen).to(torch.bfloat16).to(device) for _ in range(2)]
    out = {}
    for name in ("uniform", "zipf"):
        saved = layer.pool_bias, layer.served_bias
        if name == "zipf":
            rank = torch.randperm(EXPERTS, generator=gen).float() + 1.0
            bias = (-1.1 * torch.log(rank)).to(device)
            # the bias enters the selection only: scores + bias picks, weights come from raw scores
            layer.pool_bias = layer.served_bias = bias
        for j, x in enumerate(xs):
            _, r = layer.decode(x, state=100 + j)
        per_expert = torch.bincount(r.served_expert.reshape(-1).long().clamp(min=0), minlength=EXPERTS).cpu()
        ms_layer = time_graph(lambda i: layer.decode(xs[i % 2], state=100 + i % 2), steps, 3)
        expert_stages = _lib.STAGE_GATE_UP | _lib.STAGE_DOWN
        ms_experts = time_graph(lambda i: layer.decode(xs[i % 2], stages=expert_stages, state=100 + i % 2), steps, 3)
        out[name] = {
            "layer_ms": round(ms_layer / steps, 4), "layer_tokens_per_s": round(PREFILL_TOKENS / (ms_layer / steps * 1e-3), 1),
            "experts_ms": round(ms_experts / steps, 4), "experts_tflops": round(PREFILL_FLOPS / (ms_experts / steps * 1e-3) / 1e12, 1),
            "experts_frac_of_bf16_peak": round(PREFILL_FLOPS / (ms_experts / steps * 1e-3) / 1e12 / peak, 4),
            "routes_per_expert": {"mean": round(float(per_expert.float().mean()), 1), "max": int(per_expert.max()), "min": int(per_expert.min())}}
        if name == "uniform":  # where the layer's time goes, stage by stage
            names = {"router": _lib.STAGE_ROUTER, "prepare": _lib.STAGE_PREPARE, "gate_up": _lib.STAGE_GATE_UP,
                     "down": _lib.STAGE_DOWN, "combine": _lib.STAGE_COMBINE}
            out[name]["stage_ms"] = {k: round(time_graph(lambda i, m=m: layer.decode(xs[i % 2], stages=m, state=100 + i % 2), steps, 3) / steps, 4)
                                     for k, m in names.items()}
        layer.pool_bias, layer.served_bias = saved
    out["peak_tflops"], out["useful_flops"] = peak, PREFILL_FLOPS
    out["kernel"] = "prefill_projection_kernel (tcgen05.mma kind::i8, A decoded into tensor memory, B by TMA boxes into swizzled shared memory, two int8 MMAs per bf16-equivalent product)"
    threads = os.cpu_count() or 1
    cpu_s = cpu_expert_sample(layer, threads)
    out["cpu_baseline"] = {"seconds_per_expert": round(cpu_s, 3), "routes": 64, "cores": threads, "kind": "port",
                           "sample": "one of the 384 experts: decode of its three matrices + SwiGLU path for 64 token rows; the 4096-token call has 384 such experts",
                           "extrapolated_layer_tokens_per_s": round(PREFILL_TOKENS / (cpu_s * EXPERTS), 2)}
    return out


def operator_legs(layer, device, hbm_gbs, steps=32):
    """Config 1 (`vq_qmv`, one expert's gate matrix [2048 x 4096], one bf16 vector) and `gather_vqmm`
    with the direct strategy at 1, 4 and 16 tokens (top-6 routes over the layer's gate matrices),
    each replayed from a CUDA graph: microseconds per call and GB/s on the distinct code bytes the
    call touches, beside the CPU path of the same operator (decode + fp32 product, warmed once)."""
    from keep_b200 import kernels, vq, vq_switch
    from oracle import ops as oracle_ops

    table = vq.table_on(device, "e8p")
    gen = torch.Generator(device="cpu").manual_seed(0)
    x1 = torch.randn((HIDDEN,), generator=gen).to(torch.bfloat16).to(device)
    codes, scales = layer.w1.codes, layer.w1.scales
    out = {}
    # rotate over experts so that successive calls do not find their codes in L2
    ms = time_graph(lambda i: kernels.vq_qmv(x1, codes[i % EXPERTS], scales[i % EXPERTS], table, in_dim=HIDDEN, out_dim=INTER,
                                             group_size=HIDDEN, code_bits=16), steps, 3)
    us = ms / steps * 1e3
    c0, s0 = codes[0].cpu().numpy(), scales[0].cpu().numpy()
    xr = x1.float().cpu().numpy()
    oracle_ops.vq_qmv_reference(xr, c0, s0, None, code_bits=16)  # warm: builds the tables once
    begin = time.perf_counter()
    oracle_ops.vq_qmv_reference(xr, c0, s0, None, code_bits=16)
    cpu_s = time.perf_counter() - begin
    out["vq_qmv_2048x4096"] = {"us_per_call": round(us, 2), "code_gbs": round(CODE_BYTES_PER_PROJECTION / (us * 1e-6) / 1e9, 1),
                               "code_frac_of_hbm": round(CODE_BYTES_PER_PROJECTION / (us * 1e-6) / 1e9 / hbm_gbs, 4),
                               "cpu_us_per_call": round(cpu_s * 1e6, 1), "kernel": "keepvq_grouped_projection: group_routes, quantize_rows, projection_sweep_kernel (three launches per call)"}
    for tokens in (1, 4, 16):
        xs, picks, uniq = [], [], []
        for j in range(8):
            g = torch.Generator(device="cpu").manual_seed(100 + 8 * tokens + j)
            xs.append(torch.randn((tokens, HIDDEN), generator=g).to(torch.bfloat16).to(device))
            rhs = torch.stack([torch.randperm(EXPERTS, generator=g)[:TOP_K] for _ in range(tokens)]).to(torch.int32)
            uniq.append(len(set(rhs.reshape(-1).tolist())))
            picks.append(rhs.to(device))
        ms = time_graph(lambda i: vq_switch.gather_vqmm(xs[i % 8], codes, scales, table, picks[i % 8], input_dims=HIDDEN, output_dims=INTER,
                                                        group_size=HIDDEN, code_bits=16, route_strategy="direct"), steps, 3)
        us = ms / steps * 1e3
        touched = statistics.fmean(uniq) * CODE_BYTES_PER_PROJECTION
        out[f"gather_vqmm_direct_b{tokens}"] = {"us_per_call": round(us, 2), "routes": tokens * TOP_K, "code_gbs": round(touched / (us * 1e-6) / 1e9, 1),
                                                  "code_frac_of_hbm": round(touched / (us * 1e-6) / 1e9 / hbm_gbs, 4)}
    return out


def artifact_shape_leg(device, hbm_gbs, steps=32):
    """The shape and scale groups of the reference's shipped layers (hidden 5120 in groups of 512,
    inter 2304 in groups of 256, keep_quant.py:13-15; top-6 over 192 resident experts, the pool its
    served decode step routes over) at one and at four tokens: microseconds per layer call and
    GB/s on the distinct code bytes.  The reference's own figure for this step is 0.40-0.42 ms on
    an M4 Max (router, six lattice experts and the shared expert)."""
    from keep_b200 import moe

    experts, hidden, inter = 192, 5120, 2304
    gen = torch.Generator(device=device)
    gen.manual_seed(31)

    def proj(out, inp, group):
        codes = torch.randint(0, 1 << 16, (experts, out, inp // 8), generator=gen, device=device, dtype=torch.int32).to(torch.uint16)
        scales = (0.02 * (0.5 + torch.rand((experts, out, inp // group), generator=gen, device=device))).to(torch.float16)
        return moe.Projection(codes, scales)

    router = (0.02 * torch.randn((experts, hidden), generator=gen, device=device)).to(torch.bfloat16)
    layer = moe.RoutedMoELayer(router, proj(inter, hidden, 512), proj(inter, hidden, 512), proj(hidden, inter, 256), top_k=TOP_K)
    out = {"experts": experts, "hidden": hidden, "inter": inter, "scale_groups": "512 / 256", "kernel_path": layer.kernel_path}
    per_expert = 3 * hidden * inter // 8 * 2
    for batch in (1, 4):
        xs = [torch.randn((batch, hidden), generator=torch.Generator().manual_seed(500 + batch * 16 + j)).to(torch.bfloat16).to(device) for j in range(16)]
        uniq = statistics.fmean(int(torch.unique(layer.decode(x)[1].served_expert).numel()) for x in xs)
        ms = time_graph(lambda i: layer.decode(xs[i % 16]), steps, 3)
        us = ms / steps * 1e3
        out[str(batch)] = {"layer_us": round(us, 1), "code_frac_of_hbm": round(uniq * per_expert / (us * 1e-6) / 1e9 / hbm_gbs, 4)}
    del layer
    torch.cuda.empty_cache()
    return out


def cpu_expert_sample(layer, threads, routes=64):
    """One expert of the prefill leg on the CPU path: decode of its three matrices and the SwiGLU
    path for `routes` token rows (what the reference's CPU code does per expert).  Seconds."""
    from oracle import router as oracle_router

    torch.set_num_threads(threads)
    gen = torch.Generator(device="cpu").manual_seed(9)
    rows = torch.randn((routes, HIDDEN), generator=gen).to(torch.bfloat16)
    oracle_router.decode_torch(layer.w1.codes[1].cpu().numpy(), layer.w1.scales[1].cpu().numpy())  # warm the decode grid
    begin = time.perf_counter()
    w = {n: oracle_router.decode_torch(getattr(layer, n).codes[0].cpu().numpy(), getattr(layer, n).scales[0].cpu().numpy()) for n in ("w1", "w3", "w2")}
    slots = np.zeros((routes, 1), dtype=np.int64)
    oracle_router.moe_layer(rows, slots, np.ones((routes, 1), dtype=np.float32), {0: w["w1"]}, {0: w["w3"]}, {0: w["w2"]})
    return time.perf_counter() - begin


def cpu_layer_sample(layer, x_row, threads, experts_per_token=TOP_K):
    """One token through the CPU oracle: router, decode of its served experts' three projections
    (grid[codes] * scale, as the reference's CPU path does), the SwiGLU path with the served
    rounding points.  ``experts_per_token`` < top-k keeps only the strongest picks (a bounded
    sample).  Returns (seconds, output row)."""
    from oracle import router as oracle_router

    torch.set_num_threads(threads)
    begin = time.perf_counter()
    r = oracle_router.routed_topk(x_row, layer.router_w.cpu(), top_k=TOP_K)
    slots, weights = r["served_slot"].numpy().copy(), r["served_weight"].numpy()
    slots[:, experts_per_token:] = -1
    dense = {}
    for n in ("w1", "w3", "w2"):
        p = getattr(layer, n)
        dense[n] = {int(e): oracle_router.decode_torch(p.codes[int(e)].cpu().numpy(), p.scales[int(e)].cpu().numpy())
                    for e in slots.reshape(-1) if e >= 0}
    out = oracle_router.moe_layer(x_row, slots, weights, dense["w1"], dense["w3"], dense["w2"])
    return time.perf_counter() - begin, out


def run_reference(ns):
    """The reference arm: the CPU path of the layer on the host cores (oracle port), one token per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    device = torch.device("cuda", 0) if torch.cuda.is_available() else None
    if device is None:
        print(json.dumps({"impl": "reference", "unavailable": "the bench layer is generated on a CUDA device; none present"}))
        return
    layer = build_layer(device)
    xs = token_batches(device, 1, count=max(ns.steps + ns.warmup, 1))
    threads = os.cpu_count() or 1
    # a full token costs about 3 s of CPU; keep the whole run within a few minutes
    per_token = TOP_K if ns.steps <= 48 else max(1, (48 * TOP_K) // ns.steps)
    for i in range(min(ns.warmup, 1)):
        cpu_layer_sample(layer, xs[i].cpu(), threads, per_token)
    times = [cpu_layer_sample(layer, xs[(ns.warmup + i) % len(xs)].cpu(), threads, per_token)[0] for i in range(ns.steps)]
    total = sum(times)
    value = ns.steps * (per_token / TOP_K) / total
    line = {"metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": ns.gpus, "steps": ns.steps, "warmup": ns.warmup,
            "ms_per_step": round(total / ns.steps * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {"workload": ("decode layer (config 2)" if ns.gpus == 1 else "one layer of the expert-parallel stack (config 5; the unit is a token through one routed layer)")
                                   + ": 384 experts, hidden 4096, inter 2048, top-6 softmax router; CPU path, one token per step (bounded sample)"},
            "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"per step: router + {per_token} of a token's 6 served experts (decode of 3 projections each + SwiGLU path); value scaled to whole tokens"},
            "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


EP_LAYERS, EP_BATCH = 40, 256


def ep_shard(device, index, rank, per_rank):
    """The three projections of layer `index` for the experts rank `rank` owns (seeded per layer and rank)."""
    from keep_b200 import moe

    shard = torch.Generator(device=device)
    shard.manual_seed(100_000 + 1000 * index + rank)

    def proj(out, inp):
        codes = torch.randint(0, 1 << 16, (per_rank, out, inp // 8), generator=shard, device=device, dtype=torch.int32).to(torch.uint16)
        scales = (0.02 * (0.5 + torch.rand((per_rank, out, 1), generator=shard, device=device))).to(torch.float16)
        return moe.Projection(codes, scales)

    return proj(INTER, HIDDEN), proj(INTER, HIDDEN), proj(HIDDEN, INTER)


def ep_router(device, index):
    shared = torch.Generator(device=device)
    shared.manual_seed(100 + index)
    return (0.02 * torch.randn((EXPERTS, HIDDEN), generator=shared, device=device)).to(torch.bfloat16)


def build_ep_stack(device, rank, world, layers, exchange_kind="peer"):
    """Config 5: `layers` MoE layers, each with its 384 experts sharded contiguously over the ranks
    and a replicated router (same seed on every rank)."""
    from keep_b200 import expert_parallel, moe

    per_rank = EXPERTS // world
    stack = []
    exchange = None
    if exchange_kind == "peer":  # one set of peer-mapped buffers serves every layer of the stack
        exchange = expert_parallel.PeerExchange(per_rank, tokens=EP_BATCH // world, top_k=TOP_K, hidden=HIDDEN, dtype=torch.bfloat16, device=device)
    for index in range(layers):
        w1, w3, w2 = ep_shard(device, index, rank, per_rank)
        local = moe.RoutedMoELayer(torch.zeros((per_rank, HIDDEN), dtype=torch.bfloat16, device=device), w1, w3, w2, top_k=1)
        stack.append(expert_parallel.ExpertParallelLayer(ep_router(device, index), local, experts_per_rank=per_rank, top_k=TOP_K, exchange=exchange))
    return stack


def ep_parity_gap(stack, x, rank, world, device):
    """Layer 0 through the exchange against the same layer with every expert on one GPU: each rank
    regenerates the other ranks' shards of layer 0 from their seeds, runs the whole layer on the
    tokens of all ranks and compares its own rows.  Returns max|a - b| / max|b| over all ranks."""
    import torch.distributed as dist
    from keep_b200 import moe

    per_rank = EXPERTS // world
    shards = [ep_shard(device, 0, r, per_rank) for r in range(world)]
    cat = lambda k: moe.Projection(torch.cat([s[k].codes.view(torch.int16) for s in shards]).view(torch.uint16), torch.cat([s[k].scales for s in shards]))  # noqa: E731
    whole = moe.RoutedMoELayer(stack[0].router_w, cat(0), cat(1), cat(2), top_k=TOP_K)
    every = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(every, x)
    want = whole.decode(torch.cat(every))[0][rank * x.shape[0]:(rank + 1) * x.shape[0]].float()
    got = stack[0].forward(x).float()
    gap = ((got - want).abs().max() / want.abs().max()).reshape(1)
    dist.all_reduce(gap, op=dist.ReduceOp.MAX)
    del whole, shards
    torch.cuda.empty_cache()
    return float(gap.item())


def between_layers(y):
    """What the model does between two routed layers, reduced to its effect on scale: an RMS norm
    (torch).  Without it the tokens of a random-weight stack shrink layer by layer until every
    router sees zeros and all tokens pick the same six experts."""
    return torch.nn.functional.rms_norm(y, (y.shape[-1],))


def ep_single_gpu_record(device, layers, steps, hbm_gbs):
    """Config 5 on ONE GPU (all 384 experts of every layer local, no exchange): the base of the
    strong-scaling curve.  40 layers x 2.4 GB of codes = 96.6 GB; 256 tokens run through the
    layers one after the other (each layer's output is the next layer's input)."""
    from keep_b200 import moe

    stack = []
    for index in range(layers):
        w1, w3, w2 = ep_shard(device, index, 0, EXPERTS)
        stack.append(moe.RoutedMoELayer(ep_router(device, index), w1, w3, w2, top_k=TOP_K))
    gen = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn((EP_BATCH, HIDDEN), generator=gen).to(torch.bfloat16).to(device)

    def step(_):
        h = x
        for layer in stack:
            h = between_layers(layer.decode(h)[0])

    ms = time_graph(step, steps, 3, replays=5)
    layer_us = ms / steps / layers * 1e3
    touched = statistics.fmean(int(torch.unique(layer._buffers_for(EP_BATCH, torch.bfloat16, 0)["routing"].served_expert).numel()) for layer in stack)
    record = {"layers": layers, "batch": EP_BATCH, "layer_us": round(layer_us, 1), "tokens_x_layers_per_s": round(EP_BATCH * layers * steps / (ms * 1e-3), 1),
              "distinct_experts_per_layer": round(touched, 1),
              "code_frac_of_hbm": round(touched * CODE_BYTES_PER_EXPERT / (layer_us * 1e-6) / 1e9 / hbm_gbs, 4)}
    del stack
    torch.cuda.empty_cache()
    return record


def ep_n1_path():
    import tempfile

    return Path(tempfile.gettempdir()) / "keep_b200_ep_n1.json"


def run_expert_parallel(ns, rank, world, local, device):
    """N > 1: the 40-layer expert-parallel stack (config 5).  256 decode tokens in total, split
    evenly over the ranks; per layer: router, dispatch all-to-all, local experts, combine
    all-to-all.  Each layer's output (RMS-normalised) is the next layer's input, so the stack
    is 40 dependent layer passes per step."""
    import torch.distributed as dist
    from keep_b200 import _lib

    _lib.load()
    hbm_gbs, peak_kind = measured_peaks()
    layers = ns.layers
    stack = build_ep_stack(device, rank, world, layers, ns.exchange)
    tokens_local = EP_BATCH // world
    gen = torch.Generator(device="cpu")
    gen.manual_seed(5 + rank)
    host_in = torch.randn((tokens_local, HIDDEN), generator=gen).to(torch.bfloat16).pin_memory()
    x = host_in.to(device)
    outs = [None]

    def step():
        h = x
        for layer in stack:  # each layer's output, RMS-normalised, is the next layer's input
            h = between_layers(layer.forward(h))
        outs[0] = h

    torch.cuda.synchronize()
    dist.barrier()  # the ranks finish generating their layers at different times; the first exchange meets on the device
    parity_gap = ep_parity_gap(stack, x, rank, world, device)
    if parity_gap > 1e-2:
        raise RuntimeError(f"the expert-parallel layer differs from the single-GPU layer by {parity_gap}: the timing is invalid")
    for _ in range(max(ns.warmup, 3)):
        step()
    torch.cuda.synchronize()
    graph = None
    if not ns.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    step()
            torch.cuda.synchronize()
            dist.barrier()  # the ranks finish capturing at different times; the first replay meets on the device
            g.replay()
            torch.cuda.synchronize()
            graph = g
        except Exception as exc:  # capture of the collectives refused: fall back to eager launches
            if rank == 0:
                print(f"[bench] CUDA graph capture failed ({type(exc).__name__}: {str(exc)[:300]}); timing eager launches", file=sys.stderr)
            graph = None
    run = graph.replay if graph is not None else step

    dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(ns.steps):
            run()
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end)
        dist.barrier()
        host_out = torch.empty((tokens_local, HIDDEN), dtype=torch.bfloat16).pin_memory()
        begin.record()
        for _ in range(ns.steps):
            x.copy_(host_in, non_blocking=True)
            run()
            host_out.copy_(outs[0], non_blocking=True)
        end.record()
        torch.cuda.synchronize()
        e2e_ms = begin.elapsed_time(end)
    expired = float(stack[0].exchange.wait_expired()) if ns.exchange == "peer" else 0.0
    # BASELINE words config 5 with NCCL all-to-alls: the same local layers behind the NCCL exchange, a few eager steps
    nccl_ms = 0.0
    if ns.exchange == "peer":
        from keep_b200 import expert_parallel

        nccl_stack = [expert_parallel.ExpertParallelLayer(l.router_w, l.local, experts_per_rank=EXPERTS // world, top_k=TOP_K) for l in stack]

        def nccl_step():
            h = x
            for layer in nccl_stack:
                h = between_layers(layer.forward(h))

        for _ in range(2):
            nccl_step()
        torch.cuda.synchronize()
        dist.barrier()
        begin.record()
        for _ in range(3):
            nccl_step()
        end.record()
        torch.cuda.synchronize()
        nccl_ms = begin.elapsed_time(end) / 3
    t = torch.tensor([ms, e2e_ms, expired, nccl_ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, expired, nccl_ms = (float(v) for v in t.cpu())
    if expired:
        raise RuntimeError("a barrier of the peer exchange gave up waiting for a rank: the timing is invalid")
    if rank != 0:
        return
    # the unit is a token through one routed layer, as at N = 1: a step pushes EP_BATCH tokens through `layers` of them
    tokens = EP_BATCH * layers * ns.steps
    layer_s = ms * 1e-3 / ns.steps / layers
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    hbm_gbs = float(peaks.get("hbm_gbs", 6650.0))
    local_experts = EXPERTS // world
    touched = local_experts * (1.0 - (1.0 - 1.0 / EXPERTS) ** (EP_BATCH * TOP_K))  # expected distinct local experts per layer
    # the one-GPU run of this same stack, if an N = 1 run of this benchmark left its record on this machine
    strong = None
    try:
        base = json.loads(ep_n1_path().read_text())
        if base.get("layers") == layers:
            strong = {"n1_layer_us": base["layer_us"], "speedup": round(base["layer_us"] / (ms / ns.steps / layers * 1e3), 3),
                      "efficiency": round(base["layer_us"] / (ms / ns.steps / layers * 1e3) / world, 3)}
    except (OSError, ValueError, KeyError):
        pass
    achieved = touched * CODE_BYTES_PER_EXPERT / layer_s / 1e9
    line = {
        "metric": METRIC, "value": round(tokens / (ms * 1e-3), 1), "unit": UNIT, "n_gpus": world, "steps": ns.steps, "warmup": ns.warmup,
        "ms_per_step": round(ms / ns.steps, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"expert-parallel stack (config 5): {layers} layers x 384 experts sharded {EXPERTS // world} per GPU, top-6, "
                               f"{EP_BATCH} decode tokens in total ({tokens_local} per GPU), " + ("dispatch and combine by peer stores over NVLink with flag barriers" if ns.exchange == "peer" else "NCCL all-to-all dispatch and combine"),
                   "layers": layers, "batch": EP_BATCH, "l2": f"inputs larger than L2: {layers} layers x {EXPERTS // world * CODE_BYTES_PER_EXPERT / 1e9:.1f} GB of codes per GPU",
                   "cuda_graph": graph is not None, "exchange": ns.exchange,
                   "note": "value = tokens x layers / time: a token through one routed layer is the unit, the same as the one-GPU line"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s", "frac": round(achieved / hbm_gbs, 4), "traffic": None,
                     "peak_kind": "measured" if "hbm_gbs" in peaks else "fallback", "per": "GPU, whole layer (router, exchange and experts)",
                     "algorithmic_bytes_per_layer": int(touched * CODE_BYTES_PER_EXPERT)},
        "stack_tokens_per_s": round(EP_BATCH * ns.steps / (ms * 1e-3), 1), "cpu_baseline": None,
        "layer_us": round(ms / ns.steps / layers * 1e3, 1),
        "ep_parity_gap": parity_gap, "ep_parity": "layer 0 through the exchange vs the same layer with all 384 experts on one GPU, max|a-b|/max|b| over all ranks",
        "nccl_layer_us": round(nccl_ms / layers * 1e3, 1) if nccl_ms else None,
        "strong_scaling_vs_n1": strong,
        "e2e": {"value": round(tokens / (e2e_ms * 1e-3), 1), "unit": UNIT, "h2d_bytes_per_step": EP_BATCH * HIDDEN * 2, "d2h_bytes_per_step": EP_BATCH * HIDDEN * 2},
        "gpu_launches": (9 if ns.exchange == "peer" else 10) * layers * ns.steps * world, "kernel_path": stack[0].local.kernel_path, "clocks": clocks.summary(),
    }
    print(json.dumps(line))


def run_ours(ns):
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings: the exchange uses no multicast
        dist.init_process_group("nccl", device_id=device)
        try:
            run_expert_parallel(ns, rank, world, local, device)
        finally:
            dist.destroy_process_group()
        return
    from keep_b200 import _lib
    _lib.load()
    hbm_gbs, peak_kind = measured_peaks()
    layer = build_layer(device, seed=0)
    batch = ns.batch
    xs = token_batches(device, batch, ns.rotation)
    uniq = distinct_experts(layer, xs)

    def step(i):
        layer.decode(xs[i % len(xs)])

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    with ClockSampler(local) as clocks:
        ms, replay_ms = time_graph(step, ns.steps, ns.warmup, every=True)
        barrier()
        # end to end: pinned host tokens in, layer output back to the host, every step
        host_in = [x.cpu().pin_memory() for x in xs]
        host_out = torch.empty((batch, HIDDEN), dtype=torch.bfloat16).pin_memory()
        dev_in = torch.empty((batch, HIDDEN), dtype=torch.bfloat16, device=device)

        def e2e_step(i):
            dev_in.copy_(host_in[i % len(xs)], non_blocking=True)
            out, _ = layer.decode(dev_in)
            host_out.copy_(out, non_blocking=True)

        # The same capture-and-replay as the device-resident number: a serving loop replays one graph
        # per step too, and the copies from and to pinned host memory are nodes of that graph.  The
        # loop is double-buffered the way a server's is: while the layer works on step i, a copy
        # stream brings in the tokens of step i + 1 and another takes the outputs of step i - 1 out.
        # Every step's tokens still come from pinned host memory and every step's output still
        # lands in host memory inside the timed region.
        dev_ins = [torch.empty_like(dev_in) for _ in range(2)]
        dev_outs = [torch.empty_like(dev_in) for _ in range(2)]
        h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
        in_ready = [torch.cuda.Event() for _ in range(2)]
        out_ready = [torch.cuda.Event() for _ in range(2)]
        out_taken = [torch.cuda.Event() for _ in range(2)]

        def e2e_pipelined(i):
            main, k = torch.cuda.current_stream(), i % 2
            if i == 0:  # the first step's tokens: nothing to hide them behind
                h2d.wait_stream(main)
                with torch.cuda.stream(h2d):
                    dev_ins[0].copy_(host_in[0], non_blocking=True)
                    in_ready[0].record(h2d)
            main.wait_event(in_ready[k])
            if i + 1 < ns.steps:  # next step's tokens, behind the previous layer call (the last reader of that buffer)
                h2d.wait_stream(main)
                with torch.cuda.stream(h2d):
                    dev_ins[1 - k].copy_(host_in[(i + 1) % len(xs)], non_blocking=True)
                    in_ready[1 - k].record(h2d)
            if i >= 2:
                main.wait_event(out_taken[k])  # the outputs of step i - 2 have left this buffer
            layer.decode(dev_ins[k], out=dev_outs[k])
            out_ready[k].record(main)
            d2h.wait_event(out_ready[k])
            with torch.cuda.stream(d2h):
                host_out.copy_(dev_outs[k], non_blocking=True)
                out_taken[k].record(d2h)
            if i + 1 == ns.steps:  # join the copy streams
                main.wait_stream(h2d)
                main.wait_stream(d2h)

        e2e_ms = time_graph(e2e_pipelined, ns.steps, ns.warmup, warm_fn=e2e_step)
        e2e_serial_ms = time_graph(e2e_step, ns.steps, ns.warmup)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms, e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = (float(v) for v in t.cpu())
    tokens = batch * ns.steps * world
    value = tokens / (ms * 1e-3)
    e2e_value = tokens / (e2e_ms * 1e-3)
    if rank != 0:
        return
    mean_u = statistics.fmean(uniq[i % len(xs)] for i in range(ns.steps))
    code_gbs = mean_u * CODE_BYTES_PER_EXPERT / (ms / ns.steps * 1e-3) / 1e9
    roofline = projection_roofline(layer, xs, ns.steps, hbm_gbs, peak_kind)
    threads = os.cpu_count() or 1
    cpu_layer_sample(layer, xs[1 % len(xs)][:1].cpu(), threads, 1)  # warm: the first call builds the 65,536-entry decode grid
    cpu_s, cpu_out = cpu_layer_sample(layer, xs[0][:1].cpu(), threads)
    gpu_out, _ = layer.decode(xs[0])
    ref = cpu_out.numpy()
    parity_gap = float(np.abs(gpu_out[:1].float().cpu().numpy() - ref).max() / np.abs(ref).max())
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": ns.steps, "warmup": ns.warmup,
        "ms_per_step": round(ms / ns.steps, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"decode layer (config 2): 384 experts, hidden 4096, inter 2048, top-6 softmax router, batch {batch}",
                   "batch": batch, "l2": "inputs larger than L2: 64 rotating token batches over a 2.4 GB expert pool",
                   "distinct_experts_per_step": round(mean_u, 2),
                   "timing": f"one CUDA graph of {ns.steps} steps, replayed {REPLAYS} times after an untimed replay; ms_per_step and value are the median replay"},
        "replays": REPLAYS, "replay_ms": [round(v, 4) for v in replay_ms], "timed_region_s": round(sum(replay_ms) * 1e-3, 4),
        "layer_code_gbs": round(code_gbs, 1), "layer_code_frac_of_hbm": round(code_gbs / hbm_gbs, 4),
        "roofline": roofline, "stage_us": stage_times(layer, xs, ns.steps),
        "cpu_baseline": {"value": round(1.0 / cpu_s, 4), "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "one token (after one warm-up token): router + decode of 6 experts x 3 projections + SwiGLU path", "parity_gap_vs_gpu": parity_gap},
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": batch * HIDDEN * 2, "d2h_bytes_per_step": batch * HIDDEN * 2,
                "how": "double-buffered: the copies of steps i + 1 (in) and i - 1 (out) run on copy streams beside the layer call of step i",
                "serial_value": round(tokens / (e2e_serial_ms * 1e-3), 1)},
        "batch_sweep": batch_sweep(layer, device, ns.rotation, ns.steps, hbm_gbs) if not ns.no_prefill else None,
        "residency": residency_leg(layer, device, ns.rotation, ns.steps, hbm_gbs) if not ns.no_prefill else None,
        "prefill": prefill_leg(layer, device) if not ns.no_prefill else None,
        "operators": operator_legs(layer, device, hbm_gbs) if not ns.no_prefill else None,
        "artifact_shape": artifact_shape_leg(device, hbm_gbs) if not ns.no_prefill else None,
        "ep_n1": None,
        "gpu_launches": layer.launches_per_call(batch) * ns.steps, "kernel_path": layer.kernel_path,
        "clocks": clocks.summary(),
    }
    if not ns.no_prefill and not ns.no_ep_base:  # config 5 on this one GPU: the base the N > 1 lines compare their layer time with
        torch.cuda.empty_cache()
        line["ep_n1"] = ep_single_gpu_record(device, ns.layers, 4, hbm_gbs)
        try:
            ep_n1_path().write_text(json.dumps(line["ep_n1"]))
        except OSError:
            pass
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--rotation", type=int, default=ROTATION, help="distinct token batches to rotate over (profiling runs use fewer)")
    ap.add_argument("--layers", type=int, default=EP_LAYERS, help="layers of the expert-parallel stack (N > 1)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="expert-parallel run: how routes travel between the GPUs")
    ap.add_argument("--no-graph", action="store_true", help="expert-parallel run: time eager launches instead of a CUDA graph")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 4096-token prefill leg (config 3) and the batch sweep")
    ap.add_argument("--no-ep-base", action="store_true", help="skip the one-GPU run of the 40-layer expert-parallel stack (96.6 GB of codes; profiling runs skip it)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ns = ap.parse_args()
    if ns.impl == "reference":
        run_reference(ns)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
        run_ours(ns)


if __name__ == "__main__":
    main()
