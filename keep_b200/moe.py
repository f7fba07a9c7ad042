"""One routed MoE layer over E8P experts: the fused decode step.

``RoutedMoELayer.decode(x)`` is the call a serving loop makes per layer.  It stands in for the
reference's decode step (``scripts/v41_build/omlx_lattice.py:327-371``: stock gate -> fused top-k
-> ``e8p_m1`` / ``e8p_nested_m1`` gate, up, down -> sum over the picks) and, without a residency
mask, for ``QuantizedVQSwitchGLU`` plus the weighted sum
(``src/ramp/models/glm4_moe_adapter.py:367-372``, ``deepseek_v4_flash_adapter.py:1781-1784``).
Everything runs in ``keepvq_moe_decode_layer``: one launch sequence, no host read.

``SharedExpert`` is the dense shared expert next to it (``deepseek_v4_flash_adapter.py:1733-1784``):
its fp32 output goes into ``decode(x, shared=...)``, where the pick sum adds it before the one
rounding (the reference's shared down kernel adds the routed sum and rounds once,
``scripts/v41_build/omlx_lattice.py:372-389``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from .router import Routing
from .vq import as_device, table_on


@dataclass
class Projection:
    """Codes ``[slots, out, in/8]`` uint16 and scales ``[slots, out, groups]`` of one projection,
    plus the optional 8-bit residual arrays ``[res_rows, out, in/8]`` / ``[res_rows, out, res_groups]``."""

    codes: torch.Tensor
    scales: torch.Tensor
    res_codes: torch.Tensor | None = None
    res_scales: torch.Tensor | None = None

    def struct(self) -> _lib.ExpertWeights:
        return _lib.ExpertWeights(
            codes=_lib.ptr(self.codes), scales=_lib.ptr(self.scales), groups=int(self.scales.shape[2]),
            res_codes=_lib.ptr(self.res_codes), res_scales=_lib.ptr(self.res_scales),
            res_groups=int(self.res_scales.shape[2]) if self.res_scales is not None else 0)


class SharedExpert:
    """The dense shared expert of a layer: ``w2 (silu(w1 x) * (w3 x))`` with the same clamp as the
    routed experts (``deepseek_v4_flash_adapter.py:963-967,1733-1737``), returned in fp32 and NOT
    rounded, for ``RoutedMoELayer.decode(x, shared=...)`` to add to the routed sum.

    ``w1`` (gate), ``w3`` (up): ``[inter, hidden]``; ``w2`` (down): ``[hidden, inter]``, fp16 or
    bf16.  The three products are plain library GEMMs with fp32 accumulation; gate and up run as one
    GEMM over the stacked weights.  The reference's shared expert runs on oMLX's MXFP4 / MXFP8 /
    affine kernels, a third-party package that is not part of it: a caller holding such weights
    expands them to 16 bits first, and no parity with those kernels is claimed.
    """

    def __init__(self, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor, *, swiglu_limit: float = 0.0):
        self.device = _lib.require_cuda(w1, w3, w2)
        if w1.dtype not in (torch.float16, torch.bfloat16) or w3.dtype != w1.dtype or w2.dtype != w1.dtype:
            raise ValueError("shared expert weights must share one of fp16 / bf16")
        self.inter, self.hidden = (int(v) for v in w1.shape)
        if tuple(w3.shape) != tuple(w1.shape) or tuple(w2.shape) != (self.hidden, self.inter):
            raise ValueError("w1/w3 must be [inter, hidden] and w2 [hidden, inter]")
        self.gate_up = torch.cat([w1, w3], 0).t().contiguous()  # [hidden, 2 inter]
        self.down = w2.t().contiguous()                          # [inter, hidden]
        self.swiglu_limit = float(swiglu_limit)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` [tokens, hidden] in the weights' dtype -> fp32 ``[tokens, hidden]``."""
        if x.ndim != 2 or int(x.shape[1]) != self.hidden or x.dtype != self.down.dtype:
            raise ValueError(f"x must be [tokens, {self.hidden}] {self.down.dtype}, found {tuple(x.shape)} {x.dtype}")
        gate, up = torch.mm(x, self.gate_up, out_dtype=torch.float32).split(self.inter, dim=1)
        if self.swiglu_limit > 0:
            gate, up = gate.clamp(max=self.swiglu_limit), up.clamp(-self.swiglu_limit, self.swiglu_limit)
        h = (torch.nn.functional.silu(gate) * up).to(x.dtype)   # the hidden row in 16 bits, as the routed experts keep theirs
        return torch.mm(h, self.down, out_dtype=torch.float32)


class RoutedMoELayer:
    """Router + resident experts of one layer.

    ``w1`` (gate), ``w3`` (up): ``[slots, inter, hidden/8]``; ``w2`` (down): ``[slots, hidden, inter/8]``.
    Residency state is three device arrays the caller may rewrite between calls: ``served_bias``
    ``[pool]`` (``router.OFF`` on absent experts), ``slot_of`` ``[pool]`` and, with a residual tier,
    ``hot_of_slot`` ``[slots]``.  With ``served_bias=None`` every expert is resident and
    ``slot_of`` is the identity.
    """

    def __init__(self, router_w, w1: Projection, w3: Projection, w2: Projection, *, top_k: int, score_func: str = "softmax",
                 route_scale: float = 1.0, tau: float = 0.3, gate_temp: float = 1.0, norm_topk_prob: bool = True,
                 served_bias=None, pool_bias=None, slot_of=None, hot_of_slot=None, res_table=None, codebook=None,
                 swiglu_limit: float = 0.0):
        if score_func not in _lib.SCORE_FUNCS:
            raise ValueError("score_func must be 'softmax', 'sigmoid' or 'sqrtsoftplus'")
        self.device = _lib.require_cuda(router_w, w1.codes, w3.codes, w2.codes)
        self.router_w = router_w.contiguous()
        self.w1, self.w3, self.w2 = w1, w3, w2
        for p in (w1, w3, w2):
            if p.codes.dtype != torch.uint16:
                raise ValueError(f"expert codes must be uint16, found {p.codes.dtype}")
            if p.scales.dtype != w1.scales.dtype:
                raise ValueError("all scales must share one dtype")
        self.slots, self.inter, cw = (int(s) for s in w1.codes.shape)
        self.hidden, self.pool = cw * 8, int(router_w.shape[0])
        if tuple(w3.codes.shape) != tuple(w1.codes.shape) or tuple(w2.codes.shape) != (self.slots, self.hidden, self.inter // 8):
            raise ValueError("w1/w3 must be [slots, inter, hidden/8] and w2 [slots, hidden, inter/8]")
        if int(router_w.shape[1]) != self.hidden:
            raise ValueError("router_w must be [pool, hidden]")
        self.top_k, self.score_func = int(top_k), score_func
        self.route_scale, self.tau, self.gate_temp = float(route_scale), float(tau), float(gate_temp)
        self.norm_topk_prob, self.swiglu_limit = bool(norm_topk_prob), float(swiglu_limit)
        f32 = lambda t: None if t is None else as_device(t, self.device).to(torch.float32).contiguous()  # noqa: E731
        u32 = lambda t: None if t is None else as_device(t, self.device).contiguous()  # noqa: E731
        self.served_bias, self.pool_bias = f32(served_bias), f32(pool_bias)
        self.slot_of, self.hot_of_slot = u32(slot_of), u32(hot_of_slot)
        if self.served_bias is None and self.slot_of is None and self.slots != self.pool:
            raise ValueError("with every expert resident, codes must hold one slot per pool expert")
        self.codebook = table_on(self.device, "e8p") if codebook is None else as_device(codebook, self.device).contiguous()
        # The int8 tensor-core kernels need every table nibble odd (odd half-unit magnitudes).  The
        # E8P table is; a custom table is read back once, here, never on the token path.
        nibbles = (self.codebook.cpu().to(torch.int64) & 0xFFFFFFFF)[:, None] >> (4 * torch.arange(8))[None] & 1
        self.codebook_all_odd = bool(nibbles.all())
        self.res_rows = int(w1.res_codes.shape[0]) if w1.res_codes is not None else 0
        self.res_table = None
        if self.res_rows:
            if self.hot_of_slot is None:
                raise ValueError("a residual tier needs hot_of_slot")
            self.res_table = table_on(self.device, "e8_1bit_half2") if res_table is None else as_device(res_table, self.device).contiguous()
        self._buffers: dict[tuple, dict] = {}

    def _buffers_for(self, tokens: int, dtype: torch.dtype, state: int = 0) -> dict:
        key = (tokens, dtype, state)
        if key not in self._buffers:
            lib = _lib.load()
            nbytes = int(lib.keepvq_moe_layer_workspace_bytes(tokens, self.hidden, self.inter, self.pool, self.top_k))
            if nbytes < 0:
                _lib.check(nbytes, "keepvq_moe_layer_workspace_bytes")
            dev, k = self.device, self.top_k
            i32 = lambda: torch.empty((tokens, k), dtype=torch.int32, device=dev)  # noqa: E731
            f32 = lambda: torch.empty((tokens, k), dtype=torch.float32, device=dev)  # noqa: E731
            self._buffers[key] = dict(
                workspace=torch.empty(nbytes, dtype=torch.uint8, device=dev), nbytes=nbytes,
                out=torch.empty((tokens, self.hidden), dtype=dtype, device=dev),
                routing=Routing(served_expert=i32(), served_slot=i32(), served_weight=f32(), want=i32(), want_score=f32(), admit=i32()))
        return self._buffers[key]

    def _layer_args(self, x, out, r: Routing, *, workspace, nbytes, expected_routes: int = 0, shared=None) -> _lib.MoELayerArgs:
        """The argument struct of a layer call over the caller's tensors."""
        return _lib.MoELayerArgs(
            x=_lib.ptr(x), x_dtype=_lib.dtype_tag(x.dtype), tokens=int(x.shape[0]), hidden=self.hidden, inter=self.inter,
            router_w=_lib.ptr(self.router_w), router_dtype=_lib.dtype_tag(self.router_w.dtype), pool=self.pool,
            top_k=self.top_k, score_func=_lib.SCORE_FUNCS[self.score_func], norm_topk_prob=int(self.norm_topk_prob),
            gate_temp=self.gate_temp, route_scale=self.route_scale, tau=self.tau,
            served_bias=_lib.ptr(self.served_bias), pool_bias=_lib.ptr(self.pool_bias), slot_of=_lib.ptr(self.slot_of),
            slots=self.slots, w1=self.w1.struct(), w3=self.w3.struct(), w2=self.w2.struct(),
            scales_dtype=_lib.dtype_tag(self.w1.scales.dtype), codebook=_lib.ptr(self.codebook), res_rows=self.res_rows,
            res_table=_lib.ptr(self.res_table), hot_of_slot=_lib.ptr(self.hot_of_slot), swiglu_limit=self.swiglu_limit,
            codebook_all_odd=int(self.codebook_all_odd),
            out=_lib.ptr(out), served_expert=_lib.ptr(r.served_expert), served_slot=_lib.ptr(r.served_slot),
            served_weight=_lib.ptr(r.served_weight), want=_lib.ptr(r.want), want_score=_lib.ptr(r.want_score),
            admit=_lib.ptr(r.admit), workspace=_lib.ptr(workspace), workspace_bytes=nbytes, expected_routes=int(expected_routes),
            shared=_lib.ptr(shared))

    def _scratch_rows(self, which: str, width: int, tokens: int, dtype: torch.dtype, state: int) -> torch.Tensor:
        buf = self._buffers_for(tokens, dtype, state)
        offset = int(getattr(_lib.load(), which)(tokens, self.hidden, self.inter, self.pool, self.top_k))
        if offset < 0:
            _lib.check(offset, which)
        base = (-buf["workspace"].data_ptr()) % 256  # the library aligns the scratch to 256 bytes
        nbytes = tokens * self.top_k * width * dtype.itemsize
        return buf["workspace"][base + offset: base + offset + nbytes].view(dtype).view(tokens * self.top_k, width)

    def route_outputs(self, tokens: int, dtype: torch.dtype, state: int = 0) -> torch.Tensor:
        """The per-route outputs ``[tokens * top_k, hidden]`` the last call of this shape left in its
        scratch (the rows the pick sum adds up): a view, overwritten by the next call."""
        return self._scratch_rows("keepvq_moe_layer_route_output_offset", self.hidden, tokens, dtype, state)

    def route_hidden(self, tokens: int, dtype: torch.dtype, state: int = 0) -> torch.Tensor:
        """The routes' hidden rows ``h = silu(G) * U * weight``, ``[tokens * top_k, inter]``, that
        the gate/up stage of the last call of this shape left for the down stage: a view."""
        return self._scratch_rows("keepvq_moe_layer_route_hidden_offset", self.inter, tokens, dtype, state)

    def wait_expired(self, tokens: int, dtype: torch.dtype, state: int = 0) -> bool:
        """True when a bounded wait of the tcgen05 kernels expired during the last call of this
        shape (its outputs are then invalid).  Reads one word back: synchronises the stream."""
        buf = self._buffers_for(tokens, dtype, state)
        offset = int(_lib.load().keepvq_moe_layer_status_offset(tokens, self.hidden, self.inter, self.pool, self.top_k))
        if offset < 0:
            _lib.check(offset, "keepvq_moe_layer_status_offset")
        base = (-buf["workspace"].data_ptr()) % 256  # the library aligns the scratch to 256 bytes
        return bool(buf["workspace"][base + offset: base + offset + 4].view(torch.int32).item())

    @property
    def kernel_path(self) -> str:
        """``"tensor"`` when calls run on the int8 tensor-core kernels, else ``"general"``.  With a
        residual tier the inputs may be at most 6144 wide (the residual pass lives in the slab
        kernels, whose split form for small calls keeps 48 KB of activations in shared memory);
        wider layers with a residual tier run the general kernels."""
        ok = lambda inp, groups: inp % 256 == 0 and (inp // 256) % groups == 0  # noqa: E731
        fits = ok(self.hidden, int(self.w1.scales.shape[2])) and ok(self.inter, int(self.w2.scales.shape[2]))
        if self.res_rows:
            tiers = (self.w1, self.w3, self.w2)
            fits = fits and all(p.res_codes is not None for p in tiers) and self.hidden <= 6144 and self.inter <= 6144 \
                and ok(self.hidden, int(self.w1.res_scales.shape[2])) and ok(self.inter, int(self.w2.res_scales.shape[2]))
        return "tensor" if self.codebook_all_odd and fits else "general"

    def launches_per_call(self, tokens: int, dtype: torch.dtype = torch.bfloat16) -> int:
        """Kernel launches one ``decode`` call of ``tokens`` rows enqueues.  On the tensor-core
        kernels: logits, top-k, route grouping, quantise x, gate/up, quantise h, down, combine,
        of which two share a launch: up to 23 fp16 / bf16 tokens the logits and the quantisation
        of x, beyond that (up to 4096 routes) the quantisation of x and the route grouping."""
        if self.kernel_path != "tensor":
            return 7
        front = tokens <= 23 and dtype in (torch.float16, torch.bfloat16)
        paired = tokens * self.top_k <= 4096 and self.slots * 12 <= 40 * 1024
        return 7 if front or paired else 8

    def decode_without_scratch(self, x: torch.Tensor, out: torch.Tensor, routing: Routing) -> tuple[torch.Tensor, Routing]:
        """The same layer through ``keepvq_moe_decode_layer_static``: the caller supplies the
        output and routing tensors, and the scratch is the fixed array inside the library, so the
        call allocates nothing anywhere.  For hosts that cannot allocate device memory at call
        time (all of it already belongs to their own pool) or may not stall on an allocation.

        Limits: the scratch holds ``_lib.STATIC_SCRATCH_BYTES`` (8 MiB; about 16 tokens at hidden
        4096, inter 2048, top-6) and a larger request raises ``KeepVQError`` (capacity).  Every
        call on a device shares that one array: calls that overlap on the GPU race on it, so keep
        them on one stream.  The first call on a device sets the array up and should come before
        any stream capture.
        """
        _lib.require_cuda(x, out)
        if x.ndim != 2 or int(x.shape[1]) != self.hidden or not x.is_contiguous():
            raise ValueError(f"x must be a contiguous [tokens, {self.hidden}] tensor, found {tuple(x.shape)}")
        if tuple(out.shape) != tuple(x.shape) or out.dtype != x.dtype or not out.is_contiguous():
            raise ValueError("out must be a contiguous tensor of x's shape and dtype")
        args = self._layer_args(x, out, routing, workspace=None, nbytes=0)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().keepvq_moe_decode_layer_static(args, _lib.stream_handle(self.device)),
                       "keepvq_moe_decode_layer_static")
        return out, routing

    def decode(self, x: torch.Tensor, *, out: torch.Tensor | None = None, stages: int = _lib.STAGE_ALL,
               state: int = 0, expected_routes: int = 0, shared: torch.Tensor | None = None) -> tuple[torch.Tensor, Routing]:
        """``x`` [tokens, hidden] -> (``[tokens, hidden]`` in x's dtype, routing outputs).

        Buffers are cached per (tokens, dtype) and reused by the next call of the same shape, so
        the call is CUDA-graph capturable after one warm-up call; copy results you want to keep.
        ``stages`` (a mask of ``_lib.STAGE_*``) replays part of the sequence on the state a full
        call left behind; profilers and the benchmark use it.  ``state`` picks one of several
        independent buffer sets (each keeps its own scratch and outputs).  ``expected_routes`` (0 =
        all) tells the library how many of the ``tokens * top_k`` routes the caller expects to be
        live, which only picks the kernel family.  ``shared`` (fp32 ``[tokens, hidden]``, e.g. a
        ``SharedExpert``'s output) is added to the routed sum before the one rounding.
        """
        _lib.require_cuda(x)
        if x.ndim != 2 or int(x.shape[1]) != self.hidden:
            raise ValueError(f"x must be [tokens, {self.hidden}], found {tuple(x.shape)}")
        x = x.contiguous()
        tokens = int(x.shape[0])
        if shared is not None:
            _lib.require_cuda(shared)
            if shared.dtype != torch.float32 or tuple(shared.shape) != (tokens, self.hidden) or not shared.is_contiguous():
                raise ValueError(f"shared must be a contiguous fp32 [{tokens}, {self.hidden}] tensor")
        buf = self._buffers_for(tokens, x.dtype, state)
        r: Routing = buf["routing"]
        target = buf["out"] if out is None else out
        args = self._layer_args(x, target, r, workspace=buf["workspace"], nbytes=buf["nbytes"], expected_routes=expected_routes, shared=shared)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().keepvq_moe_decode_stages(args, int(stages), _lib.stream_handle(self.device)), "keepvq_moe_decode_stages")
        return target, r
