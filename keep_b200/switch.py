"""Holders for stacked VQ experts: one switch projection, and the gate/up/down trio of a routed MLP.

Mirrors of ``QuantizedVQSwitchLinear`` (``src/ramp/nn/switch_linear.py:93-571``) and
``QuantizedVQSwitchGLU`` (``src/ramp/models/glm4_moe_adapter.py:113-390``) over ``torch.Tensor``
on a CUDA device: the same constructor keywords, shape rules, error messages and call layouts.

What they hold is the hot path only: codes, scales, codebook, optional bias and the continuous
scale / output-bias sidecars.  The reference's other sidecars (low-rank and sparse residual rows,
RHT signs, rotation matrices) and ``from_weights`` (the RTN encoder) belong to conversion and
quality tooling; passing one raises ``NotImplementedError`` rather than being ignored.
"""

from __future__ import annotations

from typing import Callable

import torch

from . import _lib
from .kernels import e8p_m1_per_route, e8p_m1_token_layout, should_use_e8p_m1
from .vq import table_on
from .vq_switch import gather_vqmm, vq_switch_qmv

_ROUTE_STRATEGIES = ("auto", "direct", "sorted_tiled", "per_route_decoded")
_OUTSIDE = ("continuous_low_rank_left", "continuous_low_rank_right", "sparse_residual_expert_indices",
            "sparse_residual_output_indices", "sparse_residual_values", "rht_signs", "rotation_matrix")


class QuantizedVQSwitchLinear:
    """Switch-linear layer backed by stacked E8 VQ expert tensors.

    ``x [..., in]`` with ``indices [..., k]`` (token layout) gives ``[..., k, out]``; ``x [..., k, in]``
    with ``indices [..., k]`` (one row per route) gives the same shape.
    """

    def __init__(self, *, input_dims: int, output_dims: int, num_experts: int, codes: torch.Tensor, scales: torch.Tensor,
                 codebook: torch.Tensor | None = None, bias: torch.Tensor | None = None, group_size: int = 512,
                 code_bits: int = 8, use_gather_vqmm: bool = True, route_strategy: str = "auto",
                 gather_codebook_duplication: int = 8, continuous_scale_delta: torch.Tensor | None = None,
                 continuous_output_bias: torch.Tensor | None = None, **outside):
        for name, value in outside.items():
            if name not in _OUTSIDE:
                raise TypeError(f"unexpected keyword argument {name!r}")
            if value is not None:
                raise NotImplementedError(f"{name} belongs to the conversion tooling, not to the routed hot path")
        if input_dims <= 0 or output_dims <= 0 or num_experts <= 0:
            raise ValueError("input_dims, output_dims, and num_experts must be positive")
        if input_dims % 8 != 0:
            raise ValueError("input_dims must be divisible by 8")
        if input_dims % group_size != 0:
            raise ValueError("input_dims must be divisible by group_size")
        if code_bits not in (8, 16):
            raise ValueError("code_bits must be 8 or 16")
        if gather_codebook_duplication not in (1, 4, 8):
            raise ValueError("gather_codebook_duplication must be 1, 4, or 8")
        if route_strategy not in _ROUTE_STRATEGIES:
            raise ValueError("route_strategy must be 'auto', 'direct', 'sorted_tiled', or 'per_route_decoded'")
        expected_codes = (num_experts, output_dims, input_dims // 8)
        if tuple(codes.shape) != expected_codes:
            raise ValueError(f"codes must have shape {expected_codes}, found {tuple(codes.shape)}")
        expected_scales = (num_experts, output_dims, input_dims // group_size)
        if tuple(scales.shape) != expected_scales:
            raise ValueError(f"scales must have shape {expected_scales}, found {tuple(scales.shape)}")
        if bias is not None and tuple(bias.shape) != (num_experts, output_dims):
            raise ValueError(f"bias must have shape {(num_experts, output_dims)}, found {tuple(bias.shape)}")
        _lib.require_cuda(codes, scales)
        self.input_dims, self.output_dims, self.num_experts = int(input_dims), int(output_dims), int(num_experts)
        self.group_size, self.code_bits = int(group_size), int(code_bits)
        self.use_gather_vqmm, self.route_strategy = bool(use_gather_vqmm), route_strategy
        self.gather_codebook_duplication = int(gather_codebook_duplication)
        if codebook is None:  # the default table of the code width, as the reference's holder resolves it
            codebook = table_on(codes.device, "e8p" if code_bits == 16 else "e8_1bit")
        self.codes, self.scales, self.codebook, self.bias = codes, scales, codebook, bias
        self.continuous_scale_delta = None if continuous_scale_delta is None else continuous_scale_delta.float()
        self.continuous_output_bias = None if continuous_output_bias is None else continuous_output_bias.float()

    @property
    def route_backend(self) -> str:
        return f"gather_vqmm_{self.route_strategy}" if self.use_gather_vqmm else "scalar_qmv"

    @property
    def has_continuous_sidecar(self) -> bool:
        return self.continuous_scale_delta is not None or self.continuous_output_bias is not None

    @property
    def has_sparse_residual_rows(self) -> bool:
        return False

    def effective_scales(self) -> torch.Tensor:
        """``scales * exp(continuous_scale_delta)`` in fp32 when the sidecar is set (``switch_linear.py:282-286``)."""
        if self.continuous_scale_delta is None:
            return self.scales
        return self.scales.float() * torch.exp(self.continuous_scale_delta)

    def __call__(self, x: torch.Tensor, indices: torch.Tensor, *, sorted_indices: bool = False) -> torch.Tensor:
        scales = self.effective_scales()
        common = dict(input_dims=self.input_dims, output_dims=self.output_dims, group_size=self.group_size, code_bits=self.code_bits)
        token_layout = x.ndim >= 2 and indices.ndim >= 2 and tuple(x.shape[:-1]) == tuple(indices.shape[:-1])
        per_route = x.ndim >= 2 and indices.ndim >= 1 and tuple(x.shape[:-1]) == tuple(indices.shape)
        if self.use_gather_vqmm and token_layout:
            top_k = int(indices.shape[-1])
            flat_x, flat_idx = x.reshape(-1, self.input_dims), indices.reshape(-1, top_k)
            few = should_use_e8p_m1(code_bits=self.code_bits, tokens=int(flat_x.shape[0]), sorted_indices=sorted_indices,
                                    route_strategy=self.route_strategy)
            if few:
                y = e8p_m1_token_layout(flat_x, self.codes, scales, self.codebook, flat_idx, output_dims=self.output_dims)
            else:
                y = gather_vqmm(flat_x, self.codes, scales, self.codebook, flat_idx, sorted_indices=sorted_indices,
                                route_strategy=self.route_strategy, codebook_duplication=self.gather_codebook_duplication, **common)
            y = y.reshape(tuple(indices.shape) + (self.output_dims,))
        elif self.use_gather_vqmm and per_route:
            flat_x, flat_idx = x.reshape(-1, self.input_dims), indices.reshape(-1)
            tokens = int(flat_idx.numel()) // int(indices.shape[-1]) if indices.ndim >= 2 else int(flat_idx.numel())
            few = indices.ndim >= 2 and should_use_e8p_m1(code_bits=self.code_bits, tokens=tokens, sorted_indices=sorted_indices,
                                                          route_strategy=self.route_strategy)
            if few:
                y = e8p_m1_per_route(flat_x, self.codes, scales, self.codebook, flat_idx, output_dims=self.output_dims)
            else:
                rows = torch.arange(int(flat_idx.numel()), device=flat_x.device, dtype=torch.int32)
                y = gather_vqmm(flat_x, self.codes, scales, self.codebook, flat_idx, lhs_indices=rows, sorted_indices=sorted_indices,
                                route_strategy=self.route_strategy, codebook_duplication=self.gather_codebook_duplication, **common)
            y = y.reshape(tuple(indices.shape) + (self.output_dims,))
        else:
            y = vq_switch_qmv(x, self.codes, scales, self.codebook, indices, **common)
        gather = indices.long().clamp(min=0)
        if self.bias is not None:
            y = y + self.bias[gather].to(y.dtype)
        if self.continuous_output_bias is not None:
            y = y + self.continuous_output_bias[gather].to(y.dtype)
        return y


def limited_swiglu(limit: float) -> Callable[[torch.Tensor, torch.Tensor], torch.Tensor]:
    """The activation of ``LimitedSwiGLU`` (``deepseek_v4_flash_adapter.py:963-967``) as an
    ``activation(up, gate)`` hook; the fused kernels recognise it by its ``limit`` attribute."""
    def act(up: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        if limit and limit > 0:
            gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
        return torch.nn.functional.silu(gate) * up

    act.limit = float(limit)
    return act


class QuantizedVQSwitchGLU:
    """``down(act(up(x), gate(x)))`` per route: ``x [tokens, hidden]``, ``indices [tokens, k]`` ->
    ``[tokens, k, hidden]`` (``glm4_moe_adapter.py:367-372``).

    With 16-bit E8P codes, no bias or sidecars and plain or limited SwiGLU, a call runs the fused
    layer kernels (activation quantisation, gate + up + SwiGLU in one launch, down in another);
    any other configuration composes the three projections as the reference does.
    """

    def __init__(self, *, gate_proj: QuantizedVQSwitchLinear, up_proj: QuantizedVQSwitchLinear, down_proj: QuantizedVQSwitchLinear,
                 prefill_engine: str = "auto", activation: Callable[[torch.Tensor, torch.Tensor], torch.Tensor] | None = None):
        if gate_proj.input_dims != up_proj.input_dims:
            raise ValueError("gate_proj and up_proj input dimensions must match")
        if gate_proj.output_dims != up_proj.output_dims:
            raise ValueError("gate_proj and up_proj output dimensions must match")
        if down_proj.input_dims != gate_proj.output_dims:
            raise ValueError("down_proj input dimension must match routed hidden dimension")
        if down_proj.output_dims != gate_proj.input_dims:
            raise ValueError("down_proj output dimension must match model hidden dimension")
        if len({gate_proj.num_experts, up_proj.num_experts, down_proj.num_experts}) != 1:
            raise ValueError("all switch projections must have the same expert count")
        if prefill_engine not in ("auto", "vq_metal", "nax_e8", "nax_e8p"):
            raise ValueError("prefill_engine must be 'auto', 'vq_metal', 'nax_e8', or 'nax_e8p'")
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
        self.prefill_engine, self.activation = prefill_engine, activation
        self._fused: dict = {}

    def _apply_activation(self, up: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        if self.activation is None:
            return torch.nn.functional.silu(gate) * up
        return self.activation(up, gate)

    def _fused_layer(self, top_k: int):
        """The three projections as one ``RoutedMoELayer`` with ``top_k`` picks per token (its
        router unused), or None when the configuration does not fit the layer kernels."""
        if top_k not in self._fused:
            from .moe import Projection, RoutedMoELayer

            projs = (self.gate_proj, self.up_proj, self.down_proj)
            plain = all(p.code_bits == 16 and p.bias is None and not p.has_continuous_sidecar and p.use_gather_vqmm for p in projs)
            act_ok = self.activation is None or hasattr(self.activation, "limit")
            same_book = all(p.codebook is self.gate_proj.codebook or (p.codebook is not None and self.gate_proj.codebook is not None
                                                                     and torch.equal(p.codebook, self.gate_proj.codebook)) for p in projs)
            self._fused[top_k] = None
            if plain and act_ok and same_book:
                g = self.gate_proj
                layer = RoutedMoELayer(torch.zeros((g.num_experts, g.input_dims), dtype=torch.bfloat16, device=g.codes.device),
                                       Projection(g.codes, g.scales), Projection(self.up_proj.codes, self.up_proj.scales),
                                       Projection(self.down_proj.codes, self.down_proj.scales), top_k=top_k, codebook=g.codebook,
                                       swiglu_limit=float(getattr(self.activation, "limit", 0.0)))
                if layer.kernel_path == "tensor":
                    self._fused[top_k] = layer
        return self._fused[top_k]

    def __call__(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        fits = x.ndim == 2 and indices.ndim == 2 and x.shape[0] == indices.shape[0] and x.dtype in (torch.bfloat16, torch.float16)
        layer = self._fused_layer(int(indices.shape[1])) if fits else None
        if layer is not None:
            # token layout straight through the layer kernels: route t * k + j reads activation row t
            # (no copy of x per pick); the stages stop before the pick sum and the per-route rows
            # are what this operator returns
            tokens, k = indices.shape
            r = layer._buffers_for(tokens, x.dtype)["routing"]
            r.served_slot.copy_(indices)
            r.served_weight.fill_(1.0)
            layer.decode(x, stages=_lib.STAGE_PREPARE | _lib.STAGE_GATE_UP | _lib.STAGE_DOWN)
            out = layer.route_outputs(tokens, x.dtype).reshape(tokens, k, -1).clone()
            picks = indices.to(torch.int64)
            dead = (picks < 0) | (picks >= self.gate_proj.num_experts)  # rows the kernels never write
            return out.masked_fill_(dead[..., None], 0)
        gate = self.gate_proj(x, indices)
        up = self.up_proj(x, indices)
        return self.down_proj(self._apply_activation(up, gate), indices)
