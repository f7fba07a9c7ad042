"""The operator surface as PyTorch custom ops: ``torch.ops.keepvq.*``.

Every operator of the drop-in boundary is registered with ``torch.library`` (schema inferred from
the annotations, a fake implementation for shape propagation), so the dispatcher, ``torch.compile``
and ``torch.library.opcheck`` see them; the CUDA work underneath is unchanged: each op calls the
Python operator of the same name, which calls the C ABI of ``libkeepvq.so`` through ``ctypes``.

==============================  ==========================================================
op                              reference interface it stands in for
==============================  ==========================================================
``vq_qmv`` / ``vq_qmm``         ``src/ramp/kernels/vq_qmv.py:163-232`` / ``vq_qmm.py:93-152``
``e8p_m1_*``                    ``src/ramp/kernels/e8p_m1.py:134-183``
``e8_1bit_m1_*``                ``src/ramp/kernels/e8_1bit_m1.py:76-97``
``e8p_nested_m1_*``             ``src/ramp/kernels/e8p_nested_m1.py:90-112``
``vq_switch_qmv``               ``src/ramp/ops/vq_switch.py:547-561``
``gather_vqmm``                 ``src/ramp/ops/vq_switch.py:916-932``
``gather_vqmm_sorted_routes``   ``src/ramp/ops/vq_switch.py:620-640``
``routed_topk``                 ``scripts/v41_build/omlx_lattice.py:77-104,333-338``
``moe_decode_layer``            ``scripts/v41_build/omlx_lattice.py:327-371``
==============================  ==========================================================

Arguments are tensors and plain scalars only (what a schema can carry): tables are passed
explicitly, tuples of the nested operators are flattened, keyword-only arguments keep their names.
None of the ops mutates an argument; outputs are fresh tensors.  There is no autograd formula:
this is an inference path.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor
from torch.library import custom_op

from . import kernels, moe, router, vq_switch

__all__ = ["OPS"]

_CUDA = "cuda"


def _out_dtype(x: Tensor) -> torch.dtype:
    return x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.float32


# ---- single-matrix products ---------------------------------------------------------------------

@custom_op("keepvq::vq_qmv", mutates_args=(), device_types=_CUDA)
def vq_qmv(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, in_dim: int, out_dim: int, group_size: int, code_bits: int) -> Tensor:
    return kernels.vq_qmv(x, codes, scales, codebook, in_dim=in_dim, out_dim=out_dim, group_size=group_size, code_bits=code_bits)


@vq_qmv.register_fake
def _(x, codes, scales, codebook, in_dim, out_dim, group_size, code_bits):
    return x.new_empty((out_dim,), dtype=_out_dtype(x))


@custom_op("keepvq::vq_qmm", mutates_args=(), device_types=_CUDA)
def vq_qmm(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, in_dim: int, out_dim: int, group_size: int, code_bits: int) -> Tensor:
    return kernels.vq_qmm(x, codes, scales, codebook, in_dim=in_dim, out_dim=out_dim, group_size=group_size, code_bits=code_bits)


@vq_qmm.register_fake
def _(x, codes, scales, codebook, in_dim, out_dim, group_size, code_bits):
    return x.new_empty((x.shape[0], out_dim), dtype=_out_dtype(x))


# ---- few-token routed products --------------------------------------------------------------------

def _token_shape(x, rhs_indices, output_dims):
    return x.new_empty((rhs_indices.shape[0], rhs_indices.shape[1], output_dims), dtype=_out_dtype(x))


def _route_shape(x, rhs_indices, output_dims):
    return x.new_empty((rhs_indices.numel(), output_dims), dtype=_out_dtype(x))


@custom_op("keepvq::e8p_m1_token_layout", mutates_args=(), device_types=_CUDA)
def e8p_m1_token_layout(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, rhs_indices: Tensor, output_dims: int) -> Tensor:
    return kernels.e8p_m1_token_layout(x, codes, scales, codebook, rhs_indices, output_dims=output_dims)


@e8p_m1_token_layout.register_fake
def _(x, codes, scales, codebook, rhs_indices, output_dims):
    return _token_shape(x, rhs_indices, output_dims)


@custom_op("keepvq::e8p_m1_per_route", mutates_args=(), device_types=_CUDA)
def e8p_m1_per_route(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, rhs_indices: Tensor, output_dims: int) -> Tensor:
    return kernels.e8p_m1_per_route(x, codes, scales, codebook, rhs_indices, output_dims=output_dims)


@e8p_m1_per_route.register_fake
def _(x, codes, scales, codebook, rhs_indices, output_dims):
    return _route_shape(x, rhs_indices, output_dims)


@custom_op("keepvq::e8_1bit_m1_token_layout", mutates_args=(), device_types=_CUDA)
def e8_1bit_m1_token_layout(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, rhs_indices: Tensor, output_dims: int) -> Tensor:
    return kernels.e8_1bit_m1_token_layout(x, codes, scales, codebook, rhs_indices, output_dims=output_dims)


@e8_1bit_m1_token_layout.register_fake
def _(x, codes, scales, codebook, rhs_indices, output_dims):
    return _token_shape(x, rhs_indices, output_dims)


@custom_op("keepvq::e8_1bit_m1_per_route", mutates_args=(), device_types=_CUDA)
def e8_1bit_m1_per_route(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, rhs_indices: Tensor, output_dims: int) -> Tensor:
    return kernels.e8_1bit_m1_per_route(x, codes, scales, codebook, rhs_indices, output_dims=output_dims)


@e8_1bit_m1_per_route.register_fake
def _(x, codes, scales, codebook, rhs_indices, output_dims):
    return _route_shape(x, rhs_indices, output_dims)


@custom_op("keepvq::e8p_nested_m1_token_layout", mutates_args=(), device_types=_CUDA)
def e8p_nested_m1_token_layout(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, rhs_indices: Tensor, res_codes: Tensor,
                               res_scales: Tensor, res_table: Tensor, hot_of_slot: Tensor, output_dims: int) -> Tensor:
    return kernels.e8p_nested_m1_token_layout(x, (codes, scales, codebook), rhs_indices, (res_codes, res_scales, res_table), hot_of_slot,
                                              output_dims=output_dims)


@e8p_nested_m1_token_layout.register_fake
def _(x, codes, scales, codebook, rhs_indices, res_codes, res_scales, res_table, hot_of_slot, output_dims):
    return _token_shape(x, rhs_indices, output_dims)


@custom_op("keepvq::e8p_nested_m1_per_route", mutates_args=(), device_types=_CUDA)
def e8p_nested_m1_per_route(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, rhs_indices: Tensor, res_codes: Tensor,
                            res_scales: Tensor, res_table: Tensor, hot_of_slot: Tensor, output_dims: int) -> Tensor:
    return kernels.e8p_nested_m1_per_route(x, (codes, scales, codebook), rhs_indices, (res_codes, res_scales, res_table), hot_of_slot,
                                           output_dims=output_dims)


@e8p_nested_m1_per_route.register_fake
def _(x, codes, scales, codebook, rhs_indices, res_codes, res_scales, res_table, hot_of_slot, output_dims):
    return _route_shape(x, rhs_indices, output_dims)


# ---- the switch operators ---------------------------------------------------------------------------

@custom_op("keepvq::vq_switch_qmv", mutates_args=(), device_types=_CUDA)
def vq_switch_qmv(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, indices: Tensor, input_dims: int, output_dims: int,
                  group_size: int, code_bits: int) -> Tensor:
    return vq_switch.vq_switch_qmv(x, codes, scales, codebook, indices, input_dims=input_dims, output_dims=output_dims,
                                   group_size=group_size, code_bits=code_bits)


@vq_switch_qmv.register_fake
def _(x, codes, scales, codebook, indices, input_dims, output_dims, group_size, code_bits):
    lead = tuple(indices.shape[:-1]) if tuple(x.shape[:-1]) == tuple(indices.shape[:-1]) else tuple(x.shape[:-2])
    return x.new_empty(lead + (indices.shape[-1], output_dims), dtype=_out_dtype(x))


@custom_op("keepvq::gather_vqmm", mutates_args=(), device_types=_CUDA)
def gather_vqmm(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, rhs_indices: Tensor, lhs_indices: Optional[Tensor], input_dims: int,
                output_dims: int, group_size: int, code_bits: int, sorted_indices: bool, route_strategy: str) -> Tensor:
    return vq_switch.gather_vqmm(x, codes, scales, codebook, rhs_indices, lhs_indices=lhs_indices, input_dims=input_dims, output_dims=output_dims,
                                 group_size=group_size, code_bits=code_bits, sorted_indices=sorted_indices, route_strategy=route_strategy)


@gather_vqmm.register_fake
def _(x, codes, scales, codebook, rhs_indices, lhs_indices, input_dims, output_dims, group_size, code_bits, sorted_indices, route_strategy):
    if lhs_indices is not None:
        return x.new_empty((rhs_indices.numel(), output_dims), dtype=_out_dtype(x))
    return x.new_empty(tuple(rhs_indices.shape) + (output_dims,), dtype=_out_dtype(x))


@custom_op("keepvq::gather_vqmm_sorted_routes", mutates_args=(), device_types=_CUDA)
def gather_vqmm_sorted_routes(x: Tensor, codes: Tensor, scales: Tensor, codebook: Tensor, sorted_rhs: Tensor, sorted_lhs: Optional[Tensor],
                              input_dims: int, output_dims: int, group_size: int, code_bits: int, x_pre_sorted: bool) -> Tensor:
    return vq_switch.gather_vqmm_sorted_routes(x, codes, scales, codebook, sorted_rhs, sorted_lhs, input_dims=input_dims, output_dims=output_dims,
                                               group_size=group_size, code_bits=code_bits, x_pre_sorted=x_pre_sorted)


@gather_vqmm_sorted_routes.register_fake
def _(x, codes, scales, codebook, sorted_rhs, sorted_lhs, input_dims, output_dims, group_size, code_bits, x_pre_sorted):
    return x.new_empty((sorted_rhs.numel(), output_dims), dtype=_out_dtype(x))


# ---- router and layer ---------------------------------------------------------------------------------

@custom_op("keepvq::routed_topk", mutates_args=(), device_types=_CUDA)
def routed_topk(x: Tensor, router_w: Tensor, served_bias: Optional[Tensor], pool_bias: Optional[Tensor], slot_of: Optional[Tensor], top_k: int,
                score_func: str, route_scale: float, tau: float, gate_temp: float,
                norm_topk_prob: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """-> (served_expert, served_slot, served_weight, want, want_score, admit), each [tokens, top_k]."""
    r = router.routed_topk(x, router_w, served_bias, pool_bias, slot_of, top_k=top_k, score_func=score_func, route_scale=route_scale, tau=tau,
                           gate_temp=gate_temp, norm_topk_prob=norm_topk_prob)
    return r.served_expert, r.served_slot, r.served_weight, r.want, r.want_score, r.admit


def _routing_shapes(x, top_k):
    ints = lambda: x.new_empty((x.shape[0], top_k), dtype=torch.int32)  # noqa: E731
    floats = lambda: x.new_empty((x.shape[0], top_k), dtype=torch.float32)  # noqa: E731
    return ints(), ints(), floats(), ints(), floats(), ints()


@routed_topk.register_fake
def _(x, router_w, served_bias, pool_bias, slot_of, top_k, score_func, route_scale, tau, gate_temp, norm_topk_prob):
    return _routing_shapes(x, top_k)


_layers: dict = {}   # the weights' addresses -> the layer object that holds their scratch
_MAX_LAYERS = 128


@custom_op("keepvq::moe_decode_layer", mutates_args=(), device_types=_CUDA)
def moe_decode_layer(x: Tensor, router_w: Tensor, w1_codes: Tensor, w1_scales: Tensor, w3_codes: Tensor, w3_scales: Tensor, w2_codes: Tensor,
                     w2_scales: Tensor, served_bias: Optional[Tensor], pool_bias: Optional[Tensor], slot_of: Optional[Tensor], top_k: int,
                     score_func: str, route_scale: float, tau: float, gate_temp: float, norm_topk_prob: bool,
                     swiglu_limit: float) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """One routed MoE layer at decode: (out [tokens, hidden], then the six routing outputs of
    ``routed_topk``).  The three bias / slot tables are read on every call, so a residency policy
    may rewrite them between calls."""
    key = (router_w.data_ptr(), w1_codes.data_ptr(), w3_codes.data_ptr(), w2_codes.data_ptr(), top_k, score_func, route_scale, tau, gate_temp,
           norm_topk_prob, swiglu_limit)
    layer = _layers.get(key)
    if layer is None or layer.w1.codes is not w1_codes or layer.w1.scales is not w1_scales:
        if len(_layers) >= _MAX_LAYERS:
            _layers.pop(next(iter(_layers)))
        layer = _layers[key] = moe.RoutedMoELayer(router_w, moe.Projection(w1_codes, w1_scales), moe.Projection(w3_codes, w3_scales),
                                                  moe.Projection(w2_codes, w2_scales), top_k=top_k, score_func=score_func, route_scale=route_scale,
                                                  tau=tau, gate_temp=gate_temp, norm_topk_prob=norm_topk_prob, served_bias=served_bias,
                                                  pool_bias=pool_bias, slot_of=slot_of, swiglu_limit=swiglu_limit)
    layer.served_bias, layer.pool_bias, layer.slot_of = served_bias, pool_bias, slot_of  # the caller's current tables
    out, r = layer.decode(x)
    return (out.clone(), r.served_expert.clone(), r.served_slot.clone(), r.served_weight.clone(), r.want.clone(), r.want_score.clone(), r.admit.clone())


@moe_decode_layer.register_fake
def _(x, router_w, w1_codes, w1_scales, w3_codes, w3_scales, w2_codes, w2_scales, served_bias, pool_bias, slot_of, top_k, score_func, route_scale,
      tau, gate_temp, norm_topk_prob, swiglu_limit):
    return (torch.empty_like(x),) + _routing_shapes(x, top_k)


OPS = ("vq_qmv", "vq_qmm", "e8p_m1_token_layout", "e8p_m1_per_route", "e8_1bit_m1_token_layout", "e8_1bit_m1_per_route",
       "e8p_nested_m1_token_layout", "e8p_nested_m1_per_route", "vq_switch_qmv", "gather_vqmm", "gather_vqmm_sorted_routes", "routed_topk",
       "moe_decode_layer")
