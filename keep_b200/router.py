"""Router with routed residency: one evaluation, served and demand top-k, admission flags.

The reference spreads this over ``Gate.forward`` (``tests/fixtures/v41_reference/model.py:811-829``),
``gate_masked`` (``scripts/runpod/v41_reap/local_eval.py:69-90``), the fused ``_TOPK`` kernel
(``scripts/v41_build/omlx_lattice.py:77-104,333-338``) and ``Cache.harvest``'s admission test
(``scripts/v41_build/omlx_routed.py:184-203``).  Here it is two CUDA launches and no host read.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from .vq import as_device

#: A served bias at or below this marks an absent expert (the reference uses -1e30,
#: ``scripts/v41_build/omlx_routed.py:40``; ``-inf`` works too).
OFF = -1e30
NO_SLOT = _lib.NO_RESIDUAL


@dataclass
class Routing:
    """Outputs of :func:`routed_topk`, all ``[tokens, top_k]`` device tensors.

    ``served_expert`` / ``served_slot`` hold ``NO_SLOT`` (as -1 in int32 view) where a pick fell on
    an absent expert; ``admit`` holds the expert id to admit or -1.
    """

    served_expert: torch.Tensor
    served_slot: torch.Tensor
    served_weight: torch.Tensor
    want: torch.Tensor
    want_score: torch.Tensor
    admit: torch.Tensor
    scores: torch.Tensor | None = None


def router_logits(x: torch.Tensor, router_w: torch.Tensor, *, gate_temp: float = 1.0) -> torch.Tensor:
    """``(x @ router_w.T) / gate_temp`` in fp32 with a fixed summation order: ``[tokens, pool]``."""
    device = _lib.require_cuda(x, router_w)
    x, router_w = x.contiguous(), router_w.contiguous()
    if x.ndim != 2 or router_w.ndim != 2 or x.shape[1] != router_w.shape[1]:
        raise ValueError(f"router needs x [tokens, hidden] and router_w [pool, hidden], got {tuple(x.shape)} and {tuple(router_w.shape)}")
    tokens, hidden = (int(s) for s in x.shape)
    pool = int(router_w.shape[0])
    logits = torch.empty((tokens, pool), dtype=torch.float32, device=device)
    args = _lib.RouterLogitsArgs(
        x=_lib.ptr(x), x_dtype=_lib.dtype_tag(x.dtype), router_w=_lib.ptr(router_w),
        router_dtype=_lib.dtype_tag(router_w.dtype), tokens=tokens, pool=pool, hidden=hidden,
        gate_temp=float(gate_temp), logits=_lib.ptr(logits))
    with torch.cuda.device(device):
        _lib.check(_lib.load().keepvq_router_logits(args, _lib.stream_handle(device)), "keepvq_router_logits")
    return logits


def _opt_f32(t, device, pool):
    if t is None:
        return None
    t = as_device(t, device).to(torch.float32).contiguous()
    if tuple(t.shape) != (pool,):
        raise ValueError(f"a router bias must have shape ({pool},), found {tuple(t.shape)}")
    return t


def routed_topk(x, router_w, bias=None, pool_bias=None, slot_of=None, *, top_k: int, score_func: str = "softmax",
                route_scale: float = 1.0, tau: float = 0.3, gate_temp: float = 1.0, norm_topk_prob: bool = True,
                return_scores: bool = False, logits: torch.Tensor | None = None) -> Routing:
    """Served and demand selections from one router evaluation.

    ``bias`` is the served bias (the model's selection bias, with ``OFF`` or ``-inf`` on absent
    experts); ``pool_bias`` the model's own bias over the whole pool; ``slot_of`` maps an expert to
    its slot in the resident weight arrays (identity when None).  ``logits`` may be passed to skip
    the matmul.
    """
    if score_func not in _lib.SCORE_FUNCS:
        raise ValueError("score_func must be 'softmax', 'sigmoid' or 'sqrtsoftplus'")
    if logits is None:
        logits = router_logits(x, router_w, gate_temp=gate_temp)
    device = _lib.require_cuda(logits)
    tokens, pool = (int(s) for s in logits.shape)
    if not 1 <= top_k <= min(16, pool):
        raise ValueError(f"top_k must be in 1..{min(16, pool)}, got {top_k}")
    bias_t, pool_bias_t = _opt_f32(bias, device, pool), _opt_f32(pool_bias, device, pool)
    slot_t = None
    if slot_of is not None:
        slot_t = as_device(slot_of, device)
        slot_t = (slot_t if slot_t.dtype in (torch.uint32, torch.int32) else slot_t.to(torch.int64).to(torch.int32)).contiguous()
    u32 = lambda: torch.empty((tokens, top_k), dtype=torch.int32, device=device)  # noqa: E731 - uint32 bits
    f32 = lambda: torch.empty((tokens, top_k), dtype=torch.float32, device=device)  # noqa: E731
    out = Routing(served_expert=u32(), served_slot=u32(), served_weight=f32(), want=u32(), want_score=f32(), admit=u32(),
                  scores=torch.empty((tokens, pool), dtype=torch.float32, device=device) if return_scores else None)
    args = _lib.RoutedTopkArgs(
        logits=_lib.ptr(logits), tokens=tokens, pool=pool, top_k=top_k, score_func=_lib.SCORE_FUNCS[score_func],
        norm_topk_prob=int(bool(norm_topk_prob)), route_scale=float(route_scale), tau=float(tau),
        served_bias=_lib.ptr(bias_t), pool_bias=_lib.ptr(pool_bias_t), slot_of=_lib.ptr(slot_t), scores=_lib.ptr(out.scores),
        served_expert=_lib.ptr(out.served_expert), served_slot=_lib.ptr(out.served_slot),
        served_weight=_lib.ptr(out.served_weight), want=_lib.ptr(out.want), want_score=_lib.ptr(out.want_score),
        admit=_lib.ptr(out.admit))
    with torch.cuda.device(device):
        _lib.check(_lib.load().keepvq_routed_topk(args, _lib.stream_handle(device)), "keepvq_routed_topk")
    return out
