"""Router, residency-masked routing and the layer forward, restated on the CPU (numpy + torch CPU).

TEST INFRASTRUCTURE: the checker for the CUDA router and fused layer, never shipped.

Follows the reference:

* ``scores`` / ``gate``      ``tests/fixtures/v41_reference/model.py:811-829`` (Gate.forward)
* ``gate_masked``            ``scripts/runpod/v41_reap/local_eval.py:69-90``
* ``routed_topk``            ``scripts/v41_build/omlx_lattice.py:77-104`` (served + demand from one
                             evaluation) and ``scripts/v41_build/omlx_routed.py:184-203`` (admission)
* ``moe_layer``              ``scripts/v41_build/omlx_lattice.py:356-371,583-589`` (rounding points of
                             the served path), ``scripts/runpod/v41_reap/local_eval.py:508-512``

Ties at the top-k cut are implementation-defined in the reference (torch.topk); here they go to
the lowest expert id, and the input generators of the tests reject seeds with a tie at the cut.
"""

from __future__ import annotations

import numpy as np
import torch

from .e8 import NO_RESIDUAL, decode_weight_matrix, e8_1bit_grid

OFF = -1e30
ABSENT_BELOW = -1e29


def scores(x, router_w, *, score_func="softmax", gate_temp=1.0) -> torch.Tensor:
    """f(x.float() @ W.float().T / temp), float32 [tokens, pool]."""
    x = torch.as_tensor(np.asarray(x, dtype=np.float32)) if not isinstance(x, torch.Tensor) else x.detach().cpu().float()
    w = torch.as_tensor(np.asarray(router_w, dtype=np.float32)) if not isinstance(router_w, torch.Tensor) else router_w.detach().cpu().float()
    s = torch.nn.functional.linear(x, w) / gate_temp
    if score_func == "softmax":
        return s.softmax(dim=-1)
    if score_func == "sigmoid":
        return s.sigmoid()
    if score_func == "sqrtsoftplus":
        return torch.nn.functional.softplus(s).sqrt()
    raise ValueError(score_func)


def top_k_lowest_index(keys: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest keys per row, descending, ties to the lowest index."""
    order = np.argsort(-keys.numpy().astype(np.float64), axis=-1, kind="stable")[:, :k]
    return torch.as_tensor(order.copy())


def min_cut_gap(keys: torch.Tensor, k: int) -> float:
    """Smallest gap between the k-th and (k+1)-th key over the rows (generators assert it is > 0)."""
    top = torch.sort(keys.double(), dim=-1, descending=True).values
    if top.shape[1] <= k:
        return float("inf")
    gap = top[:, k - 1] - top[:, k]
    return float(gap[torch.isfinite(gap)].min()) if torch.isfinite(gap).any() else float("inf")


def gate_masked(sc: torch.Tensor, bias, allowed, *, top_k, norm_topk_prob=True, route_scale=1.0):
    """Top-k among the allowed experts; weights from raw scores, zero on a disallowed pick,
    renormalised over the picks, times route_scale.  Returns (weights, indices)."""
    bias = torch.zeros(sc.shape[1]) if bias is None else torch.as_tensor(np.asarray(bias, dtype=np.float32))
    allowed = torch.as_tensor(np.asarray(allowed, dtype=bool))
    if allowed.ndim == 1:
        allowed = allowed[None].expand_as(sc)
    keys = (sc + bias).masked_fill(~allowed, float("-inf"))
    idx = top_k_lowest_index(keys, top_k)
    w = sc.gather(1, idx) * allowed.gather(1, idx)
    if norm_topk_prob and top_k > 1:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return w * route_scale, idx


def routed_topk(x, router_w, served_bias=None, pool_bias=None, slot_of=None, *, top_k, score_func="softmax",
                route_scale=1.0, tau=0.3, gate_temp=1.0, norm_topk_prob=True):
    """dict of served_expert / served_slot / served_weight / want / want_score / admit, all
    [tokens, top_k].  served_bias <= -1e29 marks an absent expert."""
    sc = scores(x, router_w, score_func=score_func, gate_temp=gate_temp)
    pool = sc.shape[1]
    sb = torch.zeros(pool) if served_bias is None else torch.as_tensor(np.asarray(served_bias, dtype=np.float32))
    pb = torch.zeros(pool) if pool_bias is None else torch.as_tensor(np.asarray(pool_bias, dtype=np.float32))
    resident = sb > ABSENT_BELOW
    w, idx = gate_masked(sc, torch.where(resident, sb, torch.zeros(pool)).numpy(), resident.numpy(), top_k=top_k,
                         norm_topk_prob=norm_topk_prob, route_scale=route_scale)
    live = resident[idx]
    slot_map = torch.arange(pool) if slot_of is None else torch.as_tensor(np.asarray(slot_of).astype(np.int64))
    want = top_k_lowest_index(sc + pb, top_k)
    want_score = sc.gather(1, want)
    g = want_score / (want_score.sum(dim=-1, keepdim=True) + 1e-20) * route_scale
    admit = torch.where((~resident[want]) & (g >= tau), want, torch.full_like(want, -1))
    return dict(
        scores=sc, served_expert=torch.where(live, idx, torch.full_like(idx, -1)),
        served_slot=torch.where(live, slot_map[idx], torch.full_like(idx, -1)), served_weight=w,
        want=want, want_score=want_score, admit=admit, demand_weight=g,
        served_keys=(sc + torch.where(resident, sb, torch.full((pool,), float("-inf")))), demand_keys=sc + pb)


def _round(t: torch.Tensor, dtype) -> torch.Tensor:
    return t.to(dtype).float()


def moe_layer(x, served_slot, served_weight, dense_w1, dense_w3, dense_w2, *, dtype=torch.bfloat16, swiglu_limit=0.0):
    """The served path's forward with its rounding points.  ``dense_*`` map slot -> fp32 [out, in]
    (a dict or an indexable); ``served_slot`` < 0 marks a switched-off pick.  Returns fp32
    [tokens, hidden] holding values already rounded to ``dtype``."""
    x = x.detach().cpu().float() if isinstance(x, torch.Tensor) else torch.as_tensor(np.asarray(x, dtype=np.float32))
    slots = torch.as_tensor(np.asarray(served_slot)).long()
    weights = torch.as_tensor(np.asarray(served_weight, dtype=np.float32))
    tokens, k = slots.shape
    out = None
    for t in range(tokens):
        y = None
        for j in range(k):
            s = int(slots[t, j])
            if s < 0 or s == NO_RESIDUAL:
                continue
            w1, w3, w2 = (torch.as_tensor(np.asarray(d[s], dtype=np.float32)) for d in (dense_w1, dense_w3, dense_w2))
            g = _round(w1 @ x[t], dtype)
            u = _round(w3 @ x[t], dtype)
            if swiglu_limit > 0:
                g, u = g.clamp(max=swiglu_limit), u.clamp(-swiglu_limit, swiglu_limit)
            h = _round(torch.nn.functional.silu(g) * u * weights[t, j], dtype)
            d = _round(w2 @ h, dtype)
            y = d.clone() if y is None else y + d
        if y is None:
            y = torch.zeros(dense_hidden(dense_w2, slots))
        row = _round(y, dtype)
        out = torch.zeros((tokens, row.shape[0])) if out is None else out
        out[t] = row
    return out


def dense_hidden(dense_w2, slots) -> int:
    any_slot = next(iter(dense_w2)) if isinstance(dense_w2, dict) else 0
    return int(np.asarray(dense_w2[any_slot]).shape[0])


_FULL_GRID = None


def decode_torch(codes, scales) -> torch.Tensor:
    """[out, in/8] uint16 codes + [out, groups] scales -> fp32 [out, in] by indexing the full
    65,536-entry grid, the way the reference's CPU path decodes
    (``scripts/runpod/v41_reap/keep_quant.py`` ``decode_codes``: grid[codes] * scale)."""
    global _FULL_GRID
    if _FULL_GRID is None:
        from .e8 import e8p_full_grid
        _FULL_GRID = torch.from_numpy(np.array(e8p_full_grid()))
    c = torch.as_tensor(np.asarray(codes).astype(np.int64))
    s = torch.as_tensor(np.asarray(scales).astype(np.float32))
    w = _FULL_GRID[c]  # [out, cw, 8]
    w = w * s.repeat_interleave(c.shape[1] // s.shape[1], dim=1)[..., None]
    return w.reshape(c.shape[0], -1)


def dense_slots(codes, scales, wanted, *, res=None, hot_of_slot=None) -> dict:
    """slot -> fp32 [out, in] for the slots in ``wanted``: base decode, plus the 8-bit residual row
    ``hot_of_slot[slot]`` when the slot has one (``res`` = (res_codes, res_scales))."""
    out = {}
    codes, scales = np.asarray(codes), np.asarray(scales)
    for s in sorted({int(v) for v in np.asarray(wanted).reshape(-1) if 0 <= int(v) != NO_RESIDUAL}):
        w = decode_weight_matrix(codes[s], scales[s].astype(np.float32), code_bits=16).astype(np.float64)
        if res is not None and hot_of_slot is not None:
            h = int(np.asarray(hot_of_slot).astype(np.int64)[s]) & 0xFFFFFFFF
            if h != NO_RESIDUAL:
                rc, rs = np.asarray(res[0])[h], np.asarray(res[1])[h].astype(np.float64)
                r = e8_1bit_grid().astype(np.float64)[rc].reshape(rc.shape[0], -1)
                w = w + r * np.repeat(rs, r.shape[1] // rs.shape[-1], axis=-1)
        out[s] = w.astype(np.float32)
    return out
