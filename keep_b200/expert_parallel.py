"""Expert parallelism for the routed layer: experts sharded across the GPUs of one node, tokens
data-parallel, a dispatch all-to-all before the experts and a combine all-to-all after.

The reference has no token all-to-all; its only expert-parallel form replicates the tokens on
every rank, runs the local slice of experts and all-reduces the outputs
(``tests/fixtures/v41_reference/model.py:869-872,891-906``).  The result here is the same sum over
each token's k picks, computed with each token's hidden state visiting only the ranks that own
its experts.

Exchange without a host read.  Split sizes that depend on the routing would have to reach the
host before NCCL could be called.  Instead every (source, destination) pair owns a fixed block of
``capacity`` route slots (default: all of a rank's routes, so nothing can overflow); unused slots
carry slot id ``NO_SLOT`` and the expert kernels skip them.  At decode sizes the padding is a
few MB per layer on NVLink and the whole step stays capturable in a CUDA graph.

``RouteExchange`` is plain ``torch`` + ``torch.distributed`` and runs on CPU ranks (gloo) as well,
which is how its index arithmetic is tested without GPUs.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

NO_SLOT = -1


class RouteExchange:
    """Dispatch / combine of routes between ``world`` ranks that each own ``experts_per_rank``
    consecutive experts."""

    def __init__(self, experts_per_rank: int, *, group=None, capacity: int | None = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.experts_per_rank = int(experts_per_rank)
        self.capacity = capacity

    def plan(self, served_expert: torch.Tensor):
        """served_expert [tokens, k] (global ids, negative = dead pick) -> (position [tokens, k] of
        each route in the send buffer, with ``world * capacity`` for a dead or overflowing route;
        capacity).  Fixed-shape device arithmetic only: nothing is read back, so the exchange can
        sit inside a CUDA graph."""
        tokens, k = served_expert.shape
        routes = tokens * k
        capacity = self.capacity or routes
        rows = self.world * capacity
        flat = served_expert.reshape(-1).long()
        dest = torch.where(flat >= 0, flat // self.experts_per_rank, torch.full_like(flat, self.world))  # dead routes sort last
        order = torch.argsort(dest, stable=True)
        counts = torch.zeros(self.world + 1, dtype=torch.long, device=flat.device).scatter_add_(0, dest, torch.ones_like(dest))
        starts = torch.cumsum(counts, 0) - counts
        sorted_dest = dest[order]
        rank_in_bucket = torch.arange(routes, device=flat.device) - starts[sorted_dest]
        ok = (sorted_dest < self.world) & (rank_in_bucket < capacity)
        sorted_pos = torch.where(ok, sorted_dest * capacity + rank_in_bucket, torch.full_like(rank_in_bucket, rows))
        position = torch.empty_like(sorted_pos).scatter_(0, order, sorted_pos)
        return position.reshape(tokens, k), capacity

    def dispatch(self, x: torch.Tensor, served_expert: torch.Tensor, served_weight: torch.Tensor):
        """-> (recv_x [world * capacity, hidden], recv_slot [..] local expert or NO_SLOT,
        recv_weight [..], position [tokens, k])."""
        tokens, k = served_expert.shape
        position, capacity = self.plan(served_expert)
        rows = self.world * capacity
        flat_pos = position.reshape(-1)  # dead routes point at the spare row `rows`, cut off below
        token_of_route = torch.arange(tokens * k, device=x.device) // k
        send_x = torch.zeros((rows + 1, x.shape[1]), dtype=x.dtype, device=x.device)
        send_x.index_copy_(0, flat_pos, x[token_of_route])
        local_slot = (served_expert.reshape(-1).long().clamp(min=0) % self.experts_per_rank).to(torch.int32)
        send_slot = torch.full((rows + 1,), NO_SLOT, dtype=torch.int32, device=x.device)
        send_slot.index_copy_(0, flat_pos, local_slot)
        send_weight = torch.zeros((rows + 1,), dtype=torch.float32, device=x.device)
        send_weight.index_copy_(0, flat_pos, served_weight.reshape(-1).float())
        return (self._all_to_all(send_x[:rows]), self._all_to_all(send_slot[:rows]), self._all_to_all(send_weight[:rows]), position)

    def combine(self, y_routes: torch.Tensor, position: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """y_routes [world * capacity, hidden] (per received route) -> [tokens, hidden]: each token's
        picks summed in fp32 in pick order, one rounding."""
        back = self._all_to_all(y_routes)
        back = torch.cat([back, torch.zeros((1, back.shape[1]), dtype=back.dtype, device=back.device)])  # row of a dead route
        tokens, k = position.shape
        acc = torch.zeros((tokens, back.shape[1]), dtype=torch.float32, device=back.device)
        for j in range(k):  # pick order, as the single-GPU combine
            acc += back[position[:, j]].float()
        return acc.to(out_dtype)

    def _all_to_all(self, send: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return send
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv


class ExpertParallelLayer:
    """One routed MoE layer whose experts are sharded over the ranks of ``group``.

    ``local`` is a ``RoutedMoELayer`` built with ``top_k=1`` over this rank's shard of the experts
    (its router is not used); ``router_w`` is the full, replicated router.
    """

    def __init__(self, router_w: torch.Tensor, local, *, experts_per_rank: int, top_k: int, group=None, score_func: str = "softmax",
                 route_scale: float = 1.0, norm_topk_prob: bool = True, capacity: int | None = None):
        self.router_w, self.local = router_w.contiguous(), local
        self.top_k, self.score_func, self.route_scale, self.norm_topk_prob = top_k, score_func, route_scale, norm_topk_prob
        self.exchange = RouteExchange(experts_per_rank, group=group, capacity=capacity)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import _lib
        from .router import routed_topk

        routing = routed_topk(x, self.router_w, top_k=self.top_k, score_func=self.score_func, route_scale=self.route_scale,
                              norm_topk_prob=self.norm_topk_prob)
        recv_x, recv_slot, recv_weight, position = self.exchange.dispatch(x, routing.served_expert, routing.served_weight)
        buf = self.local._buffers_for(int(recv_x.shape[0]), recv_x.dtype)
        r = buf["routing"]
        r.served_slot.copy_(recv_slot.reshape(-1, 1))
        r.served_weight.copy_(recv_weight.reshape(-1, 1))
        y, _ = self.local.decode(recv_x, stages=_lib.STAGE_ALL & ~_lib.STAGE_ROUTER)
        return self.exchange.combine(y, position, x.dtype)
