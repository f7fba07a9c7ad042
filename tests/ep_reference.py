"""The expert-parallel exchange in plain ``torch`` (+ ``torch.distributed``): the checker of
``keep_b200.expert_parallel.RouteExchange`` and of the ``keepvq_ep_*`` kernels.  Test
infrastructure only; it runs on CPU tensors so that the index arithmetic can be exercised on
gloo ranks without GPUs."""

import torch
import torch.distributed as dist

NO_SLOT = -1


class TorchRouteExchange:
    """Same positions, buffers and sums as ``RouteExchange``, computed with torch ops."""

    def __init__(self, experts_per_rank, *, group=None, capacity=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.experts_per_rank = int(experts_per_rank)
        self.capacity = capacity

    def plan(self, served_expert):
        """served_expert [tokens, k] (global ids, negative = dead pick) -> (position [tokens, k] of
        each route in the send buffer, ``world * capacity`` for a dead or overflowing route; capacity)."""
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

    def pack(self, x, served_expert, served_weight):
        """(send_x [rows, hidden], send_slot [rows], send_weight [rows], position [tokens, k])."""
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
        return send_x[:rows], send_slot[:rows], send_weight[:rows], position

    def dispatch(self, x, served_expert, served_weight):
        send_x, send_slot, send_weight, position = self.pack(x, served_expert, served_weight)
        return self._all_to_all(send_x), self._all_to_all(send_slot), self._all_to_all(send_weight), position

    def combine(self, y_routes, position, out_dtype):
        """Each token's picks summed in fp32 in pick order, one rounding."""
        back = self._all_to_all(y_routes)
        back = torch.cat([back, torch.zeros((1, back.shape[1]), dtype=back.dtype, device=back.device)])  # row of a dead route
        tokens, k = position.shape
        acc = torch.zeros((tokens, back.shape[1]), dtype=torch.float32, device=back.device)
        for j in range(k):
            acc += back[position[:, j]].float()
        return acc.to(out_dtype)

    def _all_to_all(self, send):
        if self.world == 1:
            return send
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv
