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

``PeerExchange`` is the NVLink form: rows go straight into the peers' buffers, no collective in the
data path.  ``RouteExchange`` is the NCCL form: its packing and pick summation are the library's own
kernels (``keepvq_ep_pack``, ``keepvq_ep_combine``: a memset and three launches per layer besides
the all-to-alls).  Both take CUDA tensors only; there is no CPU path.  (The index arithmetic is
checked against a plain ``torch`` restatement that lives with the tests.)
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
        self._cuda_buffers: dict = {}

    def dispatch(self, x: torch.Tensor, served_expert: torch.Tensor, served_weight: torch.Tensor):
        """-> (recv_x [world * capacity, hidden], recv_slot [..] local expert or NO_SLOT,
        recv_weight [..], position [tokens, k]).  One library call packs rows, slots and weights;
        two all-to-alls carry them.  Buffers are cached per shape so the step can be graph-captured."""
        if not x.is_cuda:
            raise ValueError("RouteExchange works on CUDA tensors only")
        return self._dispatch_cuda(x, served_expert, served_weight)

    def _dispatch_cuda(self, x: torch.Tensor, served_expert: torch.Tensor, served_weight: torch.Tensor):
        send_x, send_meta, position = self.pack_cuda(x, served_expert, served_weight)
        if self.world == 1:
            recv_x, recv_meta = send_x, send_meta
        else:
            buf = self._cuda_buffers[(tuple(served_expert.shape), int(x.shape[1]), x.dtype)]
            recv_x, recv_meta = buf["recv_x"], buf["recv_meta"]
            dist.all_to_all_single(recv_x, send_x, group=self.group)
            dist.all_to_all_single(recv_meta, send_meta, group=self.group)
        return recv_x, recv_meta[:, 0], recv_meta[:, 1].view(torch.float32), position

    def pack_cuda(self, x: torch.Tensor, served_expert: torch.Tensor, served_weight: torch.Tensor):
        """``keepvq_ep_pack``: (send_x [rows, hidden], send_meta [rows, 2] = (local slot, weight
        bits), position [tokens, k] int32).  The tensors are cached per shape and overwritten by the
        next call."""
        from . import _lib

        tokens, k = served_expert.shape
        capacity = self.capacity or tokens * k
        rows = self.world * capacity
        x = x.contiguous()
        row_bytes = int(x.shape[1]) * x.element_size()
        key = ((tokens, k), int(x.shape[1]), x.dtype)
        buf = self._cuda_buffers.get(key)
        if buf is None:
            dev = x.device
            buf = self._cuda_buffers[key] = dict(
                send_x=torch.empty((rows, x.shape[1]), dtype=x.dtype, device=dev), recv_x=torch.empty((rows, x.shape[1]), dtype=x.dtype, device=dev),
                send_meta=torch.empty((rows, 2), dtype=torch.int32, device=dev), recv_meta=torch.empty((rows, 2), dtype=torch.int32, device=dev),
                position=torch.empty((tokens, k), dtype=torch.int32, device=dev))
        experts = served_expert.to(torch.int32).contiguous()
        weights = served_weight.contiguous().float()
        args = _lib.EpPackArgs(x=_lib.ptr(x), row_bytes=row_bytes, served_expert=_lib.ptr(experts), served_weight=_lib.ptr(weights),
                               tokens=tokens, top_k=k, world=self.world, experts_per_rank=self.experts_per_rank, capacity=capacity,
                               send_x=_lib.ptr(buf["send_x"]), send_meta=_lib.ptr(buf["send_meta"]), position=_lib.ptr(buf["position"]))
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().keepvq_ep_pack(args, _lib.stream_handle(x.device)), "keepvq_ep_pack")
        return buf["send_x"], buf["send_meta"], buf["position"]

    def _combine_cuda(self, back: torch.Tensor, position: torch.Tensor) -> torch.Tensor:
        from . import _lib

        tokens, k = position.shape
        back = back.contiguous()
        out = torch.empty((tokens, back.shape[1]), dtype=back.dtype, device=back.device)
        args = _lib.EpCombineArgs(back=_lib.ptr(back), dtype=_lib.dtype_tag(back.dtype), rows=int(back.shape[0]), hidden=int(back.shape[1]),
                                  position=_lib.ptr(position), tokens=tokens, top_k=k, out=_lib.ptr(out))
        with torch.cuda.device(back.device):
            _lib.check(_lib.load().keepvq_ep_combine(args, _lib.stream_handle(back.device)), "keepvq_ep_combine")
        return out

    def combine(self, y_routes: torch.Tensor, position: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """y_routes [world * capacity, hidden] (per received route) -> [tokens, hidden]: each token's
        picks summed in fp32 in pick order, one rounding."""
        if not y_routes.is_cuda:
            raise ValueError("RouteExchange works on CUDA tensors only")
        back = self._all_to_all(y_routes)
        if back.dtype != out_dtype:
            raise ValueError(f"the routes arrive as {back.dtype}; the sum over the picks is rounded to that dtype, not {out_dtype}")
        return self._combine_cuda(back, position)

    def _all_to_all(self, send: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return send
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv


class PeerExchange:
    """The same dispatch / combine without a collective in the data path: every rank writes its
    routes straight into the destination ranks' buffers over NVLink and a flag barrier with a
    bounded wait orders the phases (``keepvq_ep_dispatch_peer``, ``keepvq_ep_return_peer``).

    The buffers are ``torch.distributed._symmetric_memory`` allocations of a fixed shape
    (``tokens`` x ``top_k`` routes per rank, rows of ``hidden`` values of ``dtype``), made once;
    every rank must construct the exchange and call it in the same order.  One exchange serves
    any number of layers run back to back.  CUDA only, one process per GPU.
    """

    def __init__(self, experts_per_rank: int, *, tokens: int, top_k: int, hidden: int, dtype: torch.dtype, device: torch.device,
                 group=None, capacity: int | None = None, wait_spins: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.experts_per_rank, self.tokens, self.top_k, self.hidden, self.dtype = int(experts_per_rank), int(tokens), int(top_k), int(hidden), dtype
        self.capacity = int(capacity or tokens * top_k)
        rows = self.world * self.capacity
        self.row_bytes = hidden * torch.empty((), dtype=dtype).element_size()

        def shared(shape, dt):
            t = symm_mem.empty(*shape, dtype=dt, device=device)
            t.zero_()
            handle = symm_mem.rendezvous(t, self.group)
            return t, handle

        self.recv_x, hx = shared((rows, hidden), dtype)
        self.recv_meta, hm = shared((2, rows), torch.int32)  # slot plane, weight plane
        self.back, hb = shared((rows, hidden), dtype)
        self.flags, hf = shared((max(self.world, 32),), torch.int32)
        self._handles = (hx, hm, hb, hf)  # keep the mappings alive
        table = lambda h: torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=device)  # noqa: E731
        self._tables = tuple(table(h) for h in self._handles)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._arrivals = torch.zeros(1, dtype=torch.int32, device=device)  # finished blocks of the running exchange kernel
        self.position = torch.empty((tokens, top_k), dtype=torch.int32, device=device)
        self._peer = _lib.EpPeerArgs(world=self.world, rank=self.rank, capacity=self.capacity, row_bytes=self.row_bytes,
                                     recv_x=_lib.ptr(self._tables[0]), recv_meta=_lib.ptr(self._tables[1]), back=_lib.ptr(self._tables[2]),
                                     flags=_lib.ptr(self._tables[3]), epoch=_lib.ptr(self.epoch), status=_lib.ptr(self.status),
                                     wait_spins=int(wait_spins), arrivals=_lib.ptr(self._arrivals))
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # every rank's buffers are zeroed and mapped before anyone writes

    def dispatch(self, x: torch.Tensor, served_expert: torch.Tensor, served_weight: torch.Tensor):
        """-> (recv_x, recv_slot, recv_weight, position), as ``RouteExchange.dispatch``."""
        from . import _lib

        if tuple(served_expert.shape) != (self.tokens, self.top_k) or tuple(x.shape) != (self.tokens, self.hidden) or x.dtype != self.dtype:
            raise ValueError("this exchange was built for another shape or dtype")
        x = x.contiguous()
        experts = served_expert.to(torch.int32).contiguous()
        weights = served_weight.contiguous().float()
        args = _lib.EpPackArgs(x=_lib.ptr(x), row_bytes=self.row_bytes, served_expert=_lib.ptr(experts), served_weight=_lib.ptr(weights),
                               tokens=self.tokens, top_k=self.top_k, world=self.world, experts_per_rank=self.experts_per_rank,
                               capacity=self.capacity, send_x=None, send_meta=None, position=_lib.ptr(self.position))
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().keepvq_ep_dispatch_peer(args, self._peer, _lib.stream_handle(x.device)), "keepvq_ep_dispatch_peer")
        return self.recv_x, self.recv_meta[0], self.recv_meta[1].view(torch.float32), self.position

    def combine(self, y_routes: torch.Tensor, position: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        from . import _lib

        y = y_routes.contiguous()
        if y.dtype != self.dtype or out_dtype != self.dtype or tuple(y.shape) != tuple(self.recv_x.shape):
            raise ValueError("this exchange was built for another shape or dtype")
        with torch.cuda.device(y.device):
            _lib.check(_lib.load().keepvq_ep_return_peer(_lib.ptr(y), self._peer, _lib.stream_handle(y.device)), "keepvq_ep_return_peer")
        out = torch.empty((self.tokens, self.hidden), dtype=self.dtype, device=y.device)
        args = _lib.EpCombineArgs(back=_lib.ptr(self.back), dtype=_lib.dtype_tag(self.dtype), rows=int(self.back.shape[0]), hidden=self.hidden,
                                  position=_lib.ptr(position), tokens=self.tokens, top_k=self.top_k, out=_lib.ptr(out))
        with torch.cuda.device(y.device):
            _lib.check(_lib.load().keepvq_ep_combine(args, _lib.stream_handle(y.device)), "keepvq_ep_combine")
        return out

    def wait_expired(self) -> bool:
        """True when a barrier gave up waiting for a peer (results since then are invalid).  Reads
        one word back: synchronises the stream."""
        return bool(self.status.item())


class ExpertParallelLayer:
    """One routed MoE layer whose experts are sharded over the ranks of ``group``.

    ``local`` is a ``RoutedMoELayer`` built with ``top_k=1`` over this rank's shard of the experts
    (its router is not used); ``router_w`` is the full, replicated router.
    """

    def __init__(self, router_w: torch.Tensor, local, *, experts_per_rank: int, top_k: int, group=None, score_func: str = "softmax",
                 route_scale: float = 1.0, norm_topk_prob: bool = True, capacity: int | None = None, exchange=None):
        self.router_w, self.local = router_w.contiguous(), local
        self.top_k, self.score_func, self.route_scale, self.norm_topk_prob = top_k, score_func, route_scale, norm_topk_prob
        # `exchange`: a PeerExchange shared by the layers of a stack, or None for NCCL all-to-alls
        self.exchange = exchange if exchange is not None else RouteExchange(experts_per_rank, group=group, capacity=capacity)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import _lib
        from .router import routed_topk

        routing = routed_topk(x, self.router_w, top_k=self.top_k, score_func=self.score_func, route_scale=self.route_scale,
                              norm_topk_prob=self.norm_topk_prob)
        recv_x, recv_slot, recv_weight, position = self.exchange.dispatch(x, routing.served_expert, routing.served_weight)
        buf = self.local._buffers_for(int(recv_x.shape[0]), recv_x.dtype)
        r = buf["routing"]
        if recv_slot.is_contiguous() and recv_weight.is_contiguous():  # the peer exchange: the local layer reads the planes in place
            r.served_slot, r.served_weight = recv_slot.reshape(-1, 1), recv_weight.reshape(-1, 1)
        else:
            r.served_slot.copy_(recv_slot.reshape(-1, 1))
            r.served_weight.copy_(recv_weight.reshape(-1, 1))
        # by symmetry a rank receives about as many live routes as it sends; the rest of its rows are padding
        y, _ = self.local.decode(recv_x, stages=_lib.STAGE_ALL & ~_lib.STAGE_ROUTER, expected_routes=int(x.shape[0]) * self.top_k)
        return self.exchange.combine(y, position, x.dtype)
