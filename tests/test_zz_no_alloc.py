"""The layer entry point that allocates nothing (``keepvq_moe_decode_layer_static``).

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  It must pass alone in a fresh process and after the rest of the suite.

The entry point serves hosts that cannot allocate device memory when a token arrives, because all
of it already sits in their own pool or because an allocation would stall the device.  Its scratch
is a fixed array inside the library.  The test calls it through the C ABI, twice in a row on
different tokens (the array keeps the first call's contents, which must not leak into the second),
and checks each result against the regular entry point, which works in caller-provided scratch.
"""

import numpy as np
import pytest
import torch

import synthetic
from oracle import e8

pytestmark = pytest.mark.gpu
TOLERANCE = 1e-2  # the layer's stated bf16 tolerance; the two entry points in fact agree bit for bit


def layer_on(cuda, cfg, **kw):
    from keep_b200 import moe

    def proj(name):
        codes, scales = cfg[name]
        return moe.Projection(torch.from_numpy(codes).to(cuda), torch.from_numpy(scales).to(cuda))

    return moe.RoutedMoELayer(cfg["router"].to(cuda), proj("w1"), proj("w3"), proj("w2"), **kw)


def empty_routing(cuda, tokens, k):
    from keep_b200.router import Routing

    i32 = lambda: torch.empty((tokens, k), dtype=torch.int32, device=cuda)  # noqa: E731
    f32 = lambda: torch.empty((tokens, k), dtype=torch.float32, device=cuda)  # noqa: E731
    return Routing(served_expert=i32(), served_slot=i32(), served_weight=f32(), want=i32(), want_score=f32(), admit=i32())


@pytest.mark.parametrize("hidden,inter,path", [(512, 256, "tensor"), (256, 128, "general")])
def test_two_calls_in_a_row_match_the_regular_entry_point(cuda, hidden, inter, path):
    cfg = synthetic.layer(seed=31, experts=10, hidden=hidden, inter=inter)
    layer = layer_on(cuda, cfg, top_k=3)
    assert layer.kernel_path == path
    for call, tokens in enumerate((7, 4)):  # a different token count second time: stale scratch must not matter
        x = synthetic.tokens(40 + call, tokens, hidden).to(cuda)
        want, want_routing = layer.decode(x)
        want, want_slots = want.clone(), want_routing.served_slot.clone()
        out = torch.full_like(x, float("nan"))
        routing = empty_routing(cuda, tokens, 3)
        got, got_routing = layer.decode_without_scratch(x, out, routing)
        torch.cuda.synchronize()
        assert torch.equal(got_routing.served_slot, want_slots)
        assert torch.isfinite(got.float()).all()
        gap = e8.relative_gap(got.float().cpu().numpy(), want.float().cpu().numpy())
        assert gap <= TOLERANCE, gap
        assert torch.equal(got, want), "same kernels, same inputs: the results should be identical"


def test_a_request_beyond_the_built_in_scratch_is_refused(cuda):
    from keep_b200 import _lib

    cfg = synthetic.layer(seed=32, experts=6, hidden=1024, inter=512)
    layer = layer_on(cuda, cfg, top_k=3)
    tokens = 600  # needs well over 8 MiB of scratch at this shape
    lib = _lib.load()
    assert lib.keepvq_moe_layer_workspace_bytes(tokens, 1024, 512, 6, 3) > _lib.STATIC_SCRATCH_BYTES
    x = synthetic.tokens(50, tokens, 1024).to(cuda)
    with pytest.raises(_lib.KeepVQError, match="too small"):
        layer.decode_without_scratch(x, torch.empty_like(x), empty_routing(cuda, tokens, 3))
