"""The operators as PyTorch custom ops: ``torch.ops.keepvq.*`` exist, pass ``torch.library.opcheck``
(schema, fake implementation, dispatch), return what the plain Python operators return, and a
``torch.compile(fullgraph=True)`` wrapper around one decode layer traces without a graph break."""

import numpy as np
import pytest
import torch

from oracle import e8, router as oracle_router

pytestmark = pytest.mark.gpu


def make(cuda, experts=6, out=64, inp=256, seed=0):
    rng = np.random.default_rng(seed)
    codes = torch.from_numpy(rng.integers(0, 1 << 16, (experts, out, inp // 8), dtype=np.uint16)).to(cuda)
    scales = torch.from_numpy((0.02 * rng.uniform(0.5, 1.5, (experts, out, 1))).astype(np.float16)).to(cuda)
    return codes, scales


def test_every_operator_is_registered_and_passes_opcheck(cuda):
    from keep_b200 import kernels, torch_ops, vq, vq_switch

    ops = torch.ops.keepvq
    assert all(hasattr(ops, name) for name in torch_ops.OPS)
    table, res_table = vq.table_on(cuda, "e8p"), vq.table_on(cuda, "e8_1bit_half2")
    pair_table = torch.from_numpy(vq.pair_packed(vq.e8_1bit_packed()).view(np.int32)).to(cuda)
    codes, scales = make(cuda)
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.normal(size=(4, 256)).astype(np.float32)).to(cuda).to(torch.bfloat16)
    rhs = torch.from_numpy(rng.integers(0, 6, (4, 3)).astype(np.int32)).to(cuda)
    flat = rhs.reshape(-1)
    rows = x.repeat_interleave(3, dim=0)
    res_codes = torch.from_numpy(rng.integers(0, 256, (2, 64, 32), dtype=np.uint8)).to(cuda)
    res_scales = torch.full((2, 64, 1), 0.005, dtype=torch.float16, device=cuda)
    hot = torch.tensor([1, -1, -1, 0, -1, -1], dtype=torch.int32, device=cuda)
    lhs = torch.arange(12, dtype=torch.int32, device=cuda) // 3
    cases = {
        "vq_qmv": (x[0], codes[0], scales[0], table, 256, 64, 256, 16),
        "vq_qmm": (x, codes[0], scales[0], table, 256, 64, 256, 16),
        "e8p_m1_token_layout": (x, codes, scales, table, rhs, 64),
        "e8p_m1_per_route": (rows, codes, scales, table, flat, 64),
        "e8_1bit_m1_token_layout": (x, res_codes, res_scales, pair_table, rhs % 2, 64),
        "e8_1bit_m1_per_route": (rows, res_codes, res_scales, pair_table, flat % 2, 64),
        "e8p_nested_m1_token_layout": (x, codes, scales, table, rhs, res_codes, res_scales, res_table, hot, 64),
        "e8p_nested_m1_per_route": (rows, codes, scales, table, flat, res_codes, res_scales, res_table, hot, 64),
        "vq_switch_qmv": (x, codes, scales, table, rhs, 256, 64, 256, 16),
        "gather_vqmm": (x, codes, scales, table, rhs, None, 256, 64, 256, 16, False, "auto"),
        "gather_vqmm_sorted_routes": (x, codes, scales, table, flat.sort().values, lhs, 256, 64, 256, 16, False),
    }
    for name, args in cases.items():
        torch.library.opcheck(getattr(ops, name).default, args, test_utils=("test_schema", "test_faketensor", "test_aot_dispatch_static"))
    # the ops return what the plain operators return
    assert torch.equal(ops.gather_vqmm(*cases["gather_vqmm"]),
                       vq_switch.gather_vqmm(x, codes, scales, table, rhs, input_dims=256, output_dims=64, group_size=256, code_bits=16))
    assert torch.equal(ops.e8p_nested_m1_token_layout(*cases["e8p_nested_m1_token_layout"]),
                       kernels.e8p_nested_m1_token_layout(x, (codes, scales, table), rhs, (res_codes, res_scales, res_table), hot, output_dims=64))
    # with a lhs gather
    routed = ops.gather_vqmm(x, codes, scales, table, flat, lhs, 256, 64, 256, 16, False, "direct")
    assert tuple(routed.shape) == (12, 64)


def test_a_compiled_decode_layer_traces_without_a_graph_break(cuda):
    from keep_b200 import torch_ops  # noqa: F401  (registers the ops)

    rng = np.random.default_rng(5)
    experts, hidden, inter, top_k, tokens = 8, 512, 256, 2, 4
    w1, w3, w2 = make(cuda, experts, inter, hidden, 1), make(cuda, experts, inter, hidden, 2), make(cuda, experts, hidden, inter, 3)
    router_w = torch.from_numpy(rng.normal(scale=0.02, size=(experts, hidden)).astype(np.float32)).to(torch.bfloat16).to(cuda)
    x = torch.from_numpy(rng.normal(size=(tokens, hidden)).astype(np.float32)).to(torch.bfloat16).to(cuda)

    def layer(tok):
        out = torch.ops.keepvq.moe_decode_layer(tok, router_w, w1[0], w1[1], w3[0], w3[1], w2[0], w2[1], None, None, None, top_k, "softmax", 1.0, 0.3,
                                                1.0, True, 0.0)
        return out[0] + tok, out[1], out[0]  # something around the op, so the graph is more than the call

    args = (x, router_w, w1[0], w1[1], w3[0], w3[1], w2[0], w2[1], None, None, None, top_k, "softmax", 1.0, 0.3, 1.0, True, 0.0)
    torch.library.opcheck(torch.ops.keepvq.moe_decode_layer.default, args, test_utils=("test_schema", "test_faketensor", "test_aot_dispatch_static"))
    eager_out, eager_served, _ = layer(x)
    compiled = torch.compile(layer, fullgraph=True, backend="aot_eager")  # fullgraph: a graph break raises
    out, served, plain = compiled(x)
    assert torch.equal(out, eager_out) and torch.equal(served, eager_served)
    # and the result is the oracle's
    ref_route = oracle_router.routed_topk(x.cpu(), router_w.cpu(), None, None, None, top_k=top_k)
    assert np.array_equal(served.cpu().numpy(), ref_route["served_expert"].numpy())
    slots = ref_route["served_slot"].numpy()
    dense = {n: oracle_router.dense_slots(p[0].cpu().numpy(), p[1].cpu().numpy(), slots) for n, p in (("w1", w1), ("w3", w3), ("w2", w2))}
    ref = oracle_router.moe_layer(x.cpu(), slots, ref_route["served_weight"].numpy(), dense["w1"], dense["w3"], dense["w2"]).numpy()
    assert e8.relative_gap(plain.float().cpu().numpy(), ref) <= 1e-2
