"""The fused decode layer against the CPU oracle: routing exact, outputs within the stated bf16
tolerance (max|got - want| / max|want| <= 1e-2), cosine similarity reported."""

import numpy as np
import pytest
import torch

import synthetic
from oracle import e8, router as oracle_router

pytestmark = pytest.mark.gpu
TOLERANCE = 1e-2  # max relative gap the path promises for bf16 activations


def build_layer(cuda, cfg, **kw):
    from keep_b200 import moe

    def proj(name, res=None):
        codes, scales = cfg[name]
        rc, rs = (None, None) if res is None else res[name]
        dev = lambda a: None if a is None else torch.from_numpy(a).to(cuda)  # noqa: E731
        return moe.Projection(dev(codes), dev(scales), dev(rc), dev(rs))

    res = kw.pop("res", None)
    return moe.RoutedMoELayer(cfg["router"].to(cuda), proj("w1", res), proj("w3", res), proj("w2", res), **kw)


def check_layer(cfg, x, out, routing, *, top_k, served_bias=None, pool_bias=None, slot_of=None, res=None, hot_of_slot=None,
                **router_kw):
    want = oracle_router.routed_topk(x, cfg["router"], served_bias, pool_bias, slot_of, top_k=top_k, **router_kw)
    assert oracle_router.min_cut_gap(want["served_keys"], top_k) > 0
    np.testing.assert_array_equal(routing.served_expert.cpu().numpy(), want["served_expert"].numpy())
    np.testing.assert_array_equal(routing.served_slot.cpu().numpy(), want["served_slot"].numpy())
    np.testing.assert_array_equal(routing.want.cpu().numpy(), want["want"].numpy())
    np.testing.assert_array_equal(routing.admit.cpu().numpy(), want["admit"].numpy())
    np.testing.assert_allclose(routing.served_weight.cpu().numpy(), want["served_weight"].numpy(), rtol=2e-5)
    slots = want["served_slot"].numpy()
    dense = {n: oracle_router.dense_slots(*cfg[n], slots, res=None if res is None else res[n], hot_of_slot=hot_of_slot)
             for n in ("w1", "w3", "w2")}
    ref = oracle_router.moe_layer(x, slots, want["served_weight"].numpy(), dense["w1"], dense["w3"], dense["w2"])
    got = out.float().cpu().numpy()
    gap, cos = e8.relative_gap(got, ref.numpy()), e8.cosine_similarity(got, ref.numpy())
    print(f"layer output: relative gap {gap:.3e}, cosine {cos:.8f}")
    assert gap <= TOLERANCE and cos >= 0.9999
    return gap, cos


@pytest.mark.parametrize("tokens", [1, 5])
def test_small_layer_all_resident(cuda, tokens):
    cfg = synthetic.layer(seed=2, experts=12, hidden=256, inter=128)
    x = synthetic.tokens(3 + tokens, tokens, 256)
    layer = build_layer(cuda, cfg, top_k=3)
    out, routing = layer.decode(x.to(cuda))
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (tokens, 256)
    check_layer(cfg, x, out, routing, top_k=3)


def test_small_layer_grouped_scales_and_fp16(cuda):
    cfg = synthetic.layer(seed=4, experts=10, hidden=512, inter=256, group_hidden=64, group_inter=128)
    x = synthetic.tokens(9, 4, 512)
    layer = build_layer(cuda, cfg, top_k=4, score_func="sqrtsoftplus", route_scale=1.5)
    out, routing = layer.decode(x.to(cuda))
    check_layer(cfg, x, out, routing, top_k=4, score_func="sqrtsoftplus", route_scale=1.5)


def test_residency_mask_and_nested_residual(cuda):
    """Half the pool resident, a residual tier on some slots, admissions at tau = 0.3."""
    rng = np.random.default_rng(8)
    pool, slots, hidden, inter, k = 16, 8, 256, 128, 3
    cfg = synthetic.layer(seed=6, experts=pool, hidden=hidden, inter=inter)
    resident = np.sort(rng.choice(pool, slots, replace=False))
    slot_of = np.full(pool, 0xFFFFFFFF, dtype=np.uint32)
    slot_of[resident] = rng.permutation(slots).astype(np.uint32)
    served_bias = np.full(pool, oracle_router.OFF, dtype=np.float32)
    served_bias[resident] = 0.0
    slot_cfg = dict(cfg)  # weight arrays are indexed by slot: slot s holds expert resident-of-slot
    expert_of_slot = np.empty(slots, dtype=np.int64)
    expert_of_slot[slot_of[resident].astype(np.int64)] = resident
    for n in ("w1", "w3", "w2"):
        slot_cfg[n] = (cfg[n][0][expert_of_slot], cfg[n][1][expert_of_slot])
    res = synthetic.residual_tier(7, 3, hidden, inter)
    hot_of_slot = np.full(slots, 0xFFFFFFFF, dtype=np.uint32)
    hot_of_slot[[1, 4, 6]] = [2, 0, 1]
    x = synthetic.tokens(10, 6, hidden)
    layer = build_layer(cuda, slot_cfg, top_k=k, served_bias=served_bias, slot_of=slot_of, hot_of_slot=hot_of_slot, res=res, tau=0.3)
    out, routing = layer.decode(x.to(cuda))
    check_layer(slot_cfg, x, out, routing, top_k=k, served_bias=served_bias, slot_of=slot_of, res=res, hot_of_slot=hot_of_slot, tau=0.3)
    assert (routing.admit.cpu().numpy() >= 0).any(), "seed should produce at least one admission"


@pytest.mark.parametrize("tokens", [20, 6])  # 60 routes and 18 routes: the slab kernel and its split form, both with the residual pass
def test_nested_residual_at_tensor_core_shapes(cuda, tokens):
    """Half the pool resident, three hot slots with the 8-bit residual, shapes the int8 kernels take."""
    rng = np.random.default_rng(18)
    pool, slots, hidden, inter, k = 16, 8, 512, 256, 3
    cfg = synthetic.layer(seed=16, experts=pool, hidden=hidden, inter=inter)
    resident = np.sort(rng.choice(pool, slots, replace=False))
    slot_of = np.full(pool, 0xFFFFFFFF, dtype=np.uint32)
    slot_of[resident] = rng.permutation(slots).astype(np.uint32)
    served_bias = np.full(pool, oracle_router.OFF, dtype=np.float32)
    served_bias[resident] = 0.0
    expert_of_slot = np.empty(slots, dtype=np.int64)
    expert_of_slot[slot_of[resident].astype(np.int64)] = resident
    slot_cfg = dict(cfg)
    for n in ("w1", "w3", "w2"):
        slot_cfg[n] = (cfg[n][0][expert_of_slot], cfg[n][1][expert_of_slot])
    res = synthetic.residual_tier(17, 3, hidden, inter)
    hot_of_slot = np.full(slots, 0xFFFFFFFF, dtype=np.uint32)
    hot_of_slot[[0, 3, 7]] = [1, 2, 0]
    x = synthetic.tokens(19 + tokens, tokens, hidden)
    layer = build_layer(cuda, slot_cfg, top_k=k, served_bias=served_bias, slot_of=slot_of, hot_of_slot=hot_of_slot, res=res, tau=0.3)
    assert layer.kernel_path == "tensor"
    out, routing = layer.decode(x.to(cuda))
    check_layer(slot_cfg, x, out, routing, top_k=k, served_bias=served_bias, slot_of=slot_of, res=res, hot_of_slot=hot_of_slot, tau=0.3)
    # the residual does change the answer: without it the same call misses the oracle
    plain = build_layer(cuda, slot_cfg, top_k=k, served_bias=served_bias, slot_of=slot_of, tau=0.3)
    base_only, _ = plain.decode(x.to(cuda))
    assert not torch.equal(base_only, out)


def test_fewer_residents_than_top_k_leaves_dead_picks_at_zero(cuda):
    cfg = synthetic.layer(seed=11, experts=6, hidden=128, inter=64)
    served_bias = np.array([0, oracle_router.OFF, oracle_router.OFF, 0, oracle_router.OFF, oracle_router.OFF], dtype=np.float32)
    x = synthetic.tokens(12, 3, 128)
    layer = build_layer(cuda, cfg, top_k=3, served_bias=served_bias, slot_of=np.arange(6, dtype=np.uint32))
    out, routing = layer.decode(x.to(cuda))
    assert ((routing.served_slot.cpu().numpy() >= 0).sum(-1) == 2).all()
    check_layer(cfg, x, out, routing, top_k=3, served_bias=served_bias, slot_of=np.arange(6))


@pytest.mark.parametrize("tokens", [3, 30, 400])  # the sweep kernel, the slab kernel, the tcgen05 kernel
def test_dead_picks_at_tensor_core_shapes(cuda, tokens):
    """Two residents, top-3: every token has a pick without a slot, which must add nothing,
    whichever of the grouped kernels runs (they never touch the rows of such routes)."""
    cfg = synthetic.layer(seed=13, experts=6, hidden=512, inter=256)
    served_bias = np.array([0, oracle_router.OFF, oracle_router.OFF, 0, oracle_router.OFF, oracle_router.OFF], dtype=np.float32)
    x = synthetic.tokens(14 + tokens, tokens, 512)
    layer = build_layer(cuda, cfg, top_k=3, served_bias=served_bias, slot_of=np.arange(6, dtype=np.uint32))
    assert layer.kernel_path == "tensor"
    # poison the scratch so that an untouched row cannot pass as zeros by luck
    layer.decode(x.to(cuda))
    for buf in layer._buffers.values():
        buf["workspace"].fill_(0x7F)
    out, routing = layer.decode(x.to(cuda))
    assert ((routing.served_slot.cpu().numpy() >= 0).sum(-1) == 2).all()
    check_layer(cfg, x, out, routing, top_k=3, served_bias=served_bias, slot_of=np.arange(6))


@pytest.mark.parametrize("tokens,experts,top_k,group", [(3, 12, 3, None), (20, 4, 3, 256), (9, 6, 2, 256)])
def test_tensor_core_path_small_shapes(cuda, tokens, experts, top_k, group):
    """Shapes the int8 tensor-core kernels accept (input dims multiples of 256), with grouped scales
    and with more than eight routes on one expert (20 tokens x top-3 over 4 experts)."""
    cfg = synthetic.layer(seed=21, experts=experts, hidden=512, inter=256, group_hidden=group, group_inter=group)
    x = synthetic.tokens(22 + tokens, tokens, 512)
    layer = build_layer(cuda, cfg, top_k=top_k)
    assert layer.kernel_path == "tensor"
    out, routing = layer.decode(x.to(cuda))
    check_layer(cfg, x, out, routing, top_k=top_k)


def test_tensor_and_general_kernels_agree(cuda):
    """The same layer through both kernel sets: routing identical, outputs within the tolerance."""
    cfg = synthetic.layer(seed=23, experts=8, hidden=512, inter=256)
    x = synthetic.tokens(24, 7, 512).to(cuda)
    fast = build_layer(cuda, cfg, top_k=4)
    general = build_layer(cuda, cfg, top_k=4)
    general.codebook_all_odd = False  # forces the general kernels
    assert (fast.kernel_path, general.kernel_path) == ("tensor", "general")
    a, ra = fast.decode(x)
    b, rb = general.decode(x)
    assert torch.equal(ra.served_slot, rb.served_slot)
    assert e8.relative_gap(a.float().cpu().numpy(), b.float().cpu().numpy()) <= TOLERANCE


@pytest.mark.parametrize("tokens,experts,top_k", [(300, 8, 4), (1100, 5, 1)])
def test_many_routes_per_expert_take_the_tcgen05_kernels(cuda, tokens, experts, top_k):
    """From 1024 routes on, the layer runs the tcgen05 (int8, tensor memory) kernels: experts with
    more routes than one 128-column item, ragged last items, and an expert nobody picks."""
    cfg = synthetic.layer(seed=41, experts=experts, hidden=512, inter=256)
    cfg["router"][experts - 1] = -1.0  # bf16 rows of -1: this expert's logits sink, nobody routes to it
    x = synthetic.tokens(42, tokens, 512).abs()
    layer = build_layer(cuda, cfg, top_k=top_k)
    assert layer.kernel_path == "tensor" and tokens * top_k >= 1024
    out, routing = layer.decode(x.to(cuda))
    served = routing.served_expert.cpu().numpy()
    assert (served != experts - 1).all()
    assert not layer.wait_expired(tokens, x.dtype)  # no bounded wait of the tcgen05 kernels gave up
    check_layer(cfg, x, out, routing, top_k=top_k)


def test_many_routes_spread_over_many_experts_stay_on_the_decode_kernels(cuda):
    """1200 routes over 64 experts (under 24 per expert on average): the mma.sync kernels, with
    several 8-route groups per expert."""
    cfg = synthetic.layer(seed=43, experts=64, hidden=512, inter=256)
    x = synthetic.tokens(44, 400, 512)
    layer = build_layer(cuda, cfg, top_k=3)
    assert layer.kernel_path == "tensor"
    out, routing = layer.decode(x.to(cuda))
    check_layer(cfg, x, out, routing, top_k=3)


@pytest.mark.parametrize("tokens", [2, 10])
def test_shipped_artifact_shape_with_grouped_scales(cuda, tokens):
    """The shape and scale groups of the reference's shipped artifacts: hidden 5120 in groups of
    512, inter 2304 in groups of 256 (keep_quant.py:13-15).  Two tokens run the sweep kernel (20
    and 9 chunks of inputs over its 16 and 8 k parts, several scale groups per row); ten tokens x
    top-6 run the split slab kernel with eight and two scale groups per row."""
    cfg = synthetic.layer(seed=31, experts=10, hidden=5120, inter=2304, group_hidden=512, group_inter=256)
    x = synthetic.tokens(32 + tokens, tokens, 5120)
    layer = build_layer(cuda, cfg, top_k=6)
    assert layer.kernel_path == "tensor"
    out, routing = layer.decode(x.to(cuda))
    check_layer(cfg, x, out, routing, top_k=6)


@pytest.mark.parametrize("batch", [1, 16])
def test_config2_shape_decode_layer(cuda, batch):
    """The benchmark layer shape (hidden 4096, inter 2048, top-6, softmax) on a 48-expert slice of
    the pool so the CPU oracle finishes in seconds; tokens bf16 N(0,1), seed 1 + batch."""
    cfg = synthetic.layer(seed=0, experts=48)
    x = synthetic.tokens(1 + batch, batch, 4096)
    layer = build_layer(cuda, cfg, top_k=6)
    out, routing = layer.decode(x.to(cuda))
    check_layer(cfg, x, out, routing, top_k=6)


def test_a_wait_that_nothing_satisfies_runs_out_and_the_kernel_returns(cuda):
    """The tcgen05 kernel's waits are bounded by a deadline on the GPU's timer.  The library's
    self-test launches one block whose activation producers never publish their tiles: the MMA
    issuer's wait must expire after the 2 ms it is given, the block must report (status word 1),
    free its tensor memory and return, and the device must answer afterwards.  No fault, no
    endless loop: the failure is a flag that nothing sets."""
    from keep_b200 import _lib, vq

    lib = _lib.load()
    nbytes = int(lib.keepvq_wait_selftest_workspace_bytes())
    ws = torch.full((nbytes,), 0x5A, dtype=torch.uint8, device=cuda)
    with torch.cuda.device(cuda):
        _lib.check(lib.keepvq_wait_selftest(_lib.ptr(ws), nbytes, 2_000_000, _lib.stream_handle(cuda)), "keepvq_wait_selftest")
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == 1
    # the context still answers, and tensor memory was handed back: a real tcgen05 call runs right after
    codes = torch.zeros((1, 128, 16), dtype=torch.uint16, device=cuda)
    grid = vq.decode_weight_matrix(codes[0], torch.ones((128, 1), dtype=torch.float16, device=cuda), code_bits=16)
    assert torch.isfinite(grid).all()
    assert lib.keepvq_wait_selftest(_lib.ptr(ws), nbytes, 0, _lib.stream_handle(cuda)) == -2  # a deadline is mandatory (and at most a second)


@pytest.mark.parametrize("tokens,hidden,inter", [(1, 256, 128), (7, 512, 256), (300, 512, 256)])
def test_shared_expert_joins_the_routed_sum_before_the_one_rounding(cuda, tokens, hidden, inter):
    """``decode(x, shared=s)``: out = bf16(sum over the picks of the routes' bf16 outputs, in pick
    order, + s), fp32 throughout (scripts/v41_build/omlx_lattice.py:372-389 rounds once, after the
    shared down kernel has added the routed sum).  Checked to the bit against the routes' outputs
    the call leaves in its scratch; the dense shared expert itself against fp32 torch."""
    from keep_b200 import moe

    cfg = synthetic.layer(seed=31, experts=8, hidden=hidden, inter=inter)
    x = synthetic.tokens(32 + tokens, tokens, hidden).to(cuda)
    layer = build_layer(cuda, cfg, top_k=3, swiglu_limit=7.0)
    gen = torch.Generator().manual_seed(5)
    w1, w3 = (torch.randn((inter, hidden), generator=gen).mul(hidden ** -0.5).to(torch.bfloat16).to(cuda) for _ in range(2))
    w2 = torch.randn((hidden, inter), generator=gen).mul(inter ** -0.5).to(torch.bfloat16).to(cuda)
    expert = moe.SharedExpert(w1, w3, w2, swiglu_limit=7.0)
    s = expert(x)
    assert s.dtype == torch.float32 and tuple(s.shape) == (tokens, hidden)
    gate, up = x.float() @ w1.float().t(), x.float() @ w3.float().t()
    h = (torch.nn.functional.silu(gate.clamp(max=7.0)) * up.clamp(-7.0, 7.0)).to(torch.bfloat16).float()
    want_s = h @ w2.float().t()
    assert e8.relative_gap(s.cpu().numpy(), want_s.cpu().numpy()) <= 1e-2

    plain = layer.decode(x)[0].clone()
    out, _ = layer.decode(x, shared=s)
    routes = layer.route_outputs(tokens, torch.bfloat16).float().view(tokens, 3, hidden)
    total = torch.zeros((tokens, hidden), dtype=torch.float32, device=cuda)
    for j in range(3):
        total = total + routes[:, j]
    assert torch.equal(plain, total.to(torch.bfloat16))
    assert torch.equal(out, (total + s).to(torch.bfloat16))
    with pytest.raises(ValueError, match="shared must be"):
        layer.decode(x, shared=s.to(torch.bfloat16))
