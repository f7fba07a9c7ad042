"""The holder classes (QuantizedVQSwitchLinear, QuantizedVQSwitchGLU) against the oracle.

Mirrors tests/test_switch_linear.py and tests/test_glm4_moe_adapter.py of the reference in what
they check of the routed path: both call layouts, bias and the continuous sidecars, constructor
errors, and the GLU composition (fused kernels and the composed fallback)."""

import numpy as np
import pytest
import torch

import synthetic
from oracle import e8, ops

pytestmark = pytest.mark.gpu


def dense(codes, scales):
    return ops.dense_experts(codes, scales, code_bits=16)


def linear(cuda, codes, scales, **kw):
    from keep_b200.switch import QuantizedVQSwitchLinear

    experts, out, cw = codes.shape
    group = cw * 8 // scales.shape[2]
    return QuantizedVQSwitchLinear(input_dims=cw * 8, output_dims=out, num_experts=experts, codes=torch.from_numpy(codes).to(cuda),
                                   scales=torch.from_numpy(scales).to(cuda), group_size=group, code_bits=16, **kw)


@pytest.mark.parametrize("tokens,top_k", [(3, 2), (70, 4)])  # the few-token kernel, and the sorted grouped path
def test_linear_token_and_per_route_layouts(cuda, tokens, top_k):
    rng = np.random.default_rng(70 + tokens)
    codes, scales = synthetic.projection(rng, 6, 48, 256, group=64)
    layer = linear(cuda, codes, scales)
    x = rng.normal(size=(tokens, 256)).astype(np.float32)
    idx = np.stack([rng.choice(6, top_k, replace=False) for _ in range(tokens)]).astype(np.int64)
    want = ops.gather_vqmm(x, codes, scales, None, idx, code_bits=16)
    got = layer(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda))
    assert tuple(got.shape) == (tokens, top_k, 48) and got.dtype == torch.float32
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-3)
    # one activation row per route
    xr = rng.normal(size=(tokens, top_k, 256)).astype(np.float32)
    want = ops.vq_switch_qmv(xr, codes, scales, None, idx, code_bits=16)
    got = layer(torch.from_numpy(xr).to(cuda), torch.from_numpy(idx).to(cuda))
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-3)
    assert layer.route_backend == "gather_vqmm_auto" and not layer.has_continuous_sidecar and not layer.has_sparse_residual_rows


def test_linear_bias_and_continuous_sidecars(cuda):
    rng = np.random.default_rng(72)
    codes, scales = synthetic.projection(rng, 5, 24, 128, group=32)
    bias = rng.normal(size=(5, 24)).astype(np.float32)
    delta = (0.1 * rng.normal(size=scales.shape)).astype(np.float32)
    out_bias = rng.normal(size=(5, 24)).astype(np.float32)
    layer = linear(cuda, codes, scales, bias=torch.from_numpy(bias).to(cuda), continuous_scale_delta=torch.from_numpy(delta).to(cuda),
                   continuous_output_bias=torch.from_numpy(out_bias).to(cuda))
    assert layer.has_continuous_sidecar
    x = rng.normal(size=(4, 128)).astype(np.float32)
    idx = rng.integers(0, 5, (4, 2))
    eff = scales.astype(np.float32) * np.exp(delta)
    want = ops.gather_vqmm(x, codes, eff, None, idx, code_bits=16) + bias[idx] + out_bias[idx]
    got = layer(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda))
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-3)
    np.testing.assert_allclose(layer.effective_scales().cpu().numpy(), eff, rtol=1e-6)


def test_constructor_errors(cuda):
    from keep_b200.switch import QuantizedVQSwitchGLU, QuantizedVQSwitchLinear

    rng = np.random.default_rng(73)
    codes, scales = synthetic.projection(rng, 4, 16, 64, group=32)
    c, s = torch.from_numpy(codes).to(cuda), torch.from_numpy(scales).to(cuda)
    ok = dict(input_dims=64, output_dims=16, num_experts=4, codes=c, scales=s, group_size=32, code_bits=16)
    for change, message in ((dict(input_dims=0), "must be positive"), (dict(input_dims=60), "divisible by 8"),
                            (dict(group_size=48), "divisible by group_size"), (dict(code_bits=4), "code_bits must be 8 or 16"),
                            (dict(gather_codebook_duplication=2), "must be 1, 4, or 8"), (dict(route_strategy="fast"), "route_strategy"),
                            (dict(num_experts=5), "codes must have shape"), (dict(scales=s[:, :, :1]), "scales must have shape")):
        with pytest.raises(ValueError, match=message):
            QuantizedVQSwitchLinear(**{**ok, **change})
    with pytest.raises(NotImplementedError):
        QuantizedVQSwitchLinear(**ok, rht_signs=torch.ones(64, device=cuda))
    gate = QuantizedVQSwitchLinear(**ok)
    other, other_s = synthetic.projection(rng, 4, 64, 16, group=16)
    down = QuantizedVQSwitchLinear(input_dims=16, output_dims=64, num_experts=4, codes=torch.from_numpy(other).to(cuda),
                                   scales=torch.from_numpy(other_s).to(cuda), group_size=16, code_bits=16)
    with pytest.raises(ValueError, match="down_proj input dimension"):
        QuantizedVQSwitchGLU(gate_proj=gate, up_proj=gate, down_proj=gate)
    with pytest.raises(ValueError, match="prefill_engine"):
        QuantizedVQSwitchGLU(gate_proj=gate, up_proj=gate, down_proj=down, prefill_engine="cuda")


@pytest.mark.parametrize("tokens,limit", [(5, 0.0), (40, 0.0), (9, 1.5)])
def test_glu_fused_and_composed_match_the_dense_oracle(cuda, tokens, limit):
    from keep_b200.switch import QuantizedVQSwitchGLU, limited_swiglu

    cfg = synthetic.layer(seed=74, experts=6, hidden=512, inter=256)
    x = synthetic.tokens(75 + tokens, tokens, 512)
    rng = np.random.default_rng(76)
    idx = np.stack([rng.choice(6, 3, replace=False) for _ in range(tokens)]).astype(np.int64)
    w1, w3, w2 = (dense(*cfg[n]) for n in ("w1", "w3", "w2"))
    if limit:
        want = np.empty((tokens, 3, 512))
        xf = x.float().numpy().astype(np.float64)
        for t in range(tokens):
            for j, e in enumerate(idx[t]):
                g, u = np.minimum(w1[e] @ xf[t], limit), np.clip(w3[e] @ xf[t], -limit, limit)
                want[t, j] = w2[e] @ (ops.silu(g) * u)
    else:
        want = ops.dense_switch_glu(x.float().numpy(), w1, w3, w2, idx)
    act = limited_swiglu(limit) if limit else None
    fused = QuantizedVQSwitchGLU(gate_proj=linear(cuda, *cfg["w1"]), up_proj=linear(cuda, *cfg["w3"]), down_proj=linear(cuda, *cfg["w2"]), activation=act)
    got = fused(x.to(cuda), torch.from_numpy(idx).to(cuda))
    assert fused._fused_layer(3) is not None and tuple(got.shape) == (tokens, 3, 512) and got.dtype == torch.bfloat16
    assert e8.relative_gap(got.float().cpu().numpy(), want) <= 1e-2
    # a bias on one projection takes the composed path (three operator calls, activation in torch)
    zero = torch.zeros((6, 512), device=cuda)
    composed = QuantizedVQSwitchGLU(gate_proj=linear(cuda, *cfg["w1"]), up_proj=linear(cuda, *cfg["w3"]),
                                    down_proj=linear(cuda, *cfg["w2"], bias=zero), activation=act)
    got2 = composed(x.to(cuda), torch.from_numpy(idx).to(cuda))
    assert composed._fused_layer(3) is None
    assert e8.relative_gap(got2.float().cpu().numpy(), want) <= 1e-2


def test_switch_linear_from_a_safetensors_checkpoint(cuda, tmp_path):
    """<prefix>.codes / .scales with the codebook named by hash in the metadata -> a working holder."""
    import json

    from safetensors.torch import save_file

    from keep_b200 import io as layer_io, vq

    rng = np.random.default_rng(80)
    codes, scales = synthetic.projection(rng, 5, 40, 256, group=64)
    prefix = "model.layers.3.mlp.switch_mlp.gate_proj"
    config = {"quant_method": "mlx_vq_e8", "version": 1, "default_code_bits": 16, "default_group_size": 64,
              "codebook": {"name": "quip_e8p", "dtype": "uint32", "entries": 256, "sha256": vq.E8P_PACKED_ABS_SHA256}}
    tensors = {f"{prefix}.codes": torch.from_numpy(codes), f"{prefix}.scales": torch.from_numpy(scales)}
    save_file(tensors, str(tmp_path / "model.safetensors"), metadata={"quantization_config": json.dumps(config)})
    layer = layer_io.load_quantized_vq_switch_linear(tmp_path / "model.safetensors", prefix, cuda)
    assert (layer.input_dims, layer.output_dims, layer.num_experts, layer.group_size, layer.code_bits) == (256, 40, 5, 64, 16)
    x = rng.normal(size=(3, 256)).astype(np.float32)
    idx = rng.integers(0, 5, (3, 2))
    got = layer(torch.from_numpy(x).to(cuda), torch.from_numpy(idx).to(cuda))
    np.testing.assert_allclose(got.cpu().numpy(), ops.gather_vqmm(x, codes, scales, None, idx, code_bits=16), rtol=1e-4, atol=1e-3)
    config["codebook"]["sha256"] = "0" * 64
    save_file(tensors, str(tmp_path / "other.safetensors"), metadata={"quantization_config": json.dumps(config)})
    with pytest.raises(ValueError, match="not supported by this runtime"):
        layer_io.load_quantized_vq_switch_linear(tmp_path / "other.safetensors", prefix, cuda)
    with pytest.raises(KeyError, match="missing tensor"):
        layer_io.load_quantized_vq_switch_linear(tmp_path / "model.safetensors", "model.layers.4.x", cuda)
