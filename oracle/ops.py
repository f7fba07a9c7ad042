"""Operator-level oracle: dense decode then fp32/fp64 products, in numpy.

TEST INFRASTRUCTURE: the checker for the CUDA operators, never shipped or measured as product.

Follows the reference's own "reference" implementations and test oracles:

* ``vq_qmv_reference``   ``src/ramp/kernels/vq_qmv.py:126-160``  (decode_weight_matrix @ x, fp32)
* ``vq_qmm_reference``   ``src/ramp/kernels/vq_qmm.py:69-90``
* ``vq_switch_qmv``      ``src/ramp/ops/vq_switch.py:547-617``   (token vs per-route layouts)
* ``gather_vqmm``        ``src/ramp/ops/vq_switch.py:916-1221`` with ``implementation="reference"``
* ``nested_dense``       ``tests/test_e8p_nested_m1.py:22-37``   (base + residual of hot slots, fp64)
* ``dense_switch_glu``   ``tests/test_switch_routing.py:23-79``  (per-route SwiGLU over dense experts)
"""

from __future__ import annotations

import numpy as np

from .e8 import NO_RESIDUAL, decode_weight_matrix, e8_1bit_grid


def to_f32(x) -> np.ndarray:
    """Activations widened to float32 (bf16 arrives as ml_dtypes.bfloat16 or as a torch tensor)."""
    if hasattr(x, "detach"):
        x = x.detach().float().cpu().numpy()
    return np.asarray(x).astype(np.float32)


def vq_qmv_reference(x, codes, scales, codebook=None, *, code_bits=8) -> np.ndarray:
    """[in] -> [out] float32: the dense matrix is materialised on every call, as the reference does."""
    w = decode_weight_matrix(np.asarray(codes), np.asarray(scales).astype(np.float32), code_bits=code_bits, codebook=codebook)
    return (w @ to_f32(x)).astype(np.float32, copy=False)


def vq_qmm_reference(x, codes, scales, codebook=None, *, code_bits=8) -> np.ndarray:
    """[M, in] -> [M, out] float32."""
    w = decode_weight_matrix(np.asarray(codes), np.asarray(scales).astype(np.float32), code_bits=code_bits, codebook=codebook)
    return (to_f32(x) @ w.T).astype(np.float32, copy=False)


def dense_experts(codes, scales, *, code_bits=16, codebook=None, dtype=np.float32) -> np.ndarray:
    """[E, out, in/8] codes -> [E, out, in] weights."""
    codes = np.asarray(codes)
    scales = np.asarray(scales).astype(np.float32)
    return np.stack([decode_weight_matrix(codes[e], scales[e], code_bits=code_bits, codebook=codebook)
                     for e in range(codes.shape[0])]).astype(dtype)


def vq_switch_qmv(x, codes, scales, codebook, indices, *, code_bits=8, dense=None) -> np.ndarray:
    """x leading shape == indices.shape[:-1] -> [..., top_k, out]; == indices.shape -> [..., out]."""
    x = to_f32(x)
    idx = np.asarray(indices).astype(np.int64)
    experts = np.asarray(codes).shape[0]
    if idx.size and (idx.min() < 0 or idx.max() >= experts):
        raise ValueError(f"indices must be in [0, {experts}), found range [{idx.min()}, {idx.max()}]")
    if dense is None:
        dense = dense_experts(codes, scales, code_bits=code_bits, codebook=codebook)
    per_route = x.shape[:-1] == idx.shape
    flat_x = x.reshape(-1, x.shape[-1])
    if per_route:
        flat = idx.reshape(-1)
        out = np.stack([dense[e] @ flat_x[r] for r, e in enumerate(flat)]) if flat.size else np.zeros((0, dense.shape[1]), np.float32)
        return out.reshape(x.shape[:-1] + (dense.shape[1],)).astype(np.float32)
    top_k = idx.shape[-1]
    flat = idx.reshape(-1, top_k)
    out = np.stack([np.stack([dense[e] @ flat_x[t] for e in flat[t]]) for t in range(flat.shape[0])])
    return out.reshape(x.shape[:-1] + (top_k, dense.shape[1])).astype(np.float32)


def gather_vqmm(x, codes, scales, codebook, rhs_indices, *, lhs_indices=None, code_bits=8, dense=None) -> np.ndarray:
    """x [tokens, in], rhs [tokens, top_k] -> [tokens, top_k, out]; with lhs [routes] -> [routes, out]."""
    x = to_f32(x)
    rhs = np.asarray(rhs_indices).astype(np.int64)
    if dense is None:
        dense = dense_experts(codes, scales, code_bits=code_bits, codebook=codebook)
    if lhs_indices is None:
        return vq_switch_qmv(x, codes, scales, codebook, rhs, code_bits=code_bits, dense=dense)
    lhs = np.asarray(lhs_indices).astype(np.int64).reshape(-1)
    flat = rhs.reshape(-1)
    return np.stack([dense[e] @ x[r] for r, e in zip(lhs, flat)]).astype(np.float32)


def nested_dense(codes, scales, res_codes, res_scales, hot_of_slot, *, codebook=None) -> np.ndarray:
    """float64 [S, out, in]: base weights, plus the residual row of every slot that has one."""
    codes = np.asarray(codes)
    dense = dense_experts(codes, scales, code_bits=16, codebook=codebook, dtype=np.float64)
    res_codes = np.asarray(res_codes)
    rows, out, cw = res_codes.shape
    res = e8_1bit_grid().astype(np.float64)[res_codes].reshape(rows, out, cw * 8)
    rs = np.asarray(res_scales).astype(np.float64)
    res = res * np.repeat(rs, (cw * 8) // rs.shape[-1], axis=-1)
    for slot, h in enumerate(np.asarray(hot_of_slot).astype(np.int64) & 0xFFFFFFFF):
        if h != NO_RESIDUAL:
            dense[slot] += res[h]
    return dense


def silu(x):
    return x / (1.0 + np.exp(-x))


def dense_switch_glu(x, gate_w, up_w, down_w, indices) -> np.ndarray:
    """Per-route ``down(silu(gate x) * up x)`` over dense experts, float64: [..., top_k, hidden]."""
    x = np.asarray(x, dtype=np.float64)
    idx = np.asarray(indices).astype(np.int64)
    flat_x = x.reshape(-1, x.shape[-1])
    flat = idx.reshape(-1, idx.shape[-1])
    out = np.empty((flat.shape[0], flat.shape[1], down_w.shape[1]), dtype=np.float64)
    for t in range(flat.shape[0]):
        for j, e in enumerate(flat[t]):
            g = gate_w[e].astype(np.float64) @ flat_x[t]
            u = up_w[e].astype(np.float64) @ flat_x[t]
            out[t, j] = down_w[e].astype(np.float64) @ (silu(g) * u)
    return out.reshape(idx.shape + (down_w.shape[1],))
