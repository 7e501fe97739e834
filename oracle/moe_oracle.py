"""CPU oracle for the routed-MoE expert path (numpy). TEST INFRASTRUCTURE ONLY.

Restates reference/python/moe.py:7-26 (the whole-layer forward with its BF16
rounding points) and the activation of kernels/moe/swiglu.cu:12-26. Parity
status: PINNED against an output of the reference Python frozen in
tests/golden/moe_bf16.npz (floating point: compared within BF16 rounding).
"""
from __future__ import annotations

import numpy as np

from .nvfp4_oracle import bf16_to_f32, f32_to_bf16_bits


def round_bf16(x: np.ndarray) -> np.ndarray:
    """FP32 -> nearest-even BF16 -> FP32."""
    return bf16_to_f32(f32_to_bf16_bits(np.asarray(x, dtype=np.float32)))


def swiglu(gate_up: np.ndarray, route_weight: np.ndarray, clamp: float) -> np.ndarray:
    """bf16(silu(min(g, c)) * clamp(u, -c, c) * w) with g = first half, u = second half.

    reference/python/moe.py:21-23; kernels/moe/swiglu.cu:20-24.
    """
    inter = gate_up.shape[-1] // 2
    g = np.minimum(gate_up[..., :inter], np.float32(clamp)).astype(np.float32)
    u = np.clip(gate_up[..., inter:], np.float32(-clamp), np.float32(clamp)).astype(np.float32)
    silu = (g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))).astype(np.float32)
    return round_bf16(silu * u * route_weight[..., None].astype(np.float32))


def moe_forward(x, expert_ids, route_weights, w1, w2, clamp=10.0):
    """x [T,H] f32 (bf16-representable), ids [T,k] global, weights [T,k] f32,
    w1 [E,2I,H], w2 [E,H,I] f32 -> y [T,H] f32 (bf16-representable).

    Per expert in ascending order: gate_up -> bf16, activation -> bf16, expert
    output -> bf16, FP32 accumulation per token, final bf16 (moe.py:13-26).
    """
    tokens, hidden = x.shape
    out = np.zeros((tokens, hidden), dtype=np.float32)
    for e in range(w1.shape[0]):
        tok, choice = np.nonzero(expert_ids == e)
        if tok.size == 0:
            continue
        gate_up = round_bf16(x[tok] @ w1[e].T)
        act = swiglu(gate_up, route_weights[tok, choice], clamp)
        eo = round_bf16(act @ w2[e].T)
        np.add.at(out, tok, eo)
    return round_bf16(out)


def _quant_dequant_rows(v: np.ndarray) -> np.ndarray:
    """NVFP4 round trip of every row (one scale per 16 values along the row); rows are independent,
    so they are padded to whole 128-row scale atoms and cut back."""
    from .nvfp4_oracle import dequantize, quantize
    rows = v.shape[0]
    pad = -(-rows // 128) * 128
    buf = np.zeros((pad, v.shape[1]), dtype=np.float32)
    buf[:rows] = v
    return dequantize(*quantize(buf))[:rows]


def moe_forward_nvfp4_experts(x, expert_ids, route_weights, dequantised_expert, clamp=10.0):
    """moe_forward_nvfp4 for layers too large to hold as FP32 arrays: `dequantised_expert(e)` returns the
    expert's (W1 [2I,H], W2 [H,I]) as FP32 values that are already NVFP4-representable (quantised and
    dequantised by the caller), and is asked only for the experts some route uses. Ids outside the range of
    experts the callable knows (it may raise KeyError) must not occur; ids < 0 are dropped routes and add
    nothing, as in the CUDA path."""
    tokens, hidden = x.shape
    topk = expert_ids.shape[1]
    xq = _quant_dequant_rows(x)
    slots = np.zeros((tokens, topk, hidden), dtype=np.float32)
    for e in np.unique(expert_ids):
        if e < 0:
            continue
        tok, choice = np.nonzero(expert_ids == e)
        w1q, w2q = dequantised_expert(int(e))
        gate_up = round_bf16(xq[tok] @ w1q.T)
        act = swiglu(gate_up, route_weights[tok, choice], clamp)
        slots[tok, choice] = round_bf16(_quant_dequant_rows(act) @ w2q.T)
    out = np.zeros((tokens, hidden), dtype=np.float32)
    for j in range(topk):
        out = (out + slots[:, j]).astype(np.float32)
    return round_bf16(out)


def moe_forward_nvfp4(x, expert_ids, route_weights, w1, w2, clamp=10.0):
    """The same layer with both GEMMs on NVFP4 operands: the FP32 dequantise-then-matmul statement of
    what the CUDA expert path computes. Tokens are quantised along H, each expert's W1 along H and W2
    along I, the activation (after its bf16 rounding) along I; every other rounding point is the
    reference's (moe.py:18-26). The per-token sum runs over the routes in slot order, as the
    reference's reduce kernel does (kernels/moe/fused/sm90.cu:125-133).
    """
    tokens, hidden = x.shape
    topk = expert_ids.shape[1]
    xq = _quant_dequant_rows(x)
    slots = np.zeros((tokens, topk, hidden), dtype=np.float32)
    for e in range(w1.shape[0]):
        tok, choice = np.nonzero(expert_ids == e)
        if tok.size == 0:
            continue
        w1q = _quant_dequant_rows(w1[e])
        w2q = _quant_dequant_rows(w2[e])
        gate_up = round_bf16(xq[tok] @ w1q.T)
        act = swiglu(gate_up, route_weights[tok, choice], clamp)
        slots[tok, choice] = round_bf16(_quant_dequant_rows(act) @ w2q.T)
    out = np.zeros((tokens, hidden), dtype=np.float32)
    for j in range(topk):
        out = (out + slots[:, j]).astype(np.float32)
    return round_bf16(out)
