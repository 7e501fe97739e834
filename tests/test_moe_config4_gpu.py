"""The expert layer at the benchmark's own shape (H=4096, I=2048, 256 experts, top-6, clamp 10) on one GPU.

The small-shape tests cover the arithmetic against the CPU oracle on every token; this file covers what only
the full shape has: K loops of 16 (FC1) and 8 (FC2) ring steps, 16 N tiles per pool block, 256 experts in the
routing plan, experts that span several blocks next to experts with no route at all. Weights are generated
expert by expert (N(0, 0.02), bf16) as the benchmark does.

Checks per case: (1) sampled tokens against the CPU oracle `moe_forward_nvfp4_experts` (a token's output
depends on its own routes only, so the oracle runs on the sampled tokens and their experts; the experts'
NVFP4 weights are dequantised by the library's dequantise kernel, which other tests prove bit-exact against
the oracle's); (2) every token against the same arithmetic restated in FP32 torch on the GPU.
"""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as MO
from helpers import to_np

pytestmark = pytest.mark.gpu

H, I, E, TOPK, CLAMP = 4096, 2048, 256, 6, 10.0
# same acceptance as the small-shape layer tests (relative Frobenius error, max abs error over output RMS)
LAYER_REL_FROBENIUS = 2e-2
LAYER_MAX_ABS_OVER_RMS = 0.25


@pytest.fixture(scope="module")
def g():
    import gpu_kernels_b200
    return gpu_kernels_b200


@pytest.fixture(scope="module")
def weights():
    gen = torch.Generator(device="cuda").manual_seed(4)
    w1 = torch.empty((E, 2 * I, H), dtype=torch.bfloat16, device="cuda")
    w2 = torch.empty((E, H, I), dtype=torch.bfloat16, device="cuda")
    for e in range(E):
        w1[e] = (torch.randn((2 * I, H), generator=gen, device="cuda") * 0.02).bfloat16()
        w2[e] = (torch.randn((H, I), generator=gen, device="cuda") * 0.02).bfloat16()
    return w1, w2


def dequantised_expert(g, layer, e):
    """(W1 [2I, H], W2 [H, I]) of local expert e as the layer holds them (NVFP4), FP32 on the GPU, W1 in
    gate-then-up row order."""
    r0 = e * 2 * I
    w1 = g.dequantize(layer.w1q[r0:r0 + 2 * I], layer.w1s[r0 * H // 16:(r0 + 2 * I) * H // 16])
    if layer.fused:                                         # stored as 16 gate rows, 16 up rows, ...
        w1 = w1.reshape(I // 16, 2, 16, H).permute(1, 0, 2, 3).reshape(2 * I, H)
    r0 = e * H
    w2 = g.dequantize(layer.w2q[r0:r0 + H], layer.w2s[r0 * I // 16:(r0 + H) * I // 16])
    return w1, w2


def round_bf16(t):
    return t.bfloat16().float()


def torch_layer(g, layer, x, ids, wts):
    """The oracle's arithmetic in FP32 torch on the GPU (TF32 off), expert by expert, for every token."""
    tokens = x.shape[0]
    pad = -(-tokens // 128) * 128
    xp = torch.zeros((pad, H), dtype=torch.bfloat16, device="cuda")
    xp[:tokens] = x
    xq = g.dequantize(*g.quantize(xp))[:tokens]
    slots = torch.zeros((tokens, TOPK, H), dtype=torch.float32, device="cuda")
    for e in torch.unique(ids).tolist():
        tok, choice = torch.nonzero(ids == e, as_tuple=True)
        w1, w2 = dequantised_expert(g, layer, e)
        gate_up = round_bf16(xq[tok] @ w1.T)
        gate = torch.minimum(gate_up[:, :I], torch.tensor(CLAMP, device="cuda"))
        up = gate_up[:, I:].clamp(-CLAMP, CLAMP)
        act = round_bf16(gate / (1.0 + torch.exp(-gate)) * up * wts[tok, choice][:, None])
        rows = act.shape[0]
        ap = torch.zeros((-(-rows // 128) * 128, I), dtype=torch.bfloat16, device="cuda")
        ap[:rows] = act.bfloat16()
        aq = g.dequantize(*g.quantize(ap))[:rows]
        slots[tok, choice] = round_bf16(aq @ w2.T)
    out = torch.zeros((tokens, H), dtype=torch.float32, device="cuda")
    for j in range(TOPK):
        out = out + slots[:, j]
    return round_bf16(out)


def errors(y, ref):
    y, ref = np.asarray(y, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    rel = np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-30)
    worst = np.abs(y - ref).max() / max(np.sqrt((ref ** 2).mean()), 1e-30)
    return rel, worst


def routing(g, tokens, seed, skew):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((tokens, H), generator=gen, device="cuda").bfloat16()
    logits = torch.randn((tokens, E), generator=gen, device="cuda")
    if skew:
        logits[:, 5] += 9.0                                  # every token picks expert 5: two 128-row blocks
        logits[:, 200] += 6.0                                # most pick expert 200 too
        logits[:, 64:128] -= 30.0                            # a quarter of the experts get no route at all
    ids, wts = g.route(logits, TOPK)
    return x, ids, wts


# tokens, skewed routing, fused FC1 epilogue, rows per pool block (None: chosen per call)
CASES = [
    (1, False, True, None),
    (64, False, True, None),
    (64, False, False, 128),
    (200, True, True, 128),
    (200, True, True, 256),
    (200, True, False, 256),
]


@pytest.mark.parametrize("tokens,skew,fused,block_rows", CASES)
def test_benchmark_shape_against_oracle(g, weights, tokens, skew, fused, block_rows):
    torch.backends.cuda.matmul.allow_tf32 = False
    w1, w2 = weights
    x, ids, wts = routing(g, tokens, 1000 + tokens, skew)
    layer = g.Nvfp4MoE(w1, w2, E, TOPK, clamp=CLAMP, max_tokens=256, fused=fused, block_rows=block_rows)
    try:
        y = layer(x, ids, wts).clone()
        torch.cuda.synchronize()
        layer.check()
        got = to_np(y.float())
        assert not np.isnan(got).any()
        what = f"T={tokens} skew={skew} fused={fused} block_rows={block_rows}"

        # (2) every token against the FP32 torch restatement
        rel, worst = errors(got, to_np(torch_layer(g, layer, x, ids, wts)))
        assert rel <= LAYER_REL_FROBENIUS and worst <= LAYER_MAX_ABS_OVER_RMS, f"{what}: all tokens rel {rel:.3e} worst {worst:.3e}"

        # (1) sampled tokens against the CPU oracle
        sample = sorted(set([0, tokens // 2, tokens - 1] + ([7, 130] if tokens >= 200 else [])))
        ids_np, wts_np = to_np(ids)[sample], to_np(wts)[sample]
        cache = {}

        def expert(e):
            if e not in cache:
                a, b = dequantised_expert(g, layer, e)
                cache[e] = (to_np(a), to_np(b))
            return cache[e]

        ref = MO.moe_forward_nvfp4_experts(to_np(x.float())[sample], ids_np, wts_np, expert, CLAMP)
        rel_s, worst_s = errors(got[sample], ref)
        print(f"{what}: all tokens rel {rel:.2e} worst/rms {worst:.2e}; sampled vs CPU oracle rel {rel_s:.2e} worst/rms {worst_s:.2e}")
        assert rel_s <= LAYER_REL_FROBENIUS and worst_s <= LAYER_MAX_ABS_OVER_RMS, f"{what}: sampled tokens rel {rel_s:.3e} worst {worst_s:.3e}"

        # a second call with other inputs through the same object: nothing stale survives
        x2, ids2, wts2 = routing(g, tokens, 2000 + tokens, not skew)
        y2 = layer(x2, ids2, wts2).clone()
        torch.cuda.synchronize()
        rel2, worst2 = errors(to_np(y2.float()), to_np(torch_layer(g, layer, x2, ids2, wts2)))
        assert rel2 <= LAYER_REL_FROBENIUS and worst2 <= LAYER_MAX_ABS_OVER_RMS, f"{what}: second call rel {rel2:.3e} worst {worst2:.3e}"
        layer.check()
    finally:
        layer.close()
