"""Regenerate the golden fixtures in this directory from the reference's own Python.

Run in a checkout that has the reference repository mounted:

    python tests/golden/make_golden.py /path/to/gpu-kernels

It imports `reference.python.nvfp4` (and `reference.python.moe`) from that
path, feeds them seeded inputs, and freezes inputs and outputs as compressed
.npz files. The fixtures are what the tests use; the reference itself is not
needed to run the tests.
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def adversarial_input():
    """128 x 256 FP32 values aimed at every rounding rule of the quantiser."""
    rng = np.random.default_rng(1234)
    x = (rng.standard_normal((128, 256)).astype(np.float32))
    mids = np.array([.25, .75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    ladder = np.concatenate(([6.0], mids, -mids, [-6.0])).astype(np.float32)          # 16 values, amax 6
    x[0, :] = 0.0                                                                       # all-zero blocks
    x[1, :] = 1e-3; x[1, ::16] = 1e6                                                   # scale saturates at 448
    for i, s in enumerate((1.0, 0.125, 1.5, 0.0625 * 1.25, 448.0, 2.0 ** -9)):          # exact midpoints x scales
        x[2 + i, :] = np.tile(ladder * np.float32(s), 16)
    x[8, :] = -0.0; x[8, 5::16] = -1e-30; x[8, 7::16] = 1.0                             # -0.0 vs tiny negatives
    sub = (np.arange(256, dtype=np.uint32) % 127 + 1).astype(np.uint32) << 16          # bf16 subnormals
    x[9, :] = sub.view(np.float32) * np.where(np.arange(256) % 2, -1, 1)
    x[10, :] = 1.0; x[10, 3::32] = np.inf; x[10, 19::32] = -np.inf                      # infinities
    x[11, :] = 2.0; x[11, 8::64] = np.nan                                               # NaN in every fourth block
    x[12, :] = np.float32(3.4e38) * np.where(np.arange(256) % 3, 1, -1)                 # near FP32 max
    x[13, :] = np.float32(2.0 ** -9 * 6) * np.tile(ladder / 6, 16)                      # amax/6 == 2**-9 exactly
    x[14, :] = np.float32(2.0 ** -9 * 3) * np.tile(ladder / 6, 16)                      # amax/6 below the clamp
    x[15, :] = np.tile((ladder * np.float32(1.0625)), 16)                               # scale tie 1.0625 -> 1.0
    x[16, :] = np.tile((ladder * np.float32(1.1875)), 16)                               # scale tie 1.1875 -> 1.25
    x[17, :] = np.tile((ladder * np.float32(2.0 ** -7 * 1.25)), 16)                     # scale in the E4M3 subnormals
    for r in range(18, 64):                                                             # wide dynamic range, FP32 mantissas
        x[r, :] *= np.float32(10.0 ** rng.uniform(-6, 6))
    return x


def main(ref_root):
    sys.path.insert(0, ref_root)
    from reference.python import nvfp4 as R
    from reference.python import moe as RM
    manifest = {}

    def save(name, **arrays):
        np.savez_compressed(HERE / name, **arrays)
        manifest[name] = {k: hashlib.sha256(np.ascontiguousarray(v).tobytes()).hexdigest()[:16]
                          for k, v in arrays.items()}

    # Config 0 of the benchmark: M=N=K=256, bf16 N(0,1) from seed 0 (A then B), global scale 1.
    torch.manual_seed(0)
    a = torch.randn(256, 256, dtype=torch.bfloat16)
    b = torch.randn(256, 256, dtype=torch.bfloat16)
    pa, sa = R.quantize(a)
    pb, sb = R.quantize(b)
    c32 = R.dequantize(pa, sa) @ R.dequantize(pb, sb).T
    save("cfg0_256.npz", a_bf16=bf16_bits(a), b_bf16=bf16_bits(b),
         a_packed=pa.numpy(), a_scales=sa.numpy(), b_packed=pb.numpy(), b_scales=sb.numpy(),
         a_dequant=R.dequantize(pa, sa).numpy(), c_f16=c32.half().numpy().view(np.uint16), c_f32=c32.numpy())

    # Weight-like distribution N(0, 0.02) in bf16, and the reference test recipe (fp32 randn * 0.1).
    torch.manual_seed(1)
    w = (torch.randn(128, 512) * 0.02).bfloat16()
    pw, sw = R.quantize(w)
    torch.manual_seed(2026 + 256 * 3)
    f = torch.randn(256, 256) * .1
    pf, sf = R.quantize(f)
    save("dists.npz", w_bf16=bf16_bits(w), w_packed=pw.numpy(), w_scales=sw.numpy(),
         f_f32=f.numpy(), f_packed=pf.numpy(), f_scales=sf.numpy())

    # Adversarial values.
    x = adversarial_input()
    px, sx = R.quantize(torch.from_numpy(x))
    save("adversarial.npz", x_f32=x, packed=px.numpy(), scales=sx.numpy(),
         dequant=R.dequantize(px, sx).numpy())

    # Scale-address permutation of the reference's own test (tests/test_nvfp4.py:17-23).
    raw = (torch.arange(256 * 128 // 16) % 126).to(torch.uint8).reshape(256, 128 // 16)
    save("scale_layout.npz", raw=raw.numpy(), packed=R.pack_scales(raw.view(torch.float8_e4m3fn)).numpy())

    # Routed-MoE oracle (reference/python/moe.py) on NVFP4-dequantised weights, small shape.
    torch.manual_seed(7)
    T, H, I, E, topk = 24, 256, 128, 8, 2
    xm = torch.randn(T, H, dtype=torch.bfloat16)
    logits = torch.randn(T, E)
    prob = torch.softmax(logits, -1)
    wts, ids = prob.topk(topk, dim=-1)
    wts = wts / wts.sum(-1, keepdim=True)
    w1 = (torch.randn(E, 2 * I, H) * 0.02).bfloat16()
    w2 = (torch.randn(E, H, I) * 0.02).bfloat16()
    y = RM.moe_forward(xm, ids, wts, w1, w2, clamp=10.0)
    save("moe_bf16.npz", x_bf16=bf16_bits(xm), ids=ids.numpy(), weights=wts.numpy(),
         w1_bf16=bf16_bits(w1), w2_bf16=bf16_bits(w2), y_bf16=bf16_bits(y))

    (HERE / "MANIFEST.json").write_text(json.dumps(manifest, indent=1) + "\n")
    print(json.dumps(manifest, indent=1))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/gpu-kernels")
    main(sys.argv[1])
