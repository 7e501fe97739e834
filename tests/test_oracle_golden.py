"""The CPU oracle against the reference's known-answer tests and frozen reference outputs.

The first three tests restate tests/test_nvfp4.py:11-35 of the reference against
the oracle; the rest compare the oracle bit-for-bit with outputs of the
reference Python stored under tests/golden/.
"""
import numpy as np

from oracle import nvfp4_oracle as O
from oracle import moe_oracle as MO


def test_e2m1_values_and_even_ties():
    values = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -.5, -6], dtype=np.float32)
    assert O.encode_e2m1(values).tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 9, 15]
    mids = np.array([.25, .75, 1.25, 1.75, 2.5, 3.5, 5, 100], dtype=np.float32)
    assert O.encode_e2m1(mids).tolist() == [0, 2, 2, 4, 4, 6, 6, 7]


def test_scale_addresses(golden):
    rows, k = 256, 128
    raw = (np.arange(rows * k // 16) % 126).astype(np.uint8).reshape(rows, k // 16)
    packed = O.pack_scales(raw)
    for row in (0, 1, 31, 32, 127, 128, 255):
        for block in range(k // 16):
            offset = ((row // 128) * (k // 64) + block // 4) * 512
            offset += (row % 32) * 16 + ((row % 128) // 32) * 4 + block % 4
            assert packed[offset] == raw[row, block]
            assert O.scale_offset(row, block, k) == offset
    assert np.array_equal(O.unpack_scales_u8(packed, rows, k), raw)
    g = golden("scale_layout.npz")
    assert np.array_equal(g["raw"], raw) and np.array_equal(g["packed"], packed)


def test_packing_round_trip():
    values = np.tile(np.array([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32), (128, 4))
    packed, scales = O.quantize(values)
    assert packed[0, :8].tolist() == [0x10, 0x32, 0x54, 0x76, 0x90, 0xBA, 0xDC, 0xFE]
    assert np.array_equal(O.dequantize(packed, scales), values)


def test_cfg0_bit_exact(golden):
    g = golden("cfg0_256.npz")
    for name in ("a", "b"):
        packed, scales = O.quantize(O.bf16_to_f32(g[f"{name}_bf16"]))
        assert np.array_equal(packed, g[f"{name}_packed"])
        assert np.array_equal(scales, g[f"{name}_scales"])
    assert np.array_equal(O.dequantize(g["a_packed"], g["a_scales"]), g["a_dequant"])
    c = O.gemm_f32(g["a_packed"], g["a_scales"], g["b_packed"], g["b_scales"])
    ref = g["c_f32"]
    # summation order differs between BLAS builds: floating-point tolerance, stated here
    assert np.linalg.norm(c - ref) <= 1e-6 * np.linalg.norm(ref)
    c16 = O.gemm(g["a_packed"], g["a_scales"], g["b_packed"], g["b_scales"])
    ref16 = g["c_f16"].view(np.float16)
    assert np.mean(c16.view(np.uint16) == g["c_f16"]) > 0.999
    assert np.abs(c16.astype(np.float32) - ref16.astype(np.float32)).max() <= 2 ** -4  # one FP16 ulp at |c| < 128


def test_distributions_bit_exact(golden):
    g = golden("dists.npz")
    packed, scales = O.quantize(O.bf16_to_f32(g["w_bf16"]))
    assert np.array_equal(packed, g["w_packed"]) and np.array_equal(scales, g["w_scales"])
    packed, scales = O.quantize(g["f_f32"])
    assert np.array_equal(packed, g["f_packed"]) and np.array_equal(scales, g["f_scales"])


def test_adversarial_bit_exact(golden):
    g = golden("adversarial.npz")
    packed, scales = O.quantize(g["x_f32"])
    assert np.array_equal(scales, g["scales"])
    assert np.array_equal(packed, g["packed"])
    d = O.dequantize(packed, scales)
    assert np.array_equal(np.isnan(d), np.isnan(g["dequant"]))
    assert np.array_equal(np.nan_to_num(d, nan=0.0), np.nan_to_num(g["dequant"], nan=0.0))
    # landmarks of the specification
    s = O.unpack_scales_u8(scales, 128, 256)
    assert (s[0] == 0x01).all()          # all-zero block: scale 2**-9, never 0
    assert (s[1] == 0x7E).all()          # amax/6 > 448 saturates
    assert (packed[0] == 0).all()
    # -0.0 keeps code 0 while a tiny negative that rounds to zero carries the sign bit
    codes8 = np.stack((packed[8] & 15, packed[8] >> 4), -1).reshape(-1)
    assert codes8[0] == 0 and codes8[5] == 8


def test_e4m3_round_trip_all_codes():
    codes = np.arange(1, 0x7F, dtype=np.uint8)
    assert np.array_equal(O.f32_to_ue4m3(O.ue4m3_to_f32(codes)), codes)
    # ties go to the even mantissa
    assert O.f32_to_ue4m3(np.array([1.0625, 1.1875], dtype=np.float32)).tolist() == [0x38, 0x3A]


def test_moe_oracle_matches_reference_output(golden):
    g = golden("moe_bf16.npz")
    f = O.bf16_to_f32
    y = MO.moe_forward(f(g["x_bf16"]), g["ids"], g["weights"], f(g["w1_bf16"]), f(g["w2_bf16"]), clamp=10.0)
    ref = f(g["y_bf16"])
    # floating point with BF16 rounding points: allow one BF16 ulp on a few elements
    assert np.mean(y == ref) > 0.99
    assert np.abs(y - ref).max() <= 2 ** -7 * np.abs(ref).max()


def test_expert_streaming_oracle_matches_the_whole_layer_oracle():
    # moe_forward_nvfp4_experts (weights handed over expert by expert, already NVFP4-representable) is the
    # same arithmetic as moe_forward_nvfp4; a route with a negative id is dropped
    from oracle import moe_oracle as MO
    rng = np.random.default_rng(0)
    tokens, hidden, inter, experts, topk = 9, 64, 64, 4, 2
    x = MO.round_bf16(rng.standard_normal((tokens, hidden)).astype(np.float32))
    w1 = MO.round_bf16((rng.standard_normal((experts, 2 * inter, hidden)) * 0.1).astype(np.float32))
    w2 = MO.round_bf16((rng.standard_normal((experts, hidden, inter)) * 0.1).astype(np.float32))
    ids = np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)])
    wts = rng.random((tokens, topk)).astype(np.float32)
    pick = lambda e: (MO._quant_dequant_rows(w1[e]), MO._quant_dequant_rows(w2[e]))
    whole = MO.moe_forward_nvfp4(x, ids, wts, w1, w2)
    assert np.array_equal(whole, MO.moe_forward_nvfp4_experts(x, ids, wts, pick))
    dropped = ids.copy()
    dropped[2, 1] = -1
    zero_weight = wts.copy()
    zero_weight[2, 1] = 0.0
    assert np.array_equal(MO.moe_forward_nvfp4_experts(x, dropped, wts, pick),
                          MO.moe_forward_nvfp4(x, ids, zero_weight, w1, w2))


def test_mxfp4_oracle_round_trip_and_known_answers():
    # no reference fixture exists for MXFP4 (the reference has none): known answers from the format's definition
    x = np.zeros((128, 128), dtype=np.float32)
    x[0, :8] = [6.0, -6.0, 3.0, 0.5, 0.25, 0.75, -0.2, 7.0]            # amax 7: e = floor(log2 7) - 2 = 0
    x[1, :4] = [1.0, 0.1, -0.6, 0.3]                                    # amax 1: e = -2, steps of 0.125
    x[2, 32:36] = [2.0 ** 20, 3 * 2.0 ** 18, 0, 0]                      # e = 18
    x[3, 0] = np.inf
    packed, scales = O.quantize_mx(x)
    u = O.unpack_scales_u8(scales, 128, 64)
    assert [u[0, 0], u[1, 0], u[2, 1], u[3, 0], u[4, 0]] == [127, 125, 145, 255, 0]
    codes = np.stack((packed & 15, packed >> 4), axis=-1).reshape(128, 128)
    assert codes[0, :8].tolist() == [7, 15, 5, 1, 0, 2, 8, 7]          # ties to the even code; -0.2 keeps its sign
    assert codes[1, :4].tolist() == [6, 1, 12, 2]                       # 4.0, 0.4 -> 0.5, -2.4 -> -2, 1.2 -> 1.0
    assert codes[2, 32:34].tolist() == [6, 5] and (codes[3, :32] == 7).all()
    back = O.dequantize_mx(packed, scales)
    assert back[0, :8].tolist() == [6.0, -6.0, 3.0, 0.5, 0.0, 1.0, -0.0, 6.0]
    assert back[2, 32] == 2.0 ** 20 and back[2, 33] == 3 * 2.0 ** 18 and np.isnan(back[3, :32]).all()
    # idempotence: what the format can hold survives a second pass bit for bit
    rng = np.random.default_rng(3)
    y = (rng.standard_normal((256, 384)) * np.exp2(rng.integers(-20, 20, (256, 1)))).astype(np.float32)
    p1, s1 = O.quantize_mx(y)
    p2, s2 = O.quantize_mx(O.dequantize_mx(p1, s1))
    d1, d2 = O.dequantize_mx(p1, s1), O.dequantize_mx(p2, s2)
    assert np.array_equal(d1, d2)
